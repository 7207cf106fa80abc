// Prefill and vision attention on the fifth-generation tensor cores (bf16 Q/K/V rows, head
// dimension 128, or 72 padded to 80 with zero columns that the TMA unit fills in).
//
// One CTA handles 128 query rows of one (sequence, query head) and walks the keys in tiles of
// 64.  Warp 0 streams K/V tiles with TMA (128-byte swizzle) into a two-stage ring, one thread
// of warp 1 issues the MMAs, warps 2-9 are the softmax: two threads per query row, each with
// half of a tile's keys and half of the output columns.
//
//   S  = Q K^T      tcgen05.mma, A = Q (shared, K-major), B = K tile (shared, K-major),
//                   fp32 accumulator in TMEM, two S buffers so tile j+1 is scored while the
//                   softmax of tile j runs
//   P  = exp2(S - m) as bf16 pairs, written over the S buffer with tcgen05.st
//   O += P V        tcgen05.mma with the A operand read from TMEM and B = V tile as loaded
//                   (keys are its K index, so it is an MN-major operand), accumulating in TMEM
//
// TMEM columns: S/P buffers 2 x 64, O accumulator 128 (256 allocated).  Every wait is bounded
// (common.cuh: mbar_wait); on a timeout the status word is set, roles unwind and the CTA
// frees its TMEM.  Replaces the reference's flash-attn / SDPA calls for prefill without
// history (prism_infer/layers/attention.py:180-250).
//
// Prefill over the paged cache (chunked prefill, prefix hits; reference
// prism_infer/ops/paged_attention_reference.py:185-390): the keys a step can see are first
// gathered from their pages into contiguous bf16 rows (gather_pages_kernel: E4M3 payload times
// the row scale, or a plain copy of bf16 pages), once per layer and KV head, and the same
// tensor-core kernel then runs with its own key ranges (cu_kv): query row r of a sequence sees
// keys 0 .. kv_len - q_len + r.  A key is dequantised once instead of once per query tile and
// query head of its group, and the gathered rows (a few MB) stay in L2 for the TMA loads.
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(attn_tc)

namespace {

constexpr int FA_BM = 128;
constexpr int FA_BN = 64;
constexpr int FA_HD = 128;
constexpr int FA_STAGES = 2;  // 32 KB each; with Q that is 96 KB, so two CTAs share an SM
constexpr int FA_THREADS = 320;  // TMA warp, MMA warp, eight softmax warps
constexpr int Q_BYTES = FA_BM * FA_HD * 2;      // two 64-column atoms of 128 rows
constexpr int K_BYTES = FA_BN * FA_HD * 2;      // two 64-column atoms of 64 rows
constexpr int V_BYTES = FA_BN * FA_HD * 2;      // two 64-column boxes of 64 keys
constexpr int STAGE_BYTES = K_BYTES + V_BYTES;  // 32 KB
constexpr int TMEM_S = 0;                       // S/P buffer b at column b * 64
constexpr int TMEM_O = 128;                     // O accumulator, 128 columns

struct FaArgs {
  const int* cu_q;        // [S + 1] row offsets of the sequences
  const int* cu_kv;       // [S + 1] row offsets of the sequences' keys in K / V; null: the query rows' own
  __nv_bfloat16* out;     // [T][Hq * hd]
  long long o_stride;
  int Hq, Hkv;
  int hd;                 // real head dimension (<= HD_PAD)
  int causal;
  float scale;
};

__device__ __forceinline__ void named_bar(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Named barrier that also returns the OR of a predicate over the participating threads.
__device__ __forceinline__ bool named_bar_or(int id, int threads, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %3, 0;\n\t"
      "barrier.cta.red.or.pred q, %1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(id), "r"(threads), "r"((uint32_t)pred)
      : "memory");
  return out != 0;
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// HD_PAD: head dimension rounded up to a multiple of 16 (the K extent of Q K^T and the N extent
// of P V).  Shared-memory tiles always have two 64-column atoms; with HD_PAD = 80 the second
// atom holds 8 real columns and zeros.
template <int HD_PAD>
__global__ void __launch_bounds__(FA_THREADS, 2)
flash_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FaArgs a) {
  extern __shared__ uint8_t fa_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* ring = smem + Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + FA_STAGES * STAGE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                  // [FA_STAGES]
  uint64_t* kv_empty = kv_full + FA_STAGES;      // [FA_STAGES]
  uint64_t* s_full = kv_empty + FA_STAGES;       // [2] MMA -> softmax: S tile ready
  uint64_t* p_full = s_full + 2;                 // [2] softmax -> MMA: P written (256 arrivals)
  uint64_t* pv_done = p_full + 2;                // [2] MMA -> softmax: P V of tile j accumulated (slot j % 2)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  float* mx_s = reinterpret_cast<float*>(tmem_slot + 4);  // [2 buffers][2 halves][128 rows] maxima, then [2 halves][128 rows] sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // late query tiles see the most keys under a causal mask: schedule them first
  const int seq = blockIdx.z, head = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;
  const int kvh = head / (a.Hq / a.Hkv);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 256);
      mbar_init(&pv_done[b], 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  const int q_start = a.cu_q[seq];
  const int q_len = a.cu_q[seq + 1] - q_start;
  const int kv_start = a.cu_kv ? a.cu_kv[seq] : q_start;
  const int kv_len = a.cu_kv ? max(a.cu_kv[seq + 1] - kv_start, q_len) : q_len;
  const int pos_off = kv_len - q_len;  // key position of the sequence's first query row
  const int q0 = qt * FA_BM;
  const bool live = q0 < q_len;  // uniform over the CTA
  int n_tiles = 0;
  if (live) {
    int kv_end = kv_len;
    if (a.causal) kv_end = min(kv_len, pos_off + q0 + FA_BM);
    n_tiles = (kv_end + FA_BN - 1) / FA_BN;
  }

  if (warp == 0) {
    if (lane == 0 && live) {
      // ------------------------------ TMA producer ------------------------------
      mbar_expect_tx(q_full, Q_BYTES);
      tma_load_3d(q_s, &tmQ, q_full, 0, head, q_start + q0);
      tma_load_3d(q_s + Q_BYTES / 2, &tmQ, q_full, 64, head, q_start + q0);
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % FA_STAGES;
        if (j >= FA_STAGES) {
          ok = mbar_wait(&kv_empty[s], ((j / FA_STAGES) - 1) & 1, 11);
          if (!ok) break;
        }
        uint8_t* st = ring + (size_t)s * STAGE_BYTES;
        const int row = kv_start + j * FA_BN;
        mbar_expect_tx(&kv_full[s], STAGE_BYTES);
        tma_load_3d(st, &tmK, &kv_full[s], 0, kvh, row);
        tma_load_3d(st + K_BYTES / 2, &tmK, &kv_full[s], 64, kvh, row);
        tma_load_3d(st + K_BYTES, &tmV, &kv_full[s], 0, kvh, row);
        tma_load_3d(st + K_BYTES + V_BYTES / 2, &tmV, &kv_full[s], 64, kvh, row);
        issued = j + 1;
      }
      if (!ok) {
        for (int j = max(0, issued - FA_STAGES); j < issued; ++j)
          (void)mbar_wait(&kv_full[j % FA_STAGES], (j / FA_STAGES) & 1, 12);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && live) {
      // ------------------------------ MMA issuer ------------------------------
      constexpr uint32_t IDESC_S = umma_idesc_bf16(FA_BM, FA_BN);
      constexpr uint32_t IDESC_O = umma_idesc_bf16(FA_BM, HD_PAD) | UMMA_B_MN_MAJOR;
      const uint32_t q_addr = smem_u32(q_s);
      bool ok = mbar_wait(q_full, 0, 13);
      auto score = [&](int j) {  // S[j % 2] = Q K_j^T
        const uint32_t st = smem_u32(ring + (size_t)(j % FA_STAGES) * STAGE_BYTES);
        const uint32_t d = tmem_base + TMEM_S + (j & 1) * FA_BN;
#pragma unroll
        for (int k = 0; k < HD_PAD / 16; ++k) {
          const uint64_t da = umma_desc_sw128(q_addr + (k >> 2) * (Q_BYTES / 2)) + 2 * (k & 3);
          const uint64_t db = umma_desc_sw128(st + (k >> 2) * (K_BYTES / 2)) + 2 * (k & 3);
          tc_mma_f16(d, da, db, IDESC_S, k != 0);
        }
        tc_commit(&s_full[j & 1]);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, 14);
      if (ok) {
        tc_fence_after();
        score(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = j & 1;
        if (j + 1 < n_tiles) {
          ok = mbar_wait(&kv_full[(j + 1) % FA_STAGES], ((j + 1) / FA_STAGES) & 1, 15);
          if (!ok) break;
          tc_fence_after();
          score(j + 1);  // overwrites S/P[(j+1) & 1]: PV(j-1) was issued before, so it reads first
        }
        ok = mbar_wait(&p_full[b], (j >> 1) & 1, 16);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vt = smem_u32(ring + (size_t)(j % FA_STAGES) * STAGE_BYTES + K_BYTES);
        const uint32_t d = tmem_base + TMEM_O;
        const uint32_t p_t = tmem_base + TMEM_S + b * FA_BN;
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          // 16 keys per step: 8 packed columns of P, two 8-key groups (2048 bytes) of V
          const uint64_t db = umma_desc_sw128_mn(vt + k * 2048, V_BYTES / 2);
          tc_mma_f16_ts(d, p_t + k * 8, db, IDESC_O, (j | k) != 0);
        }
        tc_commit(&pv_done[b]);
        tc_commit(&kv_empty[j % FA_STAGES]);
      }
    }
  } else if (live) {
    // ------------------------------ softmax warps 2..9 ------------------------------
    // Two threads per query row: warps 2-5 take keys 0-31 of a tile and output columns 0-63,
    // warps 6-9 keys 32-63 and columns 64-127.  The pair agrees on the tile's row maximum
    // through shared memory (one named barrier per tile); each keeps the sum of its own keys.
    //
    // P is scaled by a per-row reference maximum that is only raised when a tile exceeds it
    // by more than 2^8 (P then stays below 256).  Raising it means multiplying the row of
    // the O accumulator in TMEM, which needs the previous P V product to have finished, so
    // the whole CTA takes that path together (the barrier carries an OR over all rows).  It
    // is rare after the first tiles.
    const int q = warp & 3;                 // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;
    const int r_local = q * 32 + lane;      // row inside the tile
    const int row = q0 + r_local;           // query row (local index of the sequence)
    const int last_key = pos_off + row;     // last key position this row sees under the causal mask
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const float sl2 = a.scale * 1.4426950408889634f;
    constexpr int HC = FA_BN / 2;           // keys per thread and tile
    constexpr int HO = 64;                  // first output column of the second thread of a pair
    constexpr int CHUNKS = HD_PAD / 16;     // 16-column chunks of the accumulator
    const int c_begin = half * 4, c_end = half ? CHUNKS : (CHUNKS < 4 ? CHUNKS : 4);  // this thread's chunks
    constexpr float RAISE = 8.0f;
    float m_ref = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      float s[HC];
      float mx = -INFINITY;
      const int j0 = j * FA_BN + half * HC;
      if (ok) ok = mbar_wait(&s_full[b], (j >> 1) & 1, 19);
      ok = __all_sync(0xffffffffu, ok);  // the TMEM accesses below are warp-wide
      if (ok) {
        tc_fence_after();
        uint32_t r[HC];
        {
          uint32_t(&r0)[16] = *reinterpret_cast<uint32_t(*)[16]>(&r[0]);
          uint32_t(&r1)[16] = *reinterpret_cast<uint32_t(*)[16]>(&r[16]);
          tmem_ld16(lane_addr + TMEM_S + b * FA_BN + half * HC, r0);
          tmem_ld16(lane_addr + TMEM_S + b * FA_BN + half * HC + 16, r1);
          tmem_ld_wait();
        }
#pragma unroll
        for (int i = 0; i < HC; ++i) s[i] = __uint_as_float(r[i]) * sl2;
        if (j0 + HC > kv_len || (a.causal && j0 + HC - 1 > last_key)) {
#pragma unroll
          for (int i = 0; i < HC; ++i)
            if (j0 + i >= kv_len || (a.causal && j0 + i > last_key)) s[i] = -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < HC; ++i) mx = fmaxf(mx, s[i]);
      }
      // pair maximum, and an OR over the CTA of "some row must raise its reference"
      mx_s[(b * 2 + half) * FA_BM + r_local] = mx;
      const bool raise_local = ok && j > 0 && mx > m_ref + RAISE;
      const bool raise_any = named_bar_or(1, 256, raise_local);
      if (!ok) continue;
      mx = fmaxf(mx, mx_s[(b * 2 + (half ^ 1)) * FA_BM + r_local]);
      if (j == 0) {
        m_ref = mx;  // nothing accumulated yet
      } else if (raise_any) {
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[b ^ 1], ((j - 1) >> 1) & 1, 20));  // P V of tile j-1 accumulated
        if (!ok) continue;
        tc_fence_after();
        // tcgen05.ld / st are warp-wide (.sync.aligned): every lane takes this path, rows that
        // keep their reference multiply by one
        float f = 1.0f;
        if (mx > m_ref + RAISE) {
          f = (m_ref == -INFINITY) ? 0.0f : ex2f(m_ref - mx);
          m_ref = mx;
          l_run *= f;
        }
#pragma unroll
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[16];
          tmem_ld16(lane_addr + TMEM_O + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
          tmem_st16(lane_addr + TMEM_O + c * 16, r);
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
      float sum = 0.0f;
      uint32_t packed[HC / 2];
#pragma unroll
      for (int i = 0; i < HC; i += 2) {
        const float p0 = ex2f(s[i] - m_use), p1 = ex2f(s[i + 1] - m_use);
        sum += p0 + p1;
        __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
      }
      l_run += sum;
      tmem_st16(lane_addr + TMEM_S + b * FA_BN + half * (HC / 2), packed);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[b]);
    }
    // the pair's row sum, then the finished accumulator
    mx_s[(4 + half) * FA_BM + r_local] = l_run;  // own region: the maxima slots may still be read
    named_bar(1, 256);
    l_run += mx_s[(4 + (half ^ 1)) * FA_BM + r_local];
    if (ok && n_tiles > 0) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, 21);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {  // whole warps read TMEM; only rows inside the sequence are stored
      tc_fence_after();
      const bool store = row < q_len;
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      __nv_bfloat16* dst = a.out + (size_t)(q_start + row) * a.o_stride + (size_t)head * a.hd;
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t r[16];
        tmem_ld16(lane_addr + TMEM_O + c * 16, r);
        tmem_ld_wait();
        uint4 v[2];
        uint32_t* w = reinterpret_cast<uint32_t*>(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * e]) * inv, __uint_as_float(r[2 * e + 1]) * inv);
          w[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        if (store) {  // the head dimension is a multiple of 8: whole 16-byte pieces or nothing
          if (c * 16 + 8 <= a.hd) *reinterpret_cast<uint4*>(dst + c * 16) = v[0];
          if (c * 16 + 16 <= a.hd) *reinterpret_cast<uint4*>(dst + c * 16 + 8) = v[1];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

// ---------------------------------------------------------------------------------------------
// Pages -> contiguous bf16 key / value rows.  Cache layout: payload [blocks][Hkv][page][D]
// (E4M3 bytes or bf16), scales [blocks][Hkv][page] (null: unit scale).  One warp per key row,
// looping over the KV heads; lane l converts elements 4l .. 4l+3 of K and of V.  A hole in the
// page table or a page id beyond the cache gives zero rows (the latter is also recorded in the
// status word), a key range that the table cannot describe is cut short and recorded.
// ---------------------------------------------------------------------------------------------
struct GatherArgs {
  const void* k_cache;
  const void* v_cache;
  const float* k_scale;
  const float* v_scale;
  const int* block_tables;  // [S][max_blocks]
  const int* cu_kv;         // [S + 1]
  __nv_bfloat16* k_out;     // [Tkv][Hkv * 128]
  __nv_bfloat16* v_out;
  int max_blocks, num_blocks, page, Hkv, Tkv;
};

constexpr int GATHER_ROWS = 8;  // key rows (warps) per CTA

__device__ __forceinline__ uint2 e4m3x4_to_bf16x4(uint32_t bytes, float scale) {
  const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(bytes & 0xffffu), __NV_E4M3);
  const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(bytes >> 16), __NV_E4M3);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  __nv_bfloat162 p = __floats2bfloat162_rn(a.x * scale, a.y * scale);
  __nv_bfloat162 q = __floats2bfloat162_rn(b.x * scale, b.y * scale);
  return make_uint2(*reinterpret_cast<uint32_t*>(&p), *reinterpret_cast<uint32_t*>(&q));
}

template <bool KV8>
__global__ void __launch_bounds__(GATHER_ROWS * 32) gather_pages_kernel(const GatherArgs a) {
  const int seq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();
  const int kv_start = a.cu_kv[seq];
  int kv_len = a.cu_kv[seq + 1] - kv_start;
  const long long reach = (long long)a.max_blocks * a.page;
  if ((long long)kv_len > reach) {
    if (threadIdx.x == 0 && blockIdx.x == 0) prism_report(PRISM_ERR_BOUNDS, 1);
    kv_len = (int)reach;
  }
  const int j = blockIdx.x * GATHER_ROWS + warp;
  if (j >= kv_len) return;
  const long long dst_row = (long long)kv_start + j;
  if (dst_row < 0 || dst_row >= a.Tkv) {  // offsets that do not fit the output: record, write nothing
    if (lane == 0) prism_report(PRISM_ERR_BOUNDS, 3);
    return;
  }
  int blk = a.block_tables[(size_t)seq * a.max_blocks + j / a.page];
  if (a.num_blocks > 0 && blk >= a.num_blocks) {
    if (lane == 0) prism_report(PRISM_ERR_BOUNDS, 2);
    blk = -1;
  }
  for (int h = 0; h < a.Hkv; ++h) {
    uint2 kb = make_uint2(0u, 0u), vb = make_uint2(0u, 0u);
    if (blk >= 0) {
      const size_t row = ((size_t)blk * a.Hkv + h) * a.page + (j % a.page);
      if constexpr (KV8) {
        const uint32_t k4 = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(a.k_cache) + row * FA_HD)[lane];
        const uint32_t v4 = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(a.v_cache) + row * FA_HD)[lane];
        kb = e4m3x4_to_bf16x4(k4, a.k_scale ? a.k_scale[row] : 1.0f);
        vb = e4m3x4_to_bf16x4(v4, a.v_scale ? a.v_scale[row] : 1.0f);
      } else {
        kb = reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.k_cache) + row * FA_HD)[lane];
        vb = reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.v_cache) + row * FA_HD)[lane];
      }
    }
    const size_t o = ((size_t)dst_row * a.Hkv + h) * FA_HD;
    reinterpret_cast<uint2*>(a.k_out + o)[lane] = kb;
    reinterpret_cast<uint2*>(a.v_out + o)[lane] = vb;
  }
}

}  // namespace

// Causal or bidirectional self-attention over contiguous segments, head dimension 128 or 72.
// q [T][q_stride], k / v [T][kv_stride] bf16 with the heads side by side (views into a packed
// QKV projection are fine); out [T][o_stride].  Rows and strides must be 16-byte aligned.
static int flash_tc_impl(const void* q, long long q_stride, const void* k, const void* v, long long kv_stride, void* out,
                         long long o_stride, const void* cu_q, const void* cu_kv, int T, int Tkv, int S, int max_q_len,
                         int Hq, int Hkv, int hd, int causal, float scale, void* stream, int pdl) {
  if (S <= 0 || max_q_len <= 0 || T <= 0 || Tkv <= 0) return 0;
  if (Hq % Hkv) return -1;
  if ((q_stride % 8) || (kv_stride % 8) || (o_stride % 8)) return -2;
  if ((reinterpret_cast<unsigned long long>(q) | reinterpret_cast<unsigned long long>(k) |
       reinterpret_cast<unsigned long long>(v) | reinterpret_cast<unsigned long long>(out)) & 15ull)
    return -3;
  if (hd != 128 && hd != 72) return -4;
  CUtensorMap tq, tk, tv;
  int rc = prism_make_head_tensor_map(q, (unsigned long long)T, (unsigned)Hq, (unsigned)hd, (unsigned long long)q_stride, FA_BM, &tq);
  if (rc) return rc;
  rc = prism_make_head_tensor_map(k, (unsigned long long)Tkv, (unsigned)Hkv, (unsigned)hd, (unsigned long long)kv_stride, FA_BN, &tk);
  if (rc) return rc;
  rc = prism_make_head_tensor_map(v, (unsigned long long)Tkv, (unsigned)Hkv, (unsigned)hd, (unsigned long long)kv_stride, FA_BN, &tv);
  if (rc) return rc;
  FaArgs a;
  a.cu_q = reinterpret_cast<const int*>(cu_q);
  a.cu_kv = reinterpret_cast<const int*>(cu_kv);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.o_stride = o_stride;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.hd = hd;
  a.causal = causal;
  a.scale = scale;
  const size_t smem = 1024 + Q_BYTES + (size_t)FA_STAGES * STAGE_BYTES + 32 * 8 + 64 + 6 * FA_BM * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_tc_kernel<80>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = (max_q_len + FA_BM - 1) / FA_BM;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (hd == 128)
    return (int)prism_launch(flash_tc_kernel<128>, dim3(tiles, Hq, S), dim3(FA_THREADS), smem, st, pdl != 0, tq, tk, tv, a);
  return (int)prism_launch(flash_tc_kernel<80>, dim3(tiles, Hq, S), dim3(FA_THREADS), smem, st, pdl != 0, tq, tk, tv, a);
}

PRISM_API int prism_flash_attention_tc(const void* q, long long q_stride, const void* k, const void* v,
                                       long long kv_stride, void* out, long long o_stride, const void* cu_q, int T,
                                       int S, int max_q_len, int Hq, int Hkv, int hd, int causal, float scale,
                                       void* stream, int pdl) {
  return flash_tc_impl(q, q_stride, k, v, kv_stride, out, o_stride, cu_q, nullptr, T, T, S, max_q_len, Hq, Hkv, hd, causal,
                       scale, stream, pdl);
}

// Causal attention of new tokens over the paged cache, head dimension 128: the keys each sequence
// sees (cu_kv[s+1] - cu_kv[s] of them: history, shared prefix pages and this chunk, already
// stored; at least as many as the sequence has query rows) are gathered into k_rows / v_rows
// [Tkv][Hkv * 128] bf16 and the tensor-core kernel runs over those.  kv_mode: 0 bf16 pages,
// 1 E4M3 pages with unit scale, 2 E4M3 pages with one scale per key row and head.
PRISM_API int prism_paged_prefill_tc(const void* q, long long q_stride, void* out, long long o_stride, const void* cu_q,
                                     const void* cu_kv, const void* k_cache, const void* v_cache, const void* k_scale,
                                     const void* v_scale, const void* block_tables, int max_blocks, int num_blocks,
                                     int page, void* k_rows, void* v_rows, int T, int Tkv, int S, int max_q_len,
                                     int max_kv_len, int Hq, int Hkv, int hd, int kv_mode, float scale, void* stream,
                                     int pdl) {
  if (S <= 0 || max_q_len <= 0 || T <= 0) return 0;
  if (hd != FA_HD) return -4;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  if (page <= 0 || max_blocks <= 0 || Tkv <= 0 || max_kv_len <= 0 || max_kv_len > Tkv) return -5;
  if (!cu_kv || !k_rows || !v_rows || !k_cache || !v_cache || !block_tables) return -6;
  GatherArgs g;
  g.k_cache = k_cache;
  g.v_cache = v_cache;
  g.k_scale = kv_mode == 2 ? reinterpret_cast<const float*>(k_scale) : nullptr;
  g.v_scale = kv_mode == 2 ? reinterpret_cast<const float*>(v_scale) : nullptr;
  g.block_tables = reinterpret_cast<const int*>(block_tables);
  g.cu_kv = reinterpret_cast<const int*>(cu_kv);
  g.k_out = reinterpret_cast<__nv_bfloat16*>(k_rows);
  g.v_out = reinterpret_cast<__nv_bfloat16*>(v_rows);
  g.max_blocks = max_blocks;
  g.num_blocks = num_blocks;
  g.page = page;
  g.Hkv = Hkv;
  g.Tkv = Tkv;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((max_kv_len + GATHER_ROWS - 1) / GATHER_ROWS, S);
  cudaError_t e = kv_mode == 0 ? prism_launch(gather_pages_kernel<false>, grid, dim3(GATHER_ROWS * 32), 0, st, pdl != 0, g)
                               : prism_launch(gather_pages_kernel<true>, grid, dim3(GATHER_ROWS * 32), 0, st, pdl != 0, g);
  if (e != cudaSuccess) return (int)e;
  return flash_tc_impl(q, q_stride, k_rows, v_rows, (long long)Hkv * FA_HD, out, o_stride, cu_q, cu_kv, T, Tkv, S, max_q_len,
                       Hq, Hkv, hd, 1, scale, stream, pdl);
}
