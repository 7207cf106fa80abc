// Attention kernels.
//
//  * paged_decode_kernel: one new query token per sequence against a paged KV cache
//    (bf16, unit-scale fp8 or scaled fp8 with one fp32 scale per token and KV head).
//    One CTA handles ALL query heads that share a KV head (GQA packing), so every KV byte
//    is read once instead of Hq/Hkv times, and the context is split across CTAs
//    (split-KV) with a small combine kernel; the loop bound comes from a device array so
//    one CUDA graph serves every context length.  Replaces the reference's Triton
//    one-program-per-query-head kernel (prism_infer/ops/paged_decode.py:41-180).
//  * flash_fwd_kernel: tiled online-softmax attention for prefill and for the vision
//    tower.  Keys/values come either from contiguous bf16 rows (no history, ViT frame
//    segments) or straight from the paged cache, including shared read-only prefix
//    pages and scaled-fp8 pages, so chunked prefill and prefix hits no longer go through
//    a per-sequence Python gather loop (prism_infer/ops/paged_attention_reference.py:185-390).
//
// Cache layout everywhere: payload [blocks][Hkv][page][D], scales [blocks][Hkv][page].
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(attn)

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float2 fp8x2_to_float2(unsigned short v) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// =====================================================================================
// Decode
// =====================================================================================
struct DecodeArgs {
  const bf16* q;            // [B][Hq][D]
  const void* k_cache;
  const void* v_cache;
  const float* k_scale;     // null unless scaled fp8
  const float* v_scale;
  const int* block_tables;  // [B][max_blocks], < 0 = hole
  const int* context_lens;  // [B]
  float* part_o;            // [B][Hq][nsplit][D]
  float* part_ml;           // [B][Hq][nsplit][2]  (max, sum)
  bf16* out;                // [B][Hq][D] (written directly when nsplit == 1)
  int* counters;            // [B * Hkv] zero-initialised, self-resetting; null = separate combine kernel
  int Hq, Hkv, page, max_blocks, nsplit;
  int num_blocks;           // pages in the cache; <= 0: unknown, only holes (< 0) are skipped
  float scale;
};

// Page-table guards shared by the decode and prefill kernels.  A context longer than the
// table can describe is cut to the table's reach, and a page id at or beyond the cache is
// treated as a hole; both are recorded in the status word (PRISM_ERR_BOUNDS) and the access
// is skipped, so a stale table or an over-long length costs wrong tokens that the engine
// reports, never an out-of-range read.
__device__ __forceinline__ int clamp_context(int ctx, int max_blocks, int page) {
  const long long reach = (long long)max_blocks * page;
  if ((long long)ctx > reach) {
    if (threadIdx.x == 0) prism_report(PRISM_ERR_BOUNDS, 1);
    return (int)reach;
  }
  return ctx < 0 ? 0 : ctx;
}
__device__ __forceinline__ int checked_page(int blk, int num_blocks) {
  if (num_blocks > 0 && blk >= num_blocks) {
    prism_report(PRISM_ERR_BOUNDS, 2);
    return -1;
  }
  return blk;
}

// KV8 = true: fp8 payload (16 elements per lane), false: bf16 payload (8 elements per lane)
template <int D, int G, bool KV8>
__global__ void __launch_bounds__(128) paged_decode_kernel(const DecodeArgs a) {
  constexpr int EPL = KV8 ? 16 : 8;   // elements per lane
  constexpr int LPT = D / EPL;        // lanes per token
  constexpr int TPW = 32 / LPT;       // tokens per warp iteration
  constexpr int NWARP = 4;
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = lane / LPT;        // token slot inside the warp
  const int part = lane % LPT;        // which EPL-wide slice of the head dim
  pdl_launch_dependents();
  pdl_wait();
  const int ctx = clamp_context(a.context_lens[b], a.max_blocks, a.page);
  const int per_split = ((ctx + a.nsplit - 1) / a.nsplit + TPW * NWARP * 4 - 1) / (TPW * NWARP * 4) * (TPW * NWARP * 4);
  const int j_begin = split * per_split;
  const int j_end = min(ctx, j_begin + per_split);

  float q[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const bf16* qp = a.q + ((size_t)b * a.Hq + (size_t)kvh * G + g) * D + part * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) q[g][e] = __bfloat162float(qp[e]) * a.scale;
  }
  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
  }
  const int* bt = a.block_tables + (size_t)b * a.max_blocks;

  // UNR independent token groups per warp iteration: all page-table, payload and scale
  // loads of an iteration are issued before any arithmetic, so a short context costs one
  // or two memory round trips instead of one per group.
  constexpr int UNR = 4;
  for (int j0 = j_begin + warp * TPW * UNR; j0 < j_end; j0 += TPW * NWARP * UNR) {
    uint4 kr[UNR], vr[UNR];
    float ks[UNR], vs[UNR];
    bool valid[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int j = j0 + u * TPW + slot;
      int blk = -1;
      if (j < j_end) blk = checked_page(bt[j / a.page], a.num_blocks);
      valid[u] = blk >= 0;
      kr[u] = make_uint4(0, 0, 0, 0);
      vr[u] = make_uint4(0, 0, 0, 0);
      ks[u] = 1.0f;
      vs[u] = 1.0f;
      if (valid[u]) {
        const size_t row = ((size_t)blk * a.Hkv + kvh) * a.page + (j % a.page);
        const size_t off = row * D * (KV8 ? 1 : 2) + (size_t)part * 16;
        kr[u] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.k_cache) + off));
        vr[u] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.v_cache) + off));
        if (KV8 && a.k_scale != nullptr) {
          ks[u] = __ldg(a.k_scale + row);
          vs[u] = __ldg(a.v_scale + row);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      float kf[EPL], vf[EPL];
      if (KV8) {
        const unsigned short* kp = reinterpret_cast<const unsigned short*>(&kr[u]);
        const unsigned short* vp = reinterpret_cast<const unsigned short*>(&vr[u]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 kk = fp8x2_to_float2(kp[e]);
          const float2 vv = fp8x2_to_float2(vp[e]);
          kf[(2 * e) % EPL] = kk.x;
          kf[(2 * e + 1) % EPL] = kk.y;
          vf[(2 * e) % EPL] = vv.x;
          vf[(2 * e + 1) % EPL] = vv.y;
        }
      } else {
        const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kr[u]);
        const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&vr[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 kk = __bfloat1622float2(kp[e]);
          const float2 vv = __bfloat1622float2(vp[e]);
          kf[2 * e] = kk.x;
          kf[2 * e + 1] = kk.y;
          vf[2 * e] = vv.x;
          vf[2 * e + 1] = vv.y;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) s += q[g][e] * kf[e];
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid[u]) {
          s *= ks[u];
          const float mn = fmaxf(m[g], s);
          const float corr = __expf(m[g] - mn);
          const float p = __expf(s - mn);
          l[g] = l[g] * corr + p;
          const float pv = p * vs[u];
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + pv * vf[e];
          m[g] = mn;
        }
      }
    }
  }
  // merge the TPW token slots of the warp
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int o = LPT; o < 32; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo);
      const float c0 = (m[g] == -INFINITY) ? 0.0f : __expf(m[g] - mn);
      const float c1 = (mo == -INFINITY) ? 0.0f : __expf(mo - mn);
      l[g] = l[g] * c0 + lo * c1;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
        acc[g][e] = acc[g][e] * c0 + ao * c1;
      }
      m[g] = mn;
    }
  }
  // merge the warps through shared memory
  __shared__ float s_m[NWARP][G], s_l[NWARP][G];
  __shared__ float s_acc[NWARP][G][D];
  if (slot == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (part == 0) {
        s_m[warp][g] = m[g];
        s_l[warp][g] = l[g];
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) s_acc[warp][g][part * EPL + e] = acc[g][e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) {
      const float c = (s_m[w][g] == -INFINITY) ? 0.0f : __expf(s_m[w][g] - mm);
      ll += s_l[w][g] * c;
      oo += s_acc[w][g][d] * c;
    }
    const int hq = kvh * G + g;
    if (a.nsplit == 1) {
      a.out[((size_t)b * a.Hq + hq) * D + d] = __float2bfloat16_rn(ll > 0.0f ? oo / ll : 0.0f);
    } else {
      const size_t pidx = ((size_t)b * a.Hq + hq) * a.nsplit + split;
      a.part_o[pidx * D + d] = oo;
      if (d == 0) {
        a.part_ml[pidx * 2] = mm;
        a.part_ml[pidx * 2 + 1] = ll;
      }
    }
  }
  if (a.nsplit == 1 || a.counters == nullptr) return;
  // The last split CTA of this (sequence, KV head) to finish merges all splits, which saves
  // the separate combine launch.  Classic fence / counter / fence hand-off.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(&a.counters[b * a.Hkv + kvh], 1);
    s_last = (old == a.nsplit - 1);
    if (s_last) a.counters[b * a.Hkv + kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Merge: coefficients of every (head, split) go to shared memory first, then each thread
  // accumulates its outputs with independent loads (no serial chain over the splits).
  __shared__ float s_coef[G][32];
  __shared__ float s_inv[G];
  const int ns = a.nsplit;  // <= 32
  if (warp < G || G > NWARP) {
    for (int g = warp; g < G; g += NWARP) {
      const size_t bh = (size_t)b * a.Hq + kvh * G + g;
      const float ms = lane < ns ? __ldcg(&a.part_ml[(bh * ns + lane) * 2]) : -INFINITY;
      const float ls = lane < ns ? __ldcg(&a.part_ml[(bh * ns + lane) * 2 + 1]) : 0.0f;
      const float mm = warp_max(ms);
      const float c = (ms == -INFINITY) ? 0.0f : __expf(ms - mm);
      const float ll = warp_sum(ls * c);
      s_coef[g][lane] = c;
      if (lane == 0) s_inv[g] = ll > 0.0f ? 1.0f / ll : 0.0f;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    const size_t bh = (size_t)b * a.Hq + kvh * G + g;
    const float* po = a.part_o + bh * ns * D + d;
    float oo = 0.0f;
#pragma unroll 8
    for (int s = 0; s < ns; ++s) oo += __ldcg(po + (size_t)s * D) * s_coef[g][s];
    a.out[bh * D + d] = __float2bfloat16_rn(oo * s_inv[g]);
  }
}

__global__ void __launch_bounds__(128) decode_combine_kernel(const float* part_o, const float* part_ml, bf16* out,
                                                             int nsplit, int D) {
  const size_t bh = blockIdx.x;  // b * Hq + hq
  pdl_launch_dependents();
  pdl_wait();
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, part_ml[(bh * nsplit + s) * 2]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float ll = 0.0f, oo = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = part_ml[(bh * nsplit + s) * 2];
      const float c = (ms == -INFINITY) ? 0.0f : __expf(ms - mm);
      ll += part_ml[(bh * nsplit + s) * 2 + 1] * c;
      oo += part_o[(bh * nsplit + s) * D + d] * c;
    }
    out[bh * D + d] = __float2bfloat16_rn(ll > 0.0f ? oo / ll : 0.0f);
  }
}

// =====================================================================================
// Prefill / vision: tiled online-softmax attention on mma.sync m16n8k16 (bf16).
// The GEMM-heavy part of prefill lives in the tcgen05 kernels; this kernel is the
// memory-format adapter (paged / fp8 / ragged segments) around a 64x64 tile loop.
// =====================================================================================
struct FlashArgs {
  const bf16* q;            // token-major, q_stride elements per token, heads packed with HD_REAL
  long long q_stride;
  bf16* out;                // [T][Hq][HD_REAL]
  long long o_stride;
  const int* cu_q;          // [S+1]
  // contiguous K/V (mode 0)
  const bf16* k;
  const bf16* v;
  long long kv_stride;
  // paged K/V (mode 1 bf16, mode 2 fp8)
  const void* k_cache;
  const void* v_cache;
  const float* k_scale;
  const float* v_scale;
  const int* block_tables;
  const int* kv_lens;       // [S] total keys visible to the sequence (history + this chunk)
  int max_blocks, page;
  int num_blocks;           // pages in the cache; <= 0: unknown
  int Hq, Hkv;
  int causal;
  float scale;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
  // src-size 0 zero-fills the 16 bytes without touching global memory
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// BM query rows per CTA (16 per warp), 64-key tiles, K/V double-buffered in shared memory:
// while the warps score tile i, tile i+1 is on its way (cp.async for bf16 sources; for FP8
// pages the bytes are fetched into registers before the math and dequantised into the
// other buffer after it).  One __syncthreads per tile.
template <int HD, int HD_REAL, int MODE, int BM>
__global__ void __launch_bounds__(BM * 2, MODE == 2 ? (BM == 128 ? 1 : 2) : (BM == 128 ? 2 : 3)) flash_fwd_kernel(const FlashArgs a) {
  constexpr int BN = 64;
  constexpr int NT = BM * 2;           // threads
  constexpr int LDS = HD + 8;          // padded row (elements) -> conflict-free ldmatrix
  constexpr int CHUNKS = HD_REAL / 8;  // 8-element chunks per row
  constexpr int NI = (BN * CHUNKS + NT - 1) / NT;  // chunks per thread and tile
  extern __shared__ __align__(16) uint8_t fsm[];
  bf16* Qs = reinterpret_cast<bf16*>(fsm);
  bf16* KV = Qs + BM * LDS;  // [buffer][k|v][BN][LDS]

  const int seq = blockIdx.z, head = blockIdx.y, qt = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  pdl_launch_dependents();
  pdl_wait();
  const int q_start = a.cu_q[seq];
  const int q_len = a.cu_q[seq + 1] - q_start;
  const int q0 = qt * BM;
  if (q0 >= q_len) return;
  const int kv_len = (MODE == 0) ? q_len : clamp_context(a.kv_lens[seq], a.max_blocks, a.page);
  const int kvh = head / (a.Hq / a.Hkv);
  const int pos_off = kv_len - q_len;  // absolute key position of local query 0
  const int* bt = (MODE == 0) ? nullptr : a.block_tables + (size_t)seq * a.max_blocks;

  // zero the padding columns once (HD_REAL < HD only for the 72-wide vision heads)
  if constexpr (HD_REAL < HD) {
    for (int i = tid; i < (BM + 4 * BN) * (HD - HD_REAL); i += NT) {
      const int r = i / (HD - HD_REAL), c = HD_REAL + i % (HD - HD_REAL);
      Qs[r * LDS + c] = __float2bfloat16(0.0f);  // Q and the K/V buffers are contiguous with the same pitch
    }
  }
  for (int i = tid; i < BM * CHUNKS; i += NT) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (q0 + r < q_len)
      v = *reinterpret_cast<const uint4*>(a.q + (size_t)(q_start + q0 + r) * a.q_stride + (size_t)head * HD_REAL + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LDS + c * 8) = v;
  }

  int kv_end = kv_len;
  if (a.causal) kv_end = min(kv_len, pos_off + min(q0 + BM, q_len));
  const int n_tiles = (kv_end + BN - 1) / BN;

  // ---- tile movers ------------------------------------------------------------------
  uint2 st_k[NI], st_v[NI];
  float st_ks[NI], st_vs[NI];
  auto issue_async = [&](int tile, int buf) {  // MODE 0 / 1: global bf16 -> shared, asynchronous
    bf16* Kd = KV + (size_t)(buf * 2) * BN * LDS;
    bf16* Vd = Kd + BN * LDS;
    const int j0 = tile * BN;
#pragma unroll
    for (int it = 0; it < NI; ++it) {
      const int i = tid + it * NT;
      if (i < BN * CHUNKS) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const int j = j0 + r;
        const bf16* ksrc = a.q;  // any valid address for the zero-fill form
        const bf16* vsrc = a.q;
        bool ok = j < kv_len;
        if (ok) {
          if (MODE == 0) {
            const size_t off = (size_t)(q_start + j) * a.kv_stride + (size_t)kvh * HD_REAL + c * 8;
            ksrc = a.k + off;
            vsrc = a.v + off;
          } else {
            const int blk = checked_page(bt[j / a.page], a.num_blocks);
            ok = blk >= 0;
            if (ok) {
              const size_t row = ((size_t)blk * a.Hkv + kvh) * a.page + (j % a.page);
              ksrc = reinterpret_cast<const bf16*>(a.k_cache) + row * HD_REAL + c * 8;
              vsrc = reinterpret_cast<const bf16*>(a.v_cache) + row * HD_REAL + c * 8;
            }
          }
        }
        cp_async16(Kd + r * LDS + c * 8, ksrc, ok);
        cp_async16(Vd + r * LDS + c * 8, vsrc, ok);
      }
    }
    cp_async_commit();
  };
  auto fetch_fp8 = [&](int tile) {  // MODE 2: FP8 bytes and scales -> registers
    const int j0 = tile * BN;
#pragma unroll
    for (int it = 0; it < NI; ++it) {
      const int i = tid + it * NT;
      st_k[it] = make_uint2(0, 0);
      st_v[it] = make_uint2(0, 0);
      st_ks[it] = st_vs[it] = 0.0f;
      if (i < BN * CHUNKS) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const int j = j0 + r;
        if (j < kv_len) {
          const int blk = checked_page(bt[j / a.page], a.num_blocks);
          if (blk >= 0) {
            const size_t row = ((size_t)blk * a.Hkv + kvh) * a.page + (j % a.page);
            st_k[it] = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(a.k_cache) + row * HD_REAL + c * 8);
            st_v[it] = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(a.v_cache) + row * HD_REAL + c * 8);
            st_ks[it] = a.k_scale ? a.k_scale[row] : 1.0f;
            st_vs[it] = a.v_scale ? a.v_scale[row] : 1.0f;
          }
        }
      }
    }
  };
  auto stash_fp8 = [&](int buf) {  // registers -> bf16 in shared memory
    bf16* Kd = KV + (size_t)(buf * 2) * BN * LDS;
    bf16* Vd = Kd + BN * LDS;
#pragma unroll
    for (int it = 0; it < NI; ++it) {
      const int i = tid + it * NT;
      if (i < BN * CHUNKS) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const unsigned short* kp = reinterpret_cast<const unsigned short*>(&st_k[it]);
        const unsigned short* vp = reinterpret_cast<const unsigned short*>(&st_v[it]);
        uint4 kv4, vv4;
        uint32_t* ko = reinterpret_cast<uint32_t*>(&kv4);
        uint32_t* vo = reinterpret_cast<uint32_t*>(&vv4);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 kk = fp8x2_to_float2(kp[e]);
          const float2 vv = fp8x2_to_float2(vp[e]);
          ko[e] = pack_bf16(kk.x * st_ks[it], kk.y * st_ks[it]);
          vo[e] = pack_bf16(vv.x * st_vs[it], vv.y * st_vs[it]);
        }
        *reinterpret_cast<uint4*>(Kd + r * LDS + c * 8) = kv4;
        *reinterpret_cast<uint4*>(Vd + r * LDS + c * 8) = vv4;
      }
    }
  };

  if (MODE == 2) {
    fetch_fp8(0);
    stash_fp8(0);
  } else {
    issue_async(0, 0);
  }

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const float sl2 = a.scale * 1.4426950408889634f;
  const int q_r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
  const int q_c = 8 * (lane >> 4);
  const int warp_last_row = q0 + warp * 16 + 15;  // last query row of this warp (local index)

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    const int j0 = tile * BN;
    if (MODE != 2) cp_async_wait_all();
    __syncthreads();  // this tile is in shared memory; everyone is done with the other buffer
    const bool more = tile + 1 < n_tiles;
    if (more) {
      if (MODE == 2) fetch_fp8(tile + 1);
      else issue_async(tile + 1, buf ^ 1);
    }
    // a warp whose rows all lie before this tile's first key has nothing to add (causal)
    const bool active = !(a.causal && j0 > pos_off + warp_last_row) && (q0 + warp * 16 < q_len);
    if (active) {
      const bf16* Ks = KV + (size_t)(buf * 2) * BN * LDS;
      const bf16* Vs = Ks + BN * LDS;
      // S = Q K^T  (16 x 64 per warp)
      float s[BN / 8][4];
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t qf[4];
        ldsm_x4(qf, smem_u32(Qs + q_r * LDS + kk * 16 + q_c));
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          uint32_t kb[4];
          const int n = np * 16 + (lane & 7) + 8 * (lane >> 4);
          const int c = kk * 16 + 8 * ((lane >> 3) & 1);
          ldsm_x4(kb, smem_u32(Ks + n * LDS + c));
          mma_bf16(s[2 * np], qf, kb[0], kb[1]);
          mma_bf16(s[2 * np + 1], qf, kb[2], kb[3]);
        }
      }
      // mask + online softmax (rows g and g+8 of this warp's 16-row slab)
      const int row0 = q0 + warp * 16 + g;
      const bool need_mask = (j0 + BN > kv_len) || (a.causal && (j0 + BN - 1 > pos_off + q0 + warp * 16));
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[i][e] * sl2;
          if (need_mask) {
            const int col = j0 + i * 8 + t4 * 2 + (e & 1);
            const int row = row0 + ((e >> 1) ? 8 : 0);
            if (col >= kv_len || (a.causal && col > pos_off + row)) v = -INFINITY;
          }
          s[i][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mn = fmaxf(m_run[r], mx[r]);
        m_use[r] = (mn == -INFINITY) ? 0.0f : mn;
        corr[r] = (m_run[r] == -INFINITY) ? 0.0f : ex2_fast(m_run[r] - m_use[r]);
        m_run[r] = mn;
      }
      float rs[2] = {0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = ex2_fast(s[i][e] - m_use[e >> 1]);
          s[i][e] = p;
          rs[e >> 1] += p;
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
        l_run[r] = l_run[r] * corr[r] + rs[r];
      }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      // O += P V
#pragma unroll
      for (int kt = 0; kt < BN / 16; ++kt) {
        uint32_t pa[4];
        pa[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
        pa[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
        pa[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
        pa[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
          uint32_t vb[4];
          const int tok = kt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
          const int d = dp * 16 + 8 * (lane >> 4);
          ldsm_x4_t(vb, smem_u32(Vs + tok * LDS + d));
          mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
          mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
        }
      }
    }
    if (MODE == 2 && more) stash_fp8(buf ^ 1);
  }
  // normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = q0 + warp * 16 + g + 8 * r;
    if (row >= q_len) continue;
    const float inv = l_run[r] > 0.0f ? 1.0f / l_run[r] : 0.0f;
    bf16* dst = a.out + (size_t)(q_start + row) * a.o_stride + (size_t)head * HD_REAL;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const int d = i * 8 + t4 * 2;
      if (d < HD_REAL) {
        *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
      }
    }
  }
}

// =====================================================================================
// Decode on the tensor cores (mma.sync m16n8k16): the G query heads of a KV head are rows of
// one 16-row A tile, a 64-token K/V tile is dequantised to bf16 in shared memory once and
// each warp scores and accumulates 16 of its tokens.  Used for larger batches, where the
// SIMT kernel above is instruction-bound (one FMA per head and byte); same split-KV
// partial format and in-kernel merge.
// =====================================================================================
template <int D, int G, bool KV8>
__global__ void __launch_bounds__(128) paged_decode_mma_kernel(const DecodeArgs a) {
  constexpr int BN = 64, NWARP = 4;
  constexpr int LDS = D + 8;
  constexpr int CHUNKS = D / 8;
  extern __shared__ __align__(16) uint8_t dsm[];
  bf16* Qs = reinterpret_cast<bf16*>(dsm);
  bf16* Ks = Qs + 16 * LDS;
  bf16* Vs = Ks + BN * LDS;
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  pdl_launch_dependents();
  pdl_wait();
  const int ctx = clamp_context(a.context_lens[b], a.max_blocks, a.page);
  const int per_split = ((ctx + a.nsplit - 1) / a.nsplit + BN - 1) / BN * BN;
  const int j_begin = split * per_split;
  const int j_end = min(ctx, j_begin + per_split);
  const int* bt = a.block_tables + (size_t)b * a.max_blocks;

  for (int i = tid; i < 16 * CHUNKS; i += 128) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)b * a.Hq + (size_t)kvh * G + r) * D + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LDS + c * 8) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
  {
    const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
    const int c = 8 * (lane >> 4);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) ldsm_x4(qf[kk], smem_u32(Qs + r * LDS + kk * 16 + c));
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run = -INFINITY, l_run = 0.0f;  // row g (rows >= G are padding)
  const float sl2 = a.scale * 1.4426950408889634f;

  // Software pipeline: the global loads of tile i+1 are in flight (in registers) while
  // tile i is scored; 16-byte loads, CPR chunks per token row.
  constexpr int CPR = KV8 ? D / 16 : D / 8;      // 16-byte chunks per row
  constexpr int NL = BN * CPR / 128;             // chunks per thread (K and V each)
  __shared__ unsigned char s_valid[BN];
  uint4 kreg[NL], vreg[NL];
  float ksc[NL], vsc[NL];
  auto prefetch = [&](int j0) {
#pragma unroll
    for (int u = 0; u < NL; ++u) {
      const int idx = tid + u * 128;
      const int r = idx / CPR, c = idx % CPR;
      const int j = j0 + r;
      kreg[u] = make_uint4(0, 0, 0, 0);
      vreg[u] = make_uint4(0, 0, 0, 0);
      ksc[u] = -1.0f;  // marks an absent row
      vsc[u] = 1.0f;
      if (j < j_end) {
        const int blk = checked_page(bt[j / a.page], a.num_blocks);
        if (blk >= 0) {
          const size_t row = ((size_t)blk * a.Hkv + kvh) * a.page + (j % a.page);
          const size_t off = row * D * (KV8 ? 1 : 2) + (size_t)c * 16;
          kreg[u] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.k_cache) + off));
          vreg[u] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.v_cache) + off));
          ksc[u] = (KV8 && a.k_scale) ? __ldg(a.k_scale + row) : 1.0f;
          vsc[u] = (KV8 && a.v_scale) ? __ldg(a.v_scale + row) : 1.0f;
        }
      }
    }
  };
  if (j_begin < j_end) prefetch(j_begin);
  for (int j0 = j_begin; j0 < j_end; j0 += BN) {
    __syncthreads();
#pragma unroll
    for (int u = 0; u < NL; ++u) {
      const int idx = tid + u * 128;
      const int r = idx / CPR, c = idx % CPR;
      const bool present = ksc[u] >= 0.0f;
      if (c == 0) s_valid[r] = present ? 1 : 0;
      if (KV8) {
        const unsigned short* kp = reinterpret_cast<const unsigned short*>(&kreg[u]);
        const unsigned short* vp = reinterpret_cast<const unsigned short*>(&vreg[u]);
        uint4 ko[2], vo[2];
        uint32_t* kw = reinterpret_cast<uint32_t*>(ko);
        uint32_t* vw = reinterpret_cast<uint32_t*>(vo);
        const float ks = present ? ksc[u] : 0.0f, vs = vsc[u];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 kk = fp8x2_to_float2(kp[e]);
          const float2 vv = fp8x2_to_float2(vp[e]);
          kw[e] = pack_bf16(kk.x * ks, kk.y * ks);
          vw[e] = pack_bf16(vv.x * vs, vv.y * vs);
        }
        *reinterpret_cast<uint4*>(Ks + r * LDS + c * 16) = ko[0];
        *reinterpret_cast<uint4*>(Ks + r * LDS + c * 16 + 8) = ko[1];
        *reinterpret_cast<uint4*>(Vs + r * LDS + c * 16) = vo[0];
        *reinterpret_cast<uint4*>(Vs + r * LDS + c * 16 + 8) = vo[1];
      } else {
        *reinterpret_cast<uint4*>(Ks + r * LDS + c * 8) = kreg[u];
        *reinterpret_cast<uint4*>(Vs + r * LDS + c * 8) = vreg[u];
      }
    }
    __syncthreads();
    if (j0 + BN < j_end) prefetch(j0 + BN);
    const int tok0 = warp * 16;  // this warp's 16 tokens of the tile
    if (j0 + tok0 >= j_end) continue;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t kb[4];
      const int n = tok0 + (lane & 7) + 8 * (lane >> 4);
      const int c = kk * 16 + 8 * ((lane >> 3) & 1);
      ldsm_x4(kb, smem_u32(Ks + n * LDS + c));
      mma_bf16(s[0], qf[kk], kb[0], kb[1]);
      mma_bf16(s[1], qf[kk], kb[2], kb[3]);
    }
    // only row g (c0, c1 of each n-tile) is a real query head; rows g + 8 are padding
    float mx = -INFINITY;
    float p[2][2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool ok = s_valid[tok0 + i * 8 + t4 * 2 + e] != 0;
        const float v = ok ? s[i][e] * sl2 : -INFINITY;
        p[i][e] = v;
        mx = fmaxf(mx, v);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m_run, mx);
    const float m_use = (mn == -INFINITY) ? 0.0f : mn;
    const float corr = (m_run == -INFINITY) ? 0.0f : exp2f(m_run - m_use);
    m_run = mn;
    float rs = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p[i][e] = exp2f(p[i][e] - m_use);
        rs += p[i][e];
      }
    }
    rs += __shfl_xor_sync(0xffffffffu, rs, 1);
    rs += __shfl_xor_sync(0xffffffffu, rs, 2);
    l_run = l_run * corr + rs;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr;
      o[i][1] *= corr;
    }
    uint32_t pa[4];
    pa[0] = pack_bf16(p[0][0], p[0][1]);
    pa[1] = 0;  // rows g + 8
    pa[2] = pack_bf16(p[1][0], p[1][1]);
    pa[3] = 0;
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t vb[4];
      const int tok = tok0 + (lane & 7) + 8 * ((lane >> 3) & 1);
      const int d = dp * 16 + 8 * (lane >> 4);
      ldsm_x4_t(vb, smem_u32(Vs + tok * LDS + d));
      mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
      mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
    }
  }
  // merge the four warps (rows g < G only), reusing the tile buffers
  __syncthreads();
  float* s_m = reinterpret_cast<float*>(Ks);          // [NWARP][G]
  float* s_l = s_m + NWARP * G;                        // [NWARP][G]
  float* s_acc = s_l + NWARP * G;                      // [NWARP][G][D]
  if (g < G) {
    if (t4 == 0) {
      s_m[warp * G + g] = m_run;
      s_l[warp * G + g] = l_run;
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      s_acc[(warp * G + g) * D + i * 8 + t4 * 2] = o[i][0];
      s_acc[(warp * G + g) * D + i * 8 + t4 * 2 + 1] = o[i][1];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += 128) {
    const int gg = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) mm = fmaxf(mm, s_m[w * G + gg]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) {
      const float ms = s_m[w * G + gg];
      const float c = (ms == -INFINITY) ? 0.0f : exp2f(ms - mm);
      ll += s_l[w * G + gg] * c;
      oo += s_acc[(w * G + gg) * D + d] * c;
    }
    const int hq = kvh * G + gg;
    if (a.nsplit == 1) {
      a.out[((size_t)b * a.Hq + hq) * D + d] = __float2bfloat16_rn(ll > 0.0f ? oo / ll : 0.0f);
    } else {
      // partial format shared with the SIMT kernel: natural-log domain maximum
      const size_t pidx = ((size_t)b * a.Hq + hq) * a.nsplit + split;
      a.part_o[pidx * D + d] = oo;
      if (d == 0) {
        a.part_ml[pidx * 2] = (mm == -INFINITY) ? -INFINITY : mm * 0.6931471805599453f;
        a.part_ml[pidx * 2 + 1] = ll;
      }
    }
  }
  if (a.nsplit == 1 || a.counters == nullptr) return;
  __shared__ int s_last2;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&a.counters[b * a.Hkv + kvh], 1);
    s_last2 = (old == a.nsplit - 1);
    if (s_last2) a.counters[b * a.Hkv + kvh] = 0;
  }
  __syncthreads();
  if (!s_last2) return;
  __threadfence();
  __shared__ float s_coef2[G][32];
  __shared__ float s_inv2[G];
  const int ns = a.nsplit;
  for (int gg = warp; gg < G; gg += NWARP) {
    const size_t bh = (size_t)b * a.Hq + kvh * G + gg;
    const float ms = lane < ns ? __ldcg(&a.part_ml[(bh * ns + lane) * 2]) : -INFINITY;
    const float ls = lane < ns ? __ldcg(&a.part_ml[(bh * ns + lane) * 2 + 1]) : 0.0f;
    const float mm = warp_max(ms);
    const float c = (ms == -INFINITY) ? 0.0f : __expf(ms - mm);
    const float ll = warp_sum(ls * c);
    s_coef2[gg][lane] = c;
    if (lane == 0) s_inv2[gg] = ll > 0.0f ? 1.0f / ll : 0.0f;
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += 128) {
    const int gg = idx / D, d = idx % D;
    const size_t bh = (size_t)b * a.Hq + kvh * G + gg;
    const float* po = a.part_o + bh * ns * D + d;
    float oo = 0.0f;
#pragma unroll 8
    for (int sidx = 0; sidx < ns; ++sidx) oo += __ldcg(po + (size_t)sidx * D) * s_coef2[gg][sidx];
    a.out[bh * D + d] = __float2bfloat16_rn(oo * s_inv2[gg]);
  }
}

template <int HD, int HD_REAL, int MODE, int BM>
int launch_flash(const FlashArgs& a, int max_q_len, int S, cudaStream_t stream, bool pdl) {
  const size_t smem = (size_t)(BM + 4 * 64) * (HD + 8) * sizeof(bf16);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<HD, HD_REAL, MODE, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = (max_q_len + BM - 1) / BM;
  return (int)prism_launch(flash_fwd_kernel<HD, HD_REAL, MODE, BM>, dim3(tiles, a.Hq, S), dim3(BM * 2), smem, stream, pdl, a);
}

template <int MODE>
int dispatch_flash(const FlashArgs& a, int hd, int max_q_len, int S, cudaStream_t stream, bool pdl) {
  // 128 query rows per CTA halve the K/V traffic per query; short sequences keep 64 so that
  // more CTAs exist
  const bool wide = max_q_len > 256;
  switch (hd) {
    case 128:
      return wide ? launch_flash<128, 128, MODE, 128>(a, max_q_len, S, stream, pdl)
                  : launch_flash<128, 128, MODE, 64>(a, max_q_len, S, stream, pdl);
    case 64:
      return wide ? launch_flash<64, 64, MODE, 128>(a, max_q_len, S, stream, pdl)
                  : launch_flash<64, 64, MODE, 64>(a, max_q_len, S, stream, pdl);
    case 72:
      return wide ? launch_flash<80, 72, MODE, 128>(a, max_q_len, S, stream, pdl)
                  : launch_flash<80, 72, MODE, 64>(a, max_q_len, S, stream, pdl);
    case 32: return launch_flash<32, 32, MODE, 64>(a, max_q_len, S, stream, pdl);
  }
  return -2;
}

template <int D, int G, bool KV8>
int launch_decode_mma(const DecodeArgs& a, int B, cudaStream_t stream, bool pdl) {
  const size_t smem = (size_t)(16 + 2 * 64) * (D + 8) * sizeof(bf16);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_mma_kernel<D, G, KV8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)prism_launch(paged_decode_mma_kernel<D, G, KV8>, dim3(B, a.Hkv, a.nsplit), dim3(128), smem, stream, pdl, a);
}

// use_mma: tensor-core kernel (larger batches); otherwise the SIMT kernel (lowest latency at batch 1)
template <int D, bool KV8>
int dispatch_decode(const DecodeArgs& a, int B, cudaStream_t stream, bool pdl, bool use_mma) {
  dim3 grid(B, a.Hkv, a.nsplit), block(128);
  if (use_mma) {
    switch (a.Hq / a.Hkv) {
      case 1: return launch_decode_mma<D, 1, KV8>(a, B, stream, pdl);
      case 2: return launch_decode_mma<D, 2, KV8>(a, B, stream, pdl);
      case 4: return launch_decode_mma<D, 4, KV8>(a, B, stream, pdl);
      case 8: return launch_decode_mma<D, 8, KV8>(a, B, stream, pdl);
    }
    return -3;
  }
  switch (a.Hq / a.Hkv) {
    case 1: return (int)prism_launch(paged_decode_kernel<D, 1, KV8>, grid, block, 0, stream, pdl, a);
    case 2: return (int)prism_launch(paged_decode_kernel<D, 2, KV8>, grid, block, 0, stream, pdl, a);
    case 4: return (int)prism_launch(paged_decode_kernel<D, 4, KV8>, grid, block, 0, stream, pdl, a);
    case 8: return (int)prism_launch(paged_decode_kernel<D, 8, KV8>, grid, block, 0, stream, pdl, a);
  }
  return -3;
}

}  // namespace

// kv_mode: 0 bf16, 1 fp8 unit scale, 2 scaled fp8.  part_o / part_ml are scratch of
// B*Hq*nsplit*D and B*Hq*nsplit*2 floats (unused when nsplit == 1).
PRISM_API int prism_paged_decode(const void* q, const void* k_cache, const void* v_cache, const void* k_scale,
                                 const void* v_scale, const void* block_tables, const void* context_lens, void* part_o,
                                 void* part_ml, void* out, void* counters, int B, int Hq, int Hkv, int D, int page,
                                 int max_blocks, int num_blocks, int nsplit, int kv_mode, float scale, int use_mma,
                                 void* stream, int pdl) {
  if (B <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || page <= 0 || max_blocks <= 0) return -1;
  DecodeArgs a;
  a.q = (const bf16*)q;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.k_scale = kv_mode == 2 ? (const float*)k_scale : nullptr;
  a.v_scale = kv_mode == 2 ? (const float*)v_scale : nullptr;
  a.block_tables = (const int*)block_tables;
  a.context_lens = (const int*)context_lens;
  a.part_o = (float*)part_o;
  a.part_ml = (float*)part_ml;
  a.out = (bf16*)out;
  a.counters = (int*)counters;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.page = page;
  a.max_blocks = max_blocks;
  a.num_blocks = num_blocks;
  a.nsplit = nsplit < 1 ? 1 : (nsplit > 32 ? 32 : nsplit);
  a.scale = scale;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  const bool mma = use_mma != 0;
  if (D == 128) rc = kv_mode ? dispatch_decode<128, true>(a, B, s, pdl != 0, mma) : dispatch_decode<128, false>(a, B, s, pdl != 0, mma);
  else if (D == 64) rc = kv_mode ? dispatch_decode<64, true>(a, B, s, pdl != 0, mma) : dispatch_decode<64, false>(a, B, s, pdl != 0, mma);
  else return -2;
  if (rc) return rc;
  if (a.nsplit > 1 && a.counters == nullptr) {
    rc = (int)prism_launch(decode_combine_kernel, dim3(B * Hq), dim3(128), 0, s, pdl != 0, (const float*)part_o,
                           (const float*)part_ml, (bf16*)out, a.nsplit, D);
  }
  return rc;
}

// mode 0: contiguous bf16 K/V rows (k, v, kv_stride); mode 1: paged bf16; mode 2: paged fp8
// (k_scale/v_scale may be null for unit scale).  cu_q has S+1 entries.
PRISM_API int prism_flash_attention(const void* q, long long q_stride, void* out, long long o_stride, const void* cu_q,
                                    const void* k, const void* v, long long kv_stride, const void* k_cache,
                                    const void* v_cache, const void* k_scale, const void* v_scale,
                                    const void* block_tables, const void* kv_lens, int max_blocks, int num_blocks,
                                    int page, int S, int max_q_len, int Hq, int Hkv, int hd, int mode, int causal,
                                    float scale, void* stream, int pdl) {
  if (S <= 0 || max_q_len <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  if (mode != 0 && (page <= 0 || max_blocks <= 0)) return -1;
  FlashArgs a;
  a.q = (const bf16*)q;
  a.q_stride = q_stride;
  a.out = (bf16*)out;
  a.o_stride = o_stride;
  a.cu_q = (const int*)cu_q;
  a.k = (const bf16*)k;
  a.v = (const bf16*)v;
  a.kv_stride = kv_stride;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.k_scale = (const float*)k_scale;
  a.v_scale = (const float*)v_scale;
  a.block_tables = (const int*)block_tables;
  a.kv_lens = (const int*)kv_lens;
  a.max_blocks = max_blocks;
  a.num_blocks = num_blocks;
  a.page = page;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.causal = causal;
  a.scale = scale;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (mode) {
    case 0: return dispatch_flash<0>(a, hd, max_q_len, S, s, pdl != 0);
    case 1: return dispatch_flash<1>(a, hd, max_q_len, S, s, pdl != 0);
    case 2: return dispatch_flash<2>(a, hd, max_q_len, S, s, pdl != 0);
  }
  return -3;
}

// =====================================================================================
// Allocation-free entry point (declared in prism_noalloc.h; it has no counterpart in the
// reference).  Same split-KV decode attention as prism_paged_decode, but the split
// partials live in a fixed file-scope device array instead of caller-provided scratch, so
// a caller that must not allocate device memory can still use the split-KV path.
// =====================================================================================
#include "prism_noalloc.h"

#include <cstdio>
#include <mutex>

namespace {

// Every GPU that loads this library keeps these bytes resident until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PRISM_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {nullptr};  // device address of the array, per device
std::mutex g_noalloc_mutex;
thread_local char g_noalloc_error[256] = "";

int noalloc_fail(int code, const char* msg) {
  snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s", msg);
  return code;
}

}  // namespace

PRISM_API const char* prism_noalloc_last_error() { return g_noalloc_error; }

PRISM_API long long prism_paged_decode_noalloc_scratch_bytes(int B, int Hq, int D, int nsplit) {
  if (nsplit > 32) nsplit = 32;  // the kernels never split a context more than 32 ways
  if (nsplit <= 1 || B <= 0 || Hq <= 0 || D <= 0) return 0;
  const long long rows = (long long)B * Hq * nsplit;
  const long long part_o = (rows * D * 4 + 255) / 256 * 256;
  return part_o + rows * 2 * 4;
}

PRISM_API int prism_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const void* k_scale,
                                         const void* v_scale, const void* block_tables, const void* context_lens,
                                         void* out, int B, int Hq, int Hkv, int D, int page, int max_blocks,
                                         int num_blocks, int nsplit, int kv_mode, float scale, void* stream) {
  g_noalloc_error[0] = 0;
  if (B <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0)
    return noalloc_fail(-13, "prism_paged_decode_noalloc: Hq and Hkv must be positive and Hq a multiple of Hkv");
  if (D != 64 && D != 128) return noalloc_fail(-14, "prism_paged_decode_noalloc: head dimension must be 64 or 128");
  if (page <= 0 || max_blocks <= 0)
    return noalloc_fail(-15, "prism_paged_decode_noalloc: page and max_blocks must be positive");
  if (kv_mode < 0 || kv_mode > 2) return noalloc_fail(-16, "prism_paged_decode_noalloc: kv_mode must be 0, 1 or 2");
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 32) nsplit = 32;  // as prism_paged_decode does, before the scratch is sized
  const long long need = prism_paged_decode_noalloc_scratch_bytes(B, Hq, D, nsplit);
  if (need > (long long)PRISM_NOALLOC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "prism_paged_decode_noalloc: B=%d Hq=%d D=%d nsplit=%d needs %lld bytes of split-KV scratch, the built-in "
             "array holds %lld; lower nsplit or the batch, or use prism_paged_decode with your own scratch",
             B, Hq, D, nsplit, need, (long long)PRISM_NOALLOC_SCRATCH_BYTES);
    return noalloc_fail(-10, msg);
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail((int)e, "prism_paged_decode_noalloc: cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices) return noalloc_fail(-11, "prism_paged_decode_noalloc: device index out of range");
  void* base = nullptr;
  {
    // One-time set-up per device, with that device current: the host-side name of a
    // __device__ array is not a device address, so it is resolved here and cached.
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || p == nullptr)
        return noalloc_fail(e != cudaSuccess ? (int)e : -12, "prism_paged_decode_noalloc: cudaGetSymbolAddress failed");
      g_noalloc_ptr[dev] = p;
    }
    base = g_noalloc_ptr[dev];
  }
  const long long rows = (long long)B * Hq * nsplit;
  void* part_o = base;
  void* part_ml = static_cast<unsigned char*>(base) + (rows * D * 4 + 255) / 256 * 256;
  // Every (sequence, head, split) cell of both partial arrays is rewritten by each launch
  // (empty splits store max = -inf, sum = 0), so nothing has to be cleared between calls.
  const int rc = prism_paged_decode(q, k_cache, v_cache, k_scale, v_scale, block_tables, context_lens,
                                    nsplit > 1 ? part_o : nullptr, nsplit > 1 ? part_ml : nullptr, out, nullptr, B, Hq, Hkv,
                                    D, page, max_blocks, num_blocks, nsplit, kv_mode, scale, 0, stream, 0);
  if (rc != 0) return noalloc_fail(rc, "prism_paged_decode_noalloc: kernel launch failed");
  return 0;
}
