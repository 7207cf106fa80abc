// Two-SM (cta_group::2) persistent GEMM for prefill-sized problems.
//
// A cluster of two CTAs computes one 256-token x 256-feature output tile per step with
// tcgen05.mma.cta_group::2 (M = 256 over the pair, N = 256).  Each CTA loads its own 128 token
// rows of the activations and only HALF of the 256-row weight tile; the tensor cores of both SMs
// read both halves.  Per CTA and 64-wide k-block that is 32 KB of operands instead of the 48 KB
// of the one-SM kernel: a third less L2 traffic per FLOP and a six-stage ring in the same shared
// memory.  The operand loads carry the cta_group::2 qualifier only (no cluster-wide fan-out of
// a load exists in this file); their completion is counted on the leader CTA's barrier.
//
// Roles per CTA: warp 0 TMA producer, warp 1 TMEM allocation and (leader CTA only) MMA issue,
// warps 2-5 epilogue over the CTA's own 128 accumulator lanes (tokens), with the row-major
// vectorised epilogues of gemm_wx_persistent_kernel (bias, GELU, residual; or SwiGLU over a
// [128 gate | 128 up] weight tile).  Barriers that cross the pair are addressed with mapa;
// tcgen05.commit signals the leader's and the peer's barrier with one instruction each.
// Every wait is bounded; both CTAs meet at a cluster barrier before they exit.
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(gemm_pair)

namespace {

constexpr int PBM = 128;   // token rows per CTA (256 per pair)
constexpr int PBN = 256;   // accumulator columns per tile
constexpr int PBK = 64;
constexpr int A_BYTES = PBM * PBK * 2;        // 16 KB
constexpr int B_HALF_BYTES = (PBN / 2) * PBK * 2;  // 16 KB: this CTA's half of the weight tile
constexpr int PSTAGE = A_BYTES + B_HALF_BYTES;     // 32 KB
constexpr int PAIR_THREADS = 192;
constexpr int PAIR_SMEM_LIMIT = 232448;

struct PairArgs {
  int T, M;            // tokens, features (dual: features of the output, the weight has 2 M rows)
  int kb_total;
  int stages;
  int m_tiles, n_tiles;  // pair tiles: 256 tokens x 256 accumulator columns
  int dual;            // B tile = 128 gate rows (CTA 0) | 128 up rows (CTA 1), epilogue = SwiGLU
  int w2_row_off;
  int act;
  int debug;           // 1: write the TMEM base address of each CTA to dbg[cta]
  long long ldo, ldr;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  unsigned int* dbg;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Operand load of one CTA of the pair; bar_cluster_addr is a shared::cluster address (the leader's barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once every earlier MMA of this thread is done) on a barrier given by its shared::cluster address.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// NBUF accumulators of 256 columns per CTA (2: the store loop of a tile overlaps the next
// tile's MMAs; 1 is the probe configuration).
template <int NBUF>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const PairArgs a) {
  constexpr int ACC_COLS = PBN;
  constexpr uint32_t IDESC = umma_idesc_bf16(2 * PBM, PBN);

  extern __shared__ uint8_t pair_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pair_raw) + 1023) & ~uintptr_t(1023));
  const int stages = a.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * PSTAGE);  // used in the leader only
  uint64_t* empty = full + stages;       // per CTA: stage free again
  uint64_t* acc_full = empty + stages;   // [2] per CTA: accumulator ready for this CTA's epilogue
  uint64_t* acc_empty = acc_full + 2;    // [2] leader only: 8 epilogue warps of the pair drained it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = a.m_tiles * a.n_tiles;
  const int num_kb = a.kb_total;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, ACC_COLS * NBUF);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything crosses the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (a.debug && threadIdx.x == 0) a.dbg[blockIdx.x] = tmem_base;
  pdl_launch_dependents();

  // pair tile -> first token row of the pair / first accumulator column (features fastest:
  // consecutive pairs share the activation tile)
#define PAIR_COORDS(tile_, m0_, n0_)                     \
  const int m0_ = ((tile_) / a.n_tiles) * (2 * PBM);     \
  const int n0_ = ((tile_) % a.n_tiles) * PBN;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer (both CTAs) ------------------------------
      pdl_wait();
      long long it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        PAIR_COORDS(tile, m0, n0)
        // weight rows of this CTA's half of the tile
        const int b_row = a.dual ? (rank == 0 ? n0 / 2 : a.w2_row_off + n0 / 2) : n0 + (int)rank * (PBN / 2);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % stages);
          const uint32_t round = (uint32_t)(it / stages);
          if (round > 0) {
            ok = mbar_wait(&empty[s], (round - 1) & 1, 1);
            if (!ok) break;
          }
          uint8_t* st = smem + (size_t)s * PSTAGE;
          const uint32_t full_leader = mapa_u32(smem_u32(&full[s]), 0);
          if (leader) mbar_expect_tx(&full[s], 2 * PSTAGE);  // both CTAs' bytes land on this barrier
          tma_load_2d_pair(st, &tmA, full_leader, kb * PBK, m0 + (int)rank * PBM);
          tma_load_2d_pair(st + A_BYTES, &tmB, full_leader, kb * PBK, b_row);
        }
      }
      // copies in flight keep this CTA's shared memory busy; the cluster barrier at the end is
      // reached only after the consumer side has finished or given up
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ------------------------------ MMA issuer (leader CTA) ------------------------------
      long long it = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int buf = local % NBUF;
        const uint32_t use = (uint32_t)(local / NBUF);
        if (use > 0) {
          ok = mbar_wait(&acc_empty[buf], (use - 1) & 1, 5);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t acc_addr = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % stages);
          ok = mbar_wait(&full[s], (uint32_t)(it / stages) & 1, 2);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + (size_t)s * PSTAGE);
          const uint64_t da = umma_desc_sw128(st);
          const uint64_t db = umma_desc_sw128(st + A_BYTES);
#pragma unroll
          for (int k = 0; k < PBK / 16; ++k) tc_mma_f16_pair(acc_addr, da + 2 * k, db + 2 * k, IDESC, (kb | k) != 0);
          // the stage is free in both CTAs once these MMAs have read it
          tc_commit_pair(mapa_u32(smem_u32(&empty[s]), 0));
          tc_commit_pair(mapa_u32(smem_u32(&empty[s]), 1));
        }
        if (ok) {
          tc_commit_pair(mapa_u32(smem_u32(&acc_full[buf]), 0));
          tc_commit_pair(mapa_u32(smem_u32(&acc_full[buf]), 1));
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps 2..5 (both CTAs) ------------------------------
    const int q = warp & 3;
    pdl_wait();
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const int buf = local % NBUF;
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (uint32_t)(local / NBUF) & 1, 3))) break;
      tc_fence_after();
      PAIR_COORDS(tile, m0, n0)
      const int m = m0 + (int)rank * PBM + q * 32 + lane;  // token row of this thread
      const bool m_ok = m < a.T;
      const uint32_t t_lane = tmem_base + buf * ACC_COLS + ((uint32_t)(q * 32) << 16);
      if (a.dual) {
        const int f_base = n0 / 2;
        const int f_valid = min(PBN / 2, a.M - f_base);
        for (int c0 = 0; c0 < f_valid; c0 += 16) {
          uint32_t rg[16], ru[16];
          tmem_ld16(t_lane + c0, rg);
          tmem_ld16(t_lane + PBN / 2 + c0, ru);
          tmem_ld_wait();
          if (!m_ok) continue;
          uint4 o[2];
          __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float g0 = bf16_round(__uint_as_float(rg[2 * e])), g1 = bf16_round(__uint_as_float(rg[2 * e + 1]));
            const float u0 = bf16_round(__uint_as_float(ru[2 * e])), u1 = bf16_round(__uint_as_float(ru[2 * e + 1]));
            op[e] = __floats2bfloat162_rn(bf16_round(silu(g0)) * u0, bf16_round(silu(g1)) * u1);
          }
          __nv_bfloat16* dst = a.out + (size_t)m * a.ldo + f_base + c0;
          *reinterpret_cast<uint4*>(dst) = o[0];
          *reinterpret_cast<uint4*>(dst + 8) = o[1];
        }
      } else {
        const int n_valid = min(PBN, a.M - n0);
        for (int c0 = 0; c0 < n_valid; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(t_lane + c0, r);
          tmem_ld_wait();
          if (!m_ok) continue;
          const int f0 = n0 + c0;
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
          if (a.bias != nullptr) {
            const uint4 b0 = *reinterpret_cast<const uint4*>(a.bias + f0), b1 = *reinterpret_cast<const uint4*>(a.bias + f0 + 8);
            const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&b0);
            const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&b1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x0 = __bfloat1622float2(p0[e]), x1 = __bfloat1622float2(p1[e]);
              v[2 * e] += x0.x;
              v[2 * e + 1] += x0.y;
              v[8 + 2 * e] += x1.x;
              v[8 + 2 * e + 1] += x1.y;
            }
          }
          if (a.act == 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_tanh(v[j]);
          } else if (a.act == 2) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_erf(v[j]);
          }
          if (a.residual != nullptr) {
            const __nv_bfloat16* rs = a.residual + (size_t)m * a.ldr + f0;
            const uint4 r0 = *reinterpret_cast<const uint4*>(rs), r1 = *reinterpret_cast<const uint4*>(rs + 8);
            const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&r0);
            const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x0 = __bfloat1622float2(p0[e]), x1 = __bfloat1622float2(p1[e]);
              v[2 * e] = bf16_round(v[2 * e]) + x0.x;
              v[2 * e + 1] = bf16_round(v[2 * e + 1]) + x0.y;
              v[8 + 2 * e] = bf16_round(v[8 + 2 * e]) + x1.x;
              v[8 + 2 * e + 1] = bf16_round(v[8 + 2 * e + 1]) + x1.y;
            }
          }
          uint4 o[2];
          __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
          for (int e = 0; e < 8; ++e) op[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
          __nv_bfloat16* dst = a.out + (size_t)m * a.ldo + f0;
          *reinterpret_cast<uint4*>(dst) = o[0];
          *reinterpret_cast<uint4*>(dst + 8) = o[1];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[buf]), 0));
    }
  }
#undef PAIR_COORDS
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still address this CTA's barriers and shared memory until here
  if (warp == 1) tmem_dealloc2(tmem_base, ACC_COLS * NBUF);
}

int g_pair_sms = 0;

}  // namespace

// out[t][f] = act(X[t] . W[f] + bias[f]) (+ residual[t][f]), or with dual the SwiGLU of a packed
// [2 M, K] weight (second matrix at row w2_row_off).  X [T, K] (ldx), W [rows, K] (ldw), bf16;
// M a multiple of 16; bias / residual / out rows 16-byte aligned.  accumulators: 1 or 2 TMEM accumulators per
// CTA.  debug_out (may be null, else one u32 per CTA of the grid) receives each CTA's TMEM base address.
PRISM_API int prism_gemm_pair(const void* W, const void* X, void* out, int M, int T, int K, long long ldw, long long ldx,
                              long long ldo, int w_rows_total, const void* bias, const void* residual, long long ldr,
                              int act, int dual, int w2_row_off, int accumulators, void* debug_out, void* stream, int pdl) {
  if (T <= 0 || M <= 0 || K <= 0) return 0;
  if ((M % 16) || (ldo % 8) || (residual != nullptr && (ldr % 8))) return -1;
  const unsigned long long addr = reinterpret_cast<unsigned long long>(out) | reinterpret_cast<unsigned long long>(bias) |
                                  reinterpret_cast<unsigned long long>(residual);
  if (addr & 15ull) return -2;
  if (dual && (bias != nullptr || residual != nullptr || act != 0)) return -3;
  CUtensorMap ta, tb;
  int rc = prism_get_tensor_map(X, (unsigned long long)T, (unsigned long long)K, (unsigned long long)ldx, PBM, &ta);
  if (rc) return rc;
  rc = prism_get_tensor_map(W, (unsigned long long)w_rows_total, (unsigned long long)K, (unsigned long long)ldw, PBN / 2, &tb);
  if (rc) return rc;
  PairArgs a;
  a.T = T;
  a.M = M;
  a.kb_total = (K + PBK - 1) / PBK;
  a.m_tiles = (T + 2 * PBM - 1) / (2 * PBM);
  a.n_tiles = dual ? (M + PBN / 2 - 1) / (PBN / 2) : (M + PBN - 1) / PBN;
  a.dual = dual;
  a.w2_row_off = w2_row_off;
  a.act = act;
  a.debug = debug_out != nullptr;
  a.ldo = ldo;
  a.ldr = ldr;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.dbg = reinterpret_cast<unsigned int*>(debug_out);
  int stages = (PAIR_SMEM_LIMIT - 1024 - 512) / PSTAGE;
  if (stages > 12) stages = 12;
  a.stages = stages;
  const size_t smem = (size_t)stages * PSTAGE + 1024 + (2 * stages + 4) * 8 + 64;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_LIMIT);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_LIMIT);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (g_pair_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_pair_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      g_pair_sms = 148;
  }
  const int tiles = a.m_tiles * a.n_tiles;
  int pairs = g_pair_sms / 2;
  if (pairs > tiles) pairs = tiles;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (accumulators == 1)
    return (int)prism_launch(gemm_pair_kernel<1>, dim3(2 * pairs), dim3(PAIR_THREADS), smem, st, pdl != 0, ta, tb, a);
  return (int)prism_launch(gemm_pair_kernel<2>, dim3(2 * pairs), dim3(PAIR_THREADS), smem, st, pdl != 0, ta, tb, a);
}
