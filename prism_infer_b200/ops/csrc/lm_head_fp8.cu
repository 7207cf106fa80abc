// Greedy next token from an E4M3 copy of the LM head, then an exact rerank of the candidates.
//
// The LM head is the largest matrix of a decode step (151936 x 4096 at 8B widths: 1.24 GB in
// bf16, 0.23 ms of a 3.85 ms step at 0.81 of the copy bandwidth).  The reference's fastest mode
// generates candidates from a row-scaled FP8 copy of the head and ranks them with the original
// bf16 rows in fp32 (prism_infer/models/qwen3_vl.py:1659-1722, `logits_precision=
// "selective_fp32"` with the FP8 candidate head; candidate search in
// prism_infer/ops/selective_topk.py:26-278).  Here that is two kernels:
//
//   lm_head_fp8_topk_kernel   streams the E4M3 rows once (half the bytes).  A warp owns the rows
//                             r = warp, warp + W, ...; per row the lanes split the columns.  E4M3
//                             bytes become fp16 bit patterns with two integer operations per pair
//                             (same sign / exponent / mantissa layout, exponent bias folded into
//                             the row scale): the conversion instructions run at a quarter of the
//                             ALU rate and would bound the kernel.  Sixteen products are summed in
//                             fp16 (HFMA2 against fp16 activations in shared memory), then in fp32.
//                             Lane b keeps the best CANDS_PER_WARP (value, row) pairs of batch
//                             row b.  Rows of one warp are spread over the whole
//                             vocabulary, so the exact winner is lost only if that many other rows
//                             of the same warp beat it under FP8 rounding.
//   lm_head_rerank_kernel     one warp per candidate: the exact fp32 dot product of the bf16 row
//                             with the activations; the best of each CTA goes to a short list
//                             that merge_candidates_kernel (sampler.cu) reduces with the lowest-id
//                             tie break.
//
// At most LMH_MAX_BATCH rows; larger batches and sampled rows use the bf16 head.
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(lm_head_fp8)

namespace {

typedef __nv_bfloat16 bf16;
constexpr int LMH_MAX_BATCH = 4;
constexpr int CANDS_PER_WARP = 2;
static_assert(CANDS_PER_WARP == 2, "the insertion below is written for two entries");
constexpr int TOPK_THREADS = 512;   // 16 warps per CTA, one CTA per SM
constexpr int MAX_SLOTS = 4;        // rows a warp keeps in flight in its shared-memory ring
constexpr int SMEM_BUDGET = 224 * 1024;

// Two E4M3 bytes -> two fp16 values scaled by 2^-8: an E4M3 byte shifted into the upper byte of a half has its
// sign in place and its exponent / mantissa one bit too high; fp16's exponent bias is 15, E4M3's is 7.  Subnormal
// codes map to fp16 subnormals with the same factor.  sel picks the two bytes (0x1404: bytes 0, 1; 0x3424: 2, 3).
__device__ __forceinline__ __half2 e4m3x2_as_half2(uint32_t word, uint32_t sel) {
  const uint32_t h = __byte_perm(word, 0u, sel);
  const uint32_t bits = (h & 0x80008000u) | ((h & 0x7f007f00u) >> 1);
  return *reinterpret_cast<const __half2*>(&bits);
}
constexpr float E4M3_AS_HALF_FACTOR = 256.0f;

// Shared memory: [activations fp16 B x H][row ring: warps x slots x H bytes][mbarriers warps x slots]
template <int B>
__global__ void __launch_bounds__(TOPK_THREADS, 1)
lm_head_fp8_topk_kernel(const uint8_t* __restrict__ w8, const float* __restrict__ wscale, const bf16* __restrict__ x, long long ldx,
                        int V, int H, int slots, float* __restrict__ cand_val, int* __restrict__ cand_id) {
  // [B][H] activations as fp16, permuted so that the eight halves a lane reads for its 16-byte weight group gi
  // and half q sit at uint4 index q * groups + gi: consecutive lanes read consecutive uint4s (no bank conflicts)
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int WARPS = TOPK_THREADS / 32;
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  uint8_t* ring = smem_raw + (((size_t)B * H * 2 + 127) & ~(size_t)127);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)WARPS * slots * H);
  const int groups = H >> 4;                       // 16-byte groups per row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps_total = gridDim.x * WARPS;
  const int gw = blockIdx.x * WARPS + warp;
  uint8_t* my_ring = ring + (size_t)warp * slots * H;
  uint64_t* my_bars = bars + warp * slots;
  if (lane == 0)
    for (int k = 0; k < slots; ++k) mbar_init(&my_bars[k], 1);
  fence_barrier_init();
  __syncwarp();
  // the weights do not depend on the previous kernel: the first rows are requested before the dependency wait
  auto request = [&](int r, int k) {  // lane 0: row r into slot k (one bulk copy of H bytes)
    mbar_expect_tx(&my_bars[k], (uint32_t)H);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(my_ring + (size_t)k * H)),
                 "l"(w8 + (size_t)r * H), "r"(H), "r"(smem_u32(&my_bars[k]))
                 : "memory");
  };
  if (lane == 0)
    for (int k = 0; k < slots; ++k) {
      const int r = gw + k * warps_total;
      if (r < V) request(r, k);
    }
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < B * H; i += TOPK_THREADS) {
    const int b = i / H, c = i - b * H;
    xs[(size_t)b * H + ((((c >> 3) & 1) * groups + (c >> 4)) << 3) + (c & 7)] = __float2half_rn(__bfloat162float(x[(size_t)b * ldx + c]));
  }
  __syncthreads();
  float best_v[CANDS_PER_WARP];
  int best_i[CANDS_PER_WARP];
#pragma unroll
  for (int k = 0; k < CANDS_PER_WARP; ++k) {
    best_v[k] = -INFINITY;
    best_i[k] = -1;
  }
  int slot = 0;
  uint32_t parity = 0;
  bool ok = true;
  for (int r = gw; r < V && ok; r += warps_total) {
    ok = mbar_wait(&my_bars[slot], parity, 1);   // bounded: reports and gives up instead of hanging
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint4* row = reinterpret_cast<const uint4*>(my_ring + (size_t)slot * H);
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.0f;
#pragma unroll 2
    for (int gi = lane; gi < groups; gi += 32) {
      const uint4 w4 = row[gi];
      const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
      __half2 wh[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        wh[2 * q] = e4m3x2_as_half2(wv[q], 0x1404u);
        wh[2 * q + 1] = e4m3x2_as_half2(wv[q], 0x3424u);
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)b * H) + gi;
        const uint4 x0 = xp[0], x1 = xp[groups];
        const __half2* h0 = reinterpret_cast<const __half2*>(&x0);
        const __half2* h1 = reinterpret_cast<const __half2*>(&x1);
        // two chains of four HFMA2 (eight products per half): short fp16 sums, then fp32
        __half2 s0 = __hmul2(wh[0], h0[0]), s1 = __hmul2(wh[4], h1[0]);
#pragma unroll
        for (int q = 1; q < 4; ++q) {
          s0 = __hfma2(wh[q], h0[q], s0);
          s1 = __hfma2(wh[4 + q], h1[q], s1);
        }
        const float2 f0 = __half22float2(s0), f1 = __half22float2(s1);
        acc[b] += (f0.x + f0.y) + (f1.x + f1.y);
      }
    }
    __syncwarp();  // every lane is done with the slot before it is requested again
    if (lane == 0) {
      const int r_next = r + slots * warps_total;
      if (r_next < V) request(r_next, slot);
    }
    const float scale = wscale[r] * E4M3_AS_HALF_FACTOR;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float s = warp_sum(acc[b]) * scale;  // every lane holds the sum
      if (lane == b) {  // insertion into the two-entry descending list
        if (s > best_v[0]) {
          best_v[1] = best_v[0];
          best_i[1] = best_i[0];
          best_v[0] = s;
          best_i[0] = r;
        } else if (s > best_v[1]) {
          best_v[1] = s;
          best_i[1] = r;
        }
      }
    }
    if (++slot == slots) {
      slot = 0;
      parity ^= 1;
    }
  }
  if (!ok && lane == 0) {
    // a wait ran out: rows still in flight must land before the shared memory is released
    for (int k = 0; k < slots; ++k) {
      const long long t0 = clock64();
      while (!mbar_try_wait(&my_bars[k], 0) && !mbar_try_wait(&my_bars[k], 1) && clock64() - t0 < 4000000ll) {
      }
    }
  }
  if (lane < B) {
    const size_t base = ((size_t)lane * warps_total + gw) * CANDS_PER_WARP;
#pragma unroll
    for (int k = 0; k < CANDS_PER_WARP; ++k) {
      cand_val[base + k] = best_v[k];
      cand_id[base + k] = best_i[k];
    }
  }
}

// One warp per candidate: exact fp32 dot product of the bf16 row with the activations; the CTA's
// best (value, id) per batch row goes to out_val / out_id [cta][B].
constexpr int RERANK_WARPS = 8;
__global__ void __launch_bounds__(RERANK_WARPS * 32)
lm_head_rerank_kernel(const bf16* __restrict__ w, long long ldw, const bf16* __restrict__ x, long long ldx, int H, int V,
                      const int* __restrict__ cand_id, int n_cand, int B, long long vocab_offset, float* __restrict__ out_val,
                      long long* __restrict__ out_id) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.y;
  const int c = blockIdx.x * RERANK_WARPS + warp;
  float v = -INFINITY;
  long long id = 0x7fffffffffffffffll;
  if (c < n_cand) {
    const int row = cand_id[(size_t)b * n_cand + c];
    if (row >= 0 && row < V) {
      const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)row * ldw);
      const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)b * ldx);
      float acc = 0.0f;
      for (int g = lane; g < (H >> 3); g += 32) {
        const uint4 wv = __ldg(wr + g), xv = __ldg(xr + g);
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __bfloat1622float2(wp[e]), d = __bfloat1622float2(xp[e]);
          acc += a.x * d.x + a.y * d.y;
        }
      }
      v = warp_sum(acc);
      id = (long long)row + vocab_offset;
    } else if (row >= V && lane == 0) {
      prism_report(PRISM_ERR_BOUNDS, row);
    }
  }
  __shared__ float sv[RERANK_WARPS];
  __shared__ long long si[RERANK_WARPS];
  if (lane == 0) {
    sv[warp] = v;
    si[warp] = id;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float best = -INFINITY;
    long long best_i = 0x7fffffffffffffffll;
#pragma unroll
    for (int k = 0; k < RERANK_WARPS; ++k)
      if (sv[k] > best || (sv[k] == best && si[k] < best_i)) {
        best = sv[k];
        best_i = si[k];
      }
    out_val[(size_t)blockIdx.x * B + b] = best;
    out_id[(size_t)blockIdx.x * B + b] = best_i;
  }
}

int g_sms = 0;
int sms() {
  if (g_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) g_sms = 148;
  }
  return g_sms;
}

}  // namespace

// Sizes of the scratch arrays the caller provides: out3 = {candidates per batch row, rerank CTAs per batch row,
// largest batch}.
PRISM_API int prism_lm_head_fp8_plan(int* out3) {
  const int n_cand = sms() * (TOPK_THREADS / 32) * CANDS_PER_WARP;
  out3[0] = n_cand;
  out3[1] = (n_cand + RERANK_WARPS - 1) / RERANK_WARPS;
  out3[2] = LMH_MAX_BATCH;
  return 0;
}

// w8 [V, H] E4M3 with fp32 row scales, w [V, H] bf16 (row stride ldw), x [B, H] bf16 (row stride ldx).
// cand_val / cand_id: [B][n_cand]; list_val / list_id: [rerank CTAs][B]: the caller reduces the list with
// prism_merge_candidates.  Ids get vocab_offset added.
PRISM_API int prism_lm_head_fp8_candidates(const void* w8, const void* wscale, const void* w, long long ldw, const void* x, long long ldx,
                                           int B, int V, int H, long long vocab_offset, void* cand_val, void* cand_id,
                                           void* list_val, void* list_id, void* stream, int pdl) {
  if (B < 1 || B > LMH_MAX_BATCH || V < 1 || H < 16 || H % 16 || H > 12288) return -1;
  if ((reinterpret_cast<uintptr_t>(w8) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) return -2;
  if ((ldw % 8) || (ldx % 8)) return -3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int plan[3];
  prism_lm_head_fp8_plan(plan);
  const int n_cand = plan[0], ctas = plan[1];
  const size_t xs_bytes = ((size_t)B * H * sizeof(__half) + 127) & ~(size_t)127;
  const size_t per_slot = (size_t)(TOPK_THREADS / 32) * H;
  if (xs_bytes + per_slot + 1024 > (size_t)SMEM_BUDGET) return -4;
  int slots = (int)((SMEM_BUDGET - 1024 - xs_bytes) / per_slot);
  if (slots > MAX_SLOTS) slots = MAX_SLOTS;
  const size_t smem = xs_bytes + per_slot * slots + (size_t)(TOPK_THREADS / 32) * slots * 8 + 128;
  int rc;
#define PRISM_LMH_CASE(B_)                                                                                                        \
  case B_: {                                                                                                                      \
    static bool configured = false;                                                                                               \
    if (!configured) {                                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(lm_head_fp8_topk_kernel<B_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);     \
      if (e != cudaSuccess) return (int)e;                                                                                        \
      configured = true;                                                                                                          \
    }                                                                                                                             \
    rc = (int)prism_launch(lm_head_fp8_topk_kernel<B_>, dim3(sms()), dim3(TOPK_THREADS), smem, s, pdl != 0, (const uint8_t*)w8,   \
                           (const float*)wscale, (const bf16*)x, ldx, V, H, slots, (float*)cand_val, (int*)cand_id);              \
    break;                                                                                                                        \
  }
  switch (B) {
    PRISM_LMH_CASE(1)
    PRISM_LMH_CASE(2)
    PRISM_LMH_CASE(3)
    PRISM_LMH_CASE(4)
    default:
      return -1;
  }
#undef PRISM_LMH_CASE
  if (rc) return rc;
  return (int)prism_launch(lm_head_rerank_kernel, dim3(ctas, B), dim3(RERANK_WARPS * 32), 0, s, pdl != 0, (const bf16*)w, ldw,
                           (const bf16*)x, ldx, H, V, (const int*)cand_id, n_cand, B, vocab_offset, (float*)list_val,
                           (long long*)list_id);
}
