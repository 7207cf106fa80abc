// Persistent decode kernel: every decoder layer of one decode step (at most 16 tokens) in ONE
// launch.
//
// The per-layer chain of the reference (prism_infer/models/qwen3_vl.py:925-1022 under
// prism_infer/engine/model_runner.py:1219-1313) is add+RMSNorm -> QKV GEMM -> QK-norm + M-RoPE +
// KV store -> paged attention -> o_proj -> add+RMSNorm -> gate/up GEMM + SwiGLU -> down_proj: eight
// launches per layer even when every op is one kernel, each of which pays launch, TMEM
// allocation, barrier set-up and the first TMA round trip, while a decode step is nothing but one
// pass over the weights.  Here one CTA per SM stays resident for the whole step:
//
//   warp 0 (one thread)   TMA producer.  Walks the CTA's static list of (layer, GEMM, k-block)
//                         work items and keeps the shared-memory operand ring full.  Weight tiles
//                         never depend on activations, so it runs ahead across phase and layer
//                         boundaries; only the 2 KB activation tile of a stage waits for the phase
//                         that produces it.
//   warp 1 (one thread)   tcgen05.mma issuer; accumulators rotate through four 16-column TMEM
//                         buffers so the issuer never waits for an epilogue.
//   warps 2..9 (workers)  epilogues (TMEM -> fp32 partial slabs) and every pointwise / attention
//                         phase, separated by grid-wide barriers.
//
// GEMM work is split stream-K style: the (weight tile, k-block) units of a GEMM are cut into
// gridDim.x equal contiguous runs, so every SM streams the same number of weight bytes whatever
// the matrix shape.  A run that crosses a tile boundary produces one partial per tile; the slab a
// partial lands in and the number of slabs of a tile follow from the same arithmetic on the
// consumer side, so sums are taken in a fixed order (no atomics, deterministic).
//
// RMSNorm is folded around the GEMMs: the phase that sums the previous projection's slabs writes
// the new residual, the unnormalised activation bf16(residual * weight) and per-segment sums of
// squares; the row's 1/rms is a per-token scalar and is applied by the consumer of the next
// GEMM's slabs.  The norm therefore costs no barrier of its own.
//
// Phases of a layer (B = grid barrier):
//   reduce(down slabs of the previous layer | embedding) -> residual, xw, ssq          B
//   QKV GEMM -> slabs                                                                   B
//   per (sequence, KV head, split): q/k/v rows from the slabs (1/rms, QK-norm, M-RoPE), KV store
//     of the new token, split-KV attention over the pages, last split merges -> attn    B
//   o_proj GEMM -> slabs                                                                B
//   reduce(o slabs) -> residual, xw, ssq                                                B
//   gate/up GEMM -> slabs                                                               B
//   SwiGLU(1/rms * slabs) -> act                                                        B
//   down GEMM -> slabs                                                                  B
// and a final reduce that leaves the pre-norm hidden state for the LM head path.
//
// Every wait is bounded.  A wait that runs out sets a global abort word that all other waits
// poll, records the status word and lets the kernel unwind (copies in flight are awaited, TMEM
// is freed); nothing traps and nothing hangs.
#include <cstring>
#include <mutex>

#include "common.cuh"

PRISM_DEFINE_TU_STATUS(decode_layers)

namespace {

typedef __nv_bfloat16 bf16;

constexpr int BM = 128, BK = 64, BN = 16, UMMA_K = 16;
constexpr int W_TILE_BYTES = BM * BK * 2;   // 16 KB
constexpr int X_TILE_BYTES = BN * BK * 2;   // 2 KB
constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
constexpr int NW = 8;                        // worker warps
constexpr int NWT = NW * 32;                 // worker threads
constexpr int NTHREADS = 64 + NWT;
constexpr int NACC = 4;                      // TMEM accumulators (16 fp32 columns each)
constexpr int TMEM_COLS = 64;
constexpr int MAX_T = 16;
constexpr int SCRATCH_BYTES = 24 * 1024;
constexpr int SMEM_LIMIT = 232448;
constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN);
constexpr float FP8_MAX = 448.0f;
constexpr float FP8_SCALE_FLOOR = 1.0e-6f;
constexpr long long UNWIND_CYCLES = 4000000ll;  // in-flight copies land within microseconds

struct alignas(64) LayerDesc {
  CUtensorMap tm_w[4];  // qkv, o, gate_up, down: [rows, K] bf16, box 128 x 64, 128-byte swizzle
  const bf16* norm_in;
  const bf16* norm_post;
  const bf16* q_norm;
  const bf16* k_norm;
  void* k_cache;
  void* v_cache;
  float* k_scale;
  float* v_scale;
};
static_assert(sizeof(LayerDesc) == 576, "LayerDesc layout is mirrored by the Python side");

struct GemmGeo {
  int M;         // weight rows (output features)
  int m_tiles;   // ceil(M / 128)
  int kb;        // k-blocks per tile (K / 64)
  int U;         // m_tiles * kb
  long long slab_stride;  // floats between slabs (T * M)
  float* part;   // [P][T][M]
};

struct DLParams {
  const LayerDesc* layers;
  int n_layers;
  int T;
  int H, Hq, Hkv, I;
  int page, max_blocks, num_blocks, kv_mode;
  int nsplit;
  int stages;
  float eps, attn_scale;
  GemmGeo geo[4];
  const bf16* x0;            // [T][H] embedding rows
  const int* positions;      // [3][T]
  const long long* slots;    // [T]
  const int* block_tables;   // [T][max_blocks]
  const int* context_lens;   // [T]
  const float* inv_freq;     // [D/2]
  const int* axis;           // [D/2]
  bf16* residual;            // [T][H] running residual (output: pre-norm hidden state)
  bf16* xw;                  // [T][H]
  bf16* attn;                // [T][Hq*D]
  bf16* act;                 // [T][I]
  float* ssq;                // [2][MAX_T][32]
  float* part_o;             // [T][Hq][nsplit][D]
  float* part_ml;            // [T][Hq][nsplit][2]
  int* attn_counters;        // [T*Hkv], zero, self-resetting
  unsigned long long* gbar;  // grid barrier ticket counter (monotonic)
  int* abort_flag;           // zero; set when a wait ran out
};

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ float b2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float2 fp8x2_to_float2(unsigned short v) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
__device__ __forceinline__ float fp8_to_float(__nv_fp8_storage_t v) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// ---- stream-K arithmetic (identical on the producing and the consuming side) -----------------
// U * (G + 1) stays below 2^31 (checked on the host), so 32-bit arithmetic is exact.
__host__ __device__ __forceinline__ int sk_start(int c, int U, int G) { return (int)((unsigned)c * (unsigned)U / (unsigned)G); }
__host__ __device__ __forceinline__ int sk_owner(int u, int U, int G) {
  return (int)(((unsigned)(u + 1) * (unsigned)G - 1u) / (unsigned)U);
}
// first contributing CTA and number of slabs of weight tile m
__device__ __forceinline__ void sk_tile_slabs(const GemmGeo& g, int m, int G, int& first, int& n) {
  const int u0 = m * g.kb;
  first = sk_owner(u0, g.U, G);
  n = sk_owner(u0 + g.kb - 1, g.U, G) - first + 1;
}

// ---- abort-aware bounded waits --------------------------------------------------------------------
__device__ __forceinline__ bool aborted(const DLParams& p) { return *reinterpret_cast<volatile int*>(p.abort_flag) != 0; }
__device__ __forceinline__ void raise_abort(const DLParams& p, int code, int tag) {
  atomicExch(p.abort_flag, 1);
  prism_report(code, tag);
}
__device__ __forceinline__ bool mbar_wait_a(uint64_t* bar, uint32_t parity, const DLParams& p, int tag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (aborted(p)) return false;
    if (clock64() - t0 > PRISM_WAIT_CYCLES) {
      raise_abort(p, PRISM_ERR_MBAR_TIMEOUT, tag);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait_short(uint64_t* bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity))
    if (clock64() - t0 > UNWIND_CYCLES) return false;
  return true;
}

// Grid-wide barrier over the worker threads of every CTA.  Tickets of a monotonic 64-bit counter:
// the k-th barrier since the buffer was created owns tickets [k G, (k+1) G), so no reset and no
// launch-dependent base are needed.  Pattern: CTA barrier, fence + ticket by one thread, spin,
// fence, CTA barrier (the cooperative-groups grid sync).  Returns false when aborted.
__device__ __forceinline__ void st_release_cta(volatile int* addr, int v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(const_cast<int*>(addr))), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cta(volatile int* addr) {
  int v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(const_cast<int*>(addr))) : "memory");
  return v;
}
__device__ __forceinline__ bool grid_barrier(const DLParams& p, int wtid, volatile int* s_abort, volatile int* s_xphase,
                                             int xphase_value) {
  named_bar_sync(1, NWT);
  if (wtid == 0) {
    __threadfence();
    const unsigned long long G = gridDim.x;
    bool ok = !aborted(p);  // after an abort nobody waits for anybody any more
    const unsigned long long ticket = ok ? atomicAdd(p.gbar, 1ull) : 0ull;
    const unsigned long long target = (ticket / G + 1ull) * G;
    const long long t0 = clock64();
    while (ok) {
      unsigned long long v;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.gbar) : "memory");
      if (v >= target) break;
      if (aborted(p)) {
        ok = false;
        break;
      }
      if (clock64() - t0 > PRISM_WAIT_CYCLES) {
        raise_abort(p, PRISM_ERR_PEER_TIMEOUT, 900);
        ok = false;
        break;
      }
    }
    __threadfence();
    if (!ok) *s_abort = 1;
    else if (xphase_value > 0) st_release_cta(s_xphase, xphase_value);  // the producer may now load this phase's activations
  }
  named_bar_sync(1, NWT);
  return *s_abort == 0;
}

// ---- reduce phase: slabs (+ residual) -> residual, xw = bf16(residual * weight), ssq ---------------
// One warp per (token, 256-column segment); a lane owns 8 columns.
__device__ __forceinline__ void reduce_phase(const DLParams& p, const GemmGeo* src, const bf16* x0, const bf16* weight,
                                             bool have_residual, float* ssq_out, bool final_only, int wtid) {
  const int G = gridDim.x, cta = blockIdx.x;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int H = p.H, nseg = (H + 255) / 256;
  const int items = p.T * nseg;
  for (int it = cta + G * warp; it < items; it += G * NW) {
    const int t = it / nseg, seg = it % nseg;
    const int col = seg * 256 + lane * 8;
    float ss = 0.0f;
    if (col < H) {
      float d[8];
      if (src != nullptr) {
        int first, n;
        sk_tile_slabs(*src, col / BM, G, first, n);
        float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
        const float* base = src->part + (size_t)t * src->M + col;
        for (int s = 0; s < n; ++s) {
          const float4 v0 = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * src->slab_stride));
          const float4 v1 = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * src->slab_stride + 4));
          a0.x += v0.x; a0.y += v0.y; a0.z += v0.z; a0.w += v0.w;
          a1.x += v1.x; a1.y += v1.y; a1.z += v1.z; a1.w += v1.w;
        }
        d[0] = bf16_round(a0.x); d[1] = bf16_round(a0.y); d[2] = bf16_round(a0.z); d[3] = bf16_round(a0.w);
        d[4] = bf16_round(a1.x); d[5] = bf16_round(a1.y); d[6] = bf16_round(a1.z); d[7] = bf16_round(a1.w);
      } else {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(x0 + (size_t)t * H + col));
        const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          d[2 * e] = b2f(v[e].x);
          d[2 * e + 1] = b2f(v[e].y);
        }
      }
      bf16* res = p.residual + (size_t)t * H + col;
      if (have_residual) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(res));
        const __nv_bfloat162* r = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          d[2 * e] = bf16_round(b2f(r[e].x) + d[2 * e]);
          d[2 * e + 1] = bf16_round(b2f(r[e].y) + d[2 * e + 1]);
        }
      }
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) op[e] = __floats2bfloat162_rn(d[2 * e], d[2 * e + 1]);
      *reinterpret_cast<uint4*>(res) = o;
      if (!final_only) {
        const uint4 wraw = __ldg(reinterpret_cast<const uint4*>(weight + col));
        const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&wraw);
        uint4 xo;
        __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xo);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          xp[e] = __floats2bfloat162_rn(d[2 * e] * b2f(w[e].x), d[2 * e + 1] * b2f(w[e].y));
          ss += d[2 * e] * d[2 * e] + d[2 * e + 1] * d[2 * e + 1];
        }
        *reinterpret_cast<uint4*>(p.xw + (size_t)t * H + col) = xo;
      }
    }
    if (!final_only) {
      ss = warp_sum(ss);
      if (lane == 0) ssq_out[t * 32 + seg] = ss;
    }
  }
  fence_proxy_async_global();  // xw is read by TMA (async proxy) after the barrier
}

// 1/rms of every token from the per-segment sums of squares -> shared memory
__device__ __forceinline__ void load_rstd(const DLParams& p, const float* ssq, float* s_rstd, int wtid) {
  const int warp = wtid >> 5, lane = wtid & 31;
  const int nseg = (p.H + 255) / 256;
  for (int t = warp; t < p.T; t += NW) {
    float v = lane < nseg ? __ldcg(ssq + t * 32 + lane) : 0.0f;
    v = warp_sum(v);
    if (lane == 0) s_rstd[t] = rsqrtf(v / (float)p.H + p.eps);
  }
  named_bar_sync(1, NWT);
}

// ---- SwiGLU phase: act = bf16(bf16(silu(bf16(rstd * sum gate))) * bf16(rstd * sum up)) -------------
__device__ __forceinline__ void swiglu_phase(const DLParams& p, const float* s_rstd, int wtid) {
  const int G = gridDim.x, cta = blockIdx.x;
  const int warp = wtid >> 5, lane = wtid & 31;
  const GemmGeo& g = p.geo[2];
  const int I = p.I, nseg = (I + 255) / 256;
  const int items = p.T * nseg;
  for (int it = cta + G * warp; it < items; it += G * NW) {
    const int t = it / nseg, seg = it % nseg;
    const int col = seg * 256 + lane * 8;
    if (col >= I) continue;
    const float rstd = s_rstd[t];
    float sum[2][8];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int c = half * I + col;
      int first, n;
      sk_tile_slabs(g, c / BM, G, first, n);
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
      const float* base = g.part + (size_t)t * g.M + c;
      for (int s = 0; s < n; ++s) {
        const float4 v0 = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * g.slab_stride));
        const float4 v1 = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * g.slab_stride + 4));
        a0.x += v0.x; a0.y += v0.y; a0.z += v0.z; a0.w += v0.w;
        a1.x += v1.x; a1.y += v1.y; a1.z += v1.z; a1.w += v1.w;
      }
      sum[half][0] = a0.x; sum[half][1] = a0.y; sum[half][2] = a0.z; sum[half][3] = a0.w;
      sum[half][4] = a1.x; sum[half][5] = a1.y; sum[half][6] = a1.z; sum[half][7] = a1.w;
    }
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g0 = bf16_round(sum[0][2 * e] * rstd), g1 = bf16_round(sum[0][2 * e + 1] * rstd);
      const float u0 = bf16_round(sum[1][2 * e] * rstd), u1 = bf16_round(sum[1][2 * e + 1] * rstd);
      op[e] = __floats2bfloat162_rn(bf16_round(silu(g0)) * u0, bf16_round(silu(g1)) * u1);
    }
    *reinterpret_cast<uint4*>(p.act + (size_t)t * I + col) = o;
  }
  fence_proxy_async_global();
}

// ---- attention phase ---------------------------------------------------------------------------
struct AttnScratch {
  float rstd[MAX_T];
  float q[512];          // [GQ][D] bf16 values as floats
  float kn[128], vn[128];  // the new token's K / V as attention sees them (dequantised payload)
  float kv_scale[2];
  float m[NW][8], l[NW][8];
  float acc[NW * 512];   // [NW][GQ][D]
  float coef[8][32];
  float inv[8];
  int last;
};
static_assert(sizeof(AttnScratch) <= SCRATCH_BYTES, "worker scratch");

// One (sequence, KV head, split) item on all worker warps.
template <int D, int GQ, bool KV8>
__device__ __noinline__ void attn_item(const DLParams& p, const LayerDesc& L, AttnScratch& sc, int b, int kvh, int split,
                                       int wtid) {
  constexpr int EPL = KV8 ? 16 : 8;
  constexpr int LPT = D / EPL;
  constexpr int TPW = 32 / LPT;
  constexpr int UNR = 2;
  constexpr int PER = D / 64;
  const int G = gridDim.x;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int slot_in_warp = lane / LPT, part = lane % LPT;
  int ctx = p.context_lens[b];
  {
    const long long reach = (long long)p.max_blocks * p.page;
    if ((long long)ctx > reach) {
      if (wtid == 0) prism_report(PRISM_ERR_BOUNDS, 1);
      ctx = (int)reach;
    }
    if (ctx < 0) ctx = 0;
  }
  constexpr int QUANT = TPW * NW * UNR;
  const int per_split = ((ctx + p.nsplit - 1) / p.nsplit + QUANT - 1) / QUANT * QUANT;
  const int j_begin = split * per_split;
  const int j_end = min(ctx, j_begin + per_split);
  const bool owner = ctx > 0 && ctx - 1 >= j_begin && ctx - 1 < j_begin + per_split;  // this split sees the new token
  const float rstd = sc.rstd[b];
  const GemmGeo& gq = p.geo[0];

  // ---- rows of the packed QKV projection this item needs: GQ query heads (+ K and V of the new token)
  const int nrows = GQ + (owner ? 2 : 0);
  for (int r = warp; r < nrows; r += NW) {
    const bool is_q = r < GQ, is_k = r == GQ;
    const int h = is_q ? kvh * GQ + r : (is_k ? p.Hq + kvh : p.Hq + p.Hkv + kvh);
    const int col0 = h * D;
    int first, n;
    sk_tile_slabs(gq, col0 / BM, G, first, n);
    const float* base = gq.part + (size_t)b * gq.M + col0;
    float lo[PER], hi[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane + 32 * j;
      float s0 = 0.0f, s1 = 0.0f;
      for (int s = 0; s < n; ++s) {
        s0 += __ldcg(base + (size_t)s * gq.slab_stride + i);
        s1 += __ldcg(base + (size_t)s * gq.slab_stride + i + D / 2);
      }
      lo[j] = bf16_round(s0 * rstd);
      hi[j] = bf16_round(s1 * rstd);
    }
    if (is_q || is_k) {
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < PER; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
      ss = warp_sum(ss);
      const float hr = rsqrtf(ss / (float)D + p.eps);
      const bf16* w = is_q ? L.q_norm : L.k_norm;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + 32 * j;
        lo[j] = bf16_round(bf16_round(lo[j] * hr) * b2f(w[i]));
        hi[j] = bf16_round(bf16_round(hi[j] * hr) * b2f(w[i + D / 2]));
      }
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + 32 * j;
        const float pos = (float)p.positions[(size_t)p.axis[i] * p.T + b];
        float sn, cs;
        sincosf(pos * p.inv_freq[i], &sn, &cs);
        sn = bf16_round(sn);
        cs = bf16_round(cs);
        const float x0 = lo[j], x1 = hi[j];
        lo[j] = bf16_round(bf16_round(x0 * cs) + bf16_round(-x1 * sn));
        hi[j] = bf16_round(bf16_round(x1 * cs) + bf16_round(x0 * sn));
      }
    }
    if (is_q) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        sc.q[r * D + lane + 32 * j] = lo[j];
        sc.q[r * D + lane + 32 * j + D / 2] = hi[j];
      }
      continue;
    }
    // K or V of the new token: quantise as the cache stores it, keep what attention will see
    float* keep = is_k ? sc.kn : sc.vn;
    const long long slot = p.slots[b];
    long long blk = slot >= 0 ? slot / p.page : -1;
    if (blk >= 0 && p.num_blocks > 0 && blk >= p.num_blocks) {
      if (lane == 0) prism_report(PRISM_ERR_BOUNDS, 3);
      blk = -1;
    }
    const size_t row = blk >= 0 ? ((size_t)blk * p.Hkv + kvh) * p.page + (size_t)(slot % p.page) : 0;
    void* cache = is_k ? L.k_cache : L.v_cache;
    if (p.kv_mode == 0) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + 32 * j;
        keep[i] = lo[j];
        keep[i + D / 2] = hi[j];
        if (blk >= 0) {
          bf16* dst = reinterpret_cast<bf16*>(cache) + row * D;
          dst[i] = __float2bfloat16_rn(lo[j]);
          dst[i + D / 2] = __float2bfloat16_rn(hi[j]);
        }
      }
      if (lane == 0) sc.kv_scale[is_k ? 0 : 1] = 1.0f;
    } else {
      float scale = 1.0f;
      if (p.kv_mode == 2) {
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; ++j) am = fmaxf(am, fmaxf(fabsf(lo[j]), fabsf(hi[j])));
        am = warp_max(am);
        scale = fmaxf(am / FP8_MAX, FP8_SCALE_FLOOR);
        if (lane == 0 && blk >= 0) (is_k ? L.k_scale : L.v_scale)[row] = scale;
      }
      if (lane == 0) sc.kv_scale[is_k ? 0 : 1] = scale;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + 32 * j;
        const __nv_fp8_storage_t c0 = __nv_cvt_float_to_fp8(fminf(fmaxf(lo[j] / scale, -FP8_MAX), FP8_MAX), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8_storage_t c1 = __nv_cvt_float_to_fp8(fminf(fmaxf(hi[j] / scale, -FP8_MAX), FP8_MAX), __NV_SATFINITE, __NV_E4M3);
        keep[i] = fp8_to_float(c0);
        keep[i + D / 2] = fp8_to_float(c1);
        if (blk >= 0) {
          __nv_fp8_storage_t* dst = reinterpret_cast<__nv_fp8_storage_t*>(cache) + row * D;
          dst[i] = c0;
          dst[i + D / 2] = c1;
        }
      }
    }
  }
  named_bar_sync(1, NWT);

  // ---- split-KV attention over the cached tokens [j_begin, j_stop) ------------------------------------
  float q[GQ][EPL];
#pragma unroll
  for (int g = 0; g < GQ; ++g)
#pragma unroll
    for (int e = 0; e < EPL; ++e) q[g][e] = sc.q[g * D + part * EPL + e] * p.attn_scale;
  float m[GQ], l[GQ], acc[GQ][EPL];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
  }
  const int* bt = p.block_tables + (size_t)b * p.max_blocks;
  const int j_stop = owner ? min(j_end, ctx - 1) : j_end;  // the new token comes from shared memory

  auto fold = [&](const float (&kf)[EPL], const float (&vf)[EPL], float ks, float vs, bool valid) {
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      float s = 0.0f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) s += q[g][e] * kf[e];
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (valid) {
        s *= ks;
        const float mn = fmaxf(m[g], s);
        const float corr = __expf(m[g] - mn);
        const float pr = __expf(s - mn);
        l[g] = l[g] * corr + pr;
        const float pv = pr * vs;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + pv * vf[e];
        m[g] = mn;
      }
    }
  };

  for (int j0 = j_begin + warp * TPW * UNR; j0 < j_stop; j0 += TPW * NW * UNR) {
    uint4 kr[UNR], vr[UNR];
    float ks[UNR], vs[UNR];
    bool valid[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int j = j0 + u * TPW + slot_in_warp;
      int blk = -1;
      if (j < j_stop) {
        blk = bt[j / p.page];
        if (p.num_blocks > 0 && blk >= p.num_blocks) {
          prism_report(PRISM_ERR_BOUNDS, 2);
          blk = -1;
        }
      }
      valid[u] = blk >= 0;
      kr[u] = make_uint4(0, 0, 0, 0);
      vr[u] = make_uint4(0, 0, 0, 0);
      ks[u] = 1.0f;
      vs[u] = 1.0f;
      if (valid[u]) {
        const size_t row = ((size_t)blk * p.Hkv + kvh) * p.page + (j % p.page);
        const size_t off = row * D * (KV8 ? 1 : 2) + (size_t)part * 16;
        kr[u] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(L.k_cache) + off));
        vr[u] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(L.v_cache) + off));
        if (KV8 && p.kv_mode == 2) {
          ks[u] = __ldcg(L.k_scale + row);
          vs[u] = __ldcg(L.v_scale + row);
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
      fold(kf, vf, ks[u], vs[u], valid[u]);
    }
  }
  if (owner && warp == 0) {  // the new token, from shared memory (token slot 0 of warp 0)
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kf[e] = sc.kn[part * EPL + e];
      vf[e] = sc.vn[part * EPL + e];
    }
    fold(kf, vf, sc.kv_scale[0], sc.kv_scale[1], slot_in_warp == 0);
  }
  // merge the token slots of a warp
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
#pragma unroll
    for (int o = LPT; o < 32; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float lo2 = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo);
      const float c0 = (m[g] == -INFINITY) ? 0.0f : __expf(m[g] - mn);
      const float c1 = (mo == -INFINITY) ? 0.0f : __expf(mo - mn);
      l[g] = l[g] * c0 + lo2 * c1;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
        acc[g][e] = acc[g][e] * c0 + ao * c1;
      }
      m[g] = mn;
    }
  }
  if (slot_in_warp == 0) {
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      if (part == 0) {
        sc.m[warp][g] = m[g];
        sc.l[warp][g] = l[g];
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) sc.acc[(warp * GQ + g) * D + part * EPL + e] = acc[g][e];
    }
  }
  named_bar_sync(1, NWT);
  const int ns = p.nsplit;
  for (int idx = wtid; idx < GQ * D; idx += NWT) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, sc.m[w][g]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float c = (sc.m[w][g] == -INFINITY) ? 0.0f : __expf(sc.m[w][g] - mm);
      ll += sc.l[w][g] * c;
      oo += sc.acc[(w * GQ + g) * D + d] * c;
    }
    const int hq = kvh * GQ + g;
    if (ns == 1) {
      p.attn[((size_t)b * p.Hq + hq) * D + d] = __float2bfloat16_rn(ll > 0.0f ? oo / ll : 0.0f);
    } else {
      const size_t pidx = ((size_t)b * p.Hq + hq) * ns + split;
      p.part_o[pidx * D + d] = oo;
      if (d == 0) {
        p.part_ml[pidx * 2] = mm;
        p.part_ml[pidx * 2 + 1] = ll;
      }
    }
  }
  if (ns > 1) {
    // the last split of this (sequence, KV head) to finish merges all of them
    __threadfence();
    named_bar_sync(1, NWT);
    if (wtid == 0) {
      const int old = atomicAdd(&p.attn_counters[b * p.Hkv + kvh], 1);
      sc.last = (old == ns - 1);
      if (sc.last) p.attn_counters[b * p.Hkv + kvh] = 0;
    }
    named_bar_sync(1, NWT);
    if (sc.last) {
      __threadfence();
      for (int g = warp; g < GQ; g += NW) {
        const size_t bh = (size_t)b * p.Hq + kvh * GQ + g;
        const float ms = lane < ns ? __ldcg(&p.part_ml[(bh * ns + lane) * 2]) : -INFINITY;
        const float ls = lane < ns ? __ldcg(&p.part_ml[(bh * ns + lane) * 2 + 1]) : 0.0f;
        const float mm = warp_max(ms);
        const float c = (ms == -INFINITY) ? 0.0f : __expf(ms - mm);
        const float ll = warp_sum(ls * c);
        sc.coef[g][lane] = c;
        if (lane == 0) sc.inv[g] = ll > 0.0f ? 1.0f / ll : 0.0f;
      }
      named_bar_sync(1, NWT);
      for (int idx = wtid; idx < GQ * D; idx += NWT) {
        const int g = idx / D, d = idx % D;
        const size_t bh = (size_t)b * p.Hq + kvh * GQ + g;
        const float* po = p.part_o + bh * ns * D + d;
        float oo = 0.0f;
        for (int s = 0; s < ns; ++s) oo += __ldcg(po + (size_t)s * D) * sc.coef[g][s];
        p.attn[bh * D + d] = __float2bfloat16_rn(oo * sc.inv[g]);
      }
    }
  }
  named_bar_sync(1, NWT);  // scratch is reused by the next item
}

template <int D>
__device__ __forceinline__ void attn_phase(const DLParams& p, const LayerDesc& L, AttnScratch& sc, int wtid) {
  const int G = gridDim.x;
  const int GQ = p.Hq / p.Hkv;
  const int items = p.T * p.Hkv * p.nsplit;
  const bool kv8 = p.kv_mode != 0;
  for (int it = blockIdx.x; it < items; it += G) {
    const int split = it % p.nsplit;
    const int kvh = (it / p.nsplit) % p.Hkv;
    const int b = it / (p.nsplit * p.Hkv);
#define PRISM_ATTN_CASE(GQ_)                                                   \
  case GQ_:                                                                    \
    if (kv8) attn_item<D, GQ_, true>(p, L, sc, b, kvh, split, wtid);           \
    else attn_item<D, GQ_, false>(p, L, sc, b, kvh, split, wtid);              \
    break;
    switch (GQ) {
      PRISM_ATTN_CASE(1)
      PRISM_ATTN_CASE(2)
      PRISM_ATTN_CASE(4)
      PRISM_ATTN_CASE(8)
    }
#undef PRISM_ATTN_CASE
  }
  fence_proxy_async_global();
}

// ---- the kernel ----------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(NTHREADS, 1)
decode_layers_kernel(const __grid_constant__ CUtensorMap tmXw, const __grid_constant__ CUtensorMap tmAttn,
                     const __grid_constant__ CUtensorMap tmAct, const DLParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint8_t* scratch = smem + (size_t)stages * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(scratch + SCRATCH_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;
  uint64_t* acc_empty = acc_full + NACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + NACC);
  volatile int* s_xphase = reinterpret_cast<volatile int*>(tmem_slot + 2);
  volatile int* s_abort = s_xphase + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, cta = blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    *s_xphase = 0;
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmXw);
    tma_prefetch_desc(&tmAttn);
    tma_prefetch_desc(&tmAct);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // =============================== TMA producer ===============================
      long long it0 = 0;  // stages issued before the current GEMM
      bool ok = true;
      for (int l = 0; l < p.n_layers && ok; ++l) {
        const LayerDesc* L = p.layers + l;
        for (int g = 0; g < 4 && ok; ++g) {
          const GemmGeo& geo = p.geo[g];
          const CUtensorMap* tmW = &L->tm_w[g];
          const CUtensorMap* tmX = (g == 1) ? &tmAttn : (g == 3 ? &tmAct : &tmXw);
          const int need_phase = l * 4 + g + 1;
          const int u0 = sk_start(cta, geo.U, G), u1 = sk_start(cta + 1, geo.U, G);
          int wu = u0, xu = u0;  // next unit whose weight tile / activation tile is to be issued
          bool xready = false;
          const long long t0 = clock64();
          int idle = 0;
          while (xu < u1) {
            if (!xready && ld_acquire_cta(s_xphase) >= need_phase) {
              xready = true;
              fence_proxy_async_global();  // activations were written through the generic proxy
            }
            if (xready && xu < wu) {
              const long long it = it0 + (xu - u0);
              const int s = (int)(it % stages);
              const int kb = (int)(xu % geo.kb);
              tma_load_2d(smem + (size_t)s * STAGE_BYTES + W_TILE_BYTES, tmX, &full[s], kb * BK, 0);
              ++xu;
              idle = 0;
              continue;
            }
            if (wu < u1) {
              const long long it = it0 + (wu - u0);
              const int s = (int)(it % stages);
              const long long round = it / stages;
              if (round == 0 || mbar_try_wait(&empty[s], (uint32_t)(round - 1) & 1)) {
                const int m = (int)(wu / geo.kb), kb = (int)(wu % geo.kb);
                mbar_expect_tx(&full[s], STAGE_BYTES);
                tma_load_2d(smem + (size_t)s * STAGE_BYTES, tmW, &full[s], kb * BK, m * BM);
                ++wu;
                idle = 0;
                continue;
              }
            }
            if (++idle >= 64) {
              idle = 0;
              if (aborted(p)) {
                ok = false;
                break;
              }
              if (clock64() - t0 > PRISM_WAIT_CYCLES) {
                raise_abort(p, PRISM_ERR_MBAR_TIMEOUT, 100 + g);
                ok = false;
                break;
              }
            }
          }
          if (!ok) {
            // unwinding: weight tiles in flight must land before the CTA's shared memory is released;
            // stages whose activation tile was never issued cannot complete and are only given a short wait
            for (int u = (wu - u0 > stages ? wu - stages : u0); u < wu; ++u) {
              const long long it = it0 + (u - u0);
              (void)mbar_wait_short(&full[it % stages], (uint32_t)(it / stages) & 1);
            }
          }
          it0 += u1 - u0;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // =============================== MMA issuer ===============================
      long long it = 0;
      int segc = 0;
      bool ok = true;
      for (int l = 0; l < p.n_layers && ok; ++l) {
        for (int g = 0; g < 4 && ok; ++g) {
          const GemmGeo& geo = p.geo[g];
          const int u0 = sk_start(cta, geo.U, G), u1 = sk_start(cta + 1, geo.U, G);
          int u = u0;
          while (u < u1 && ok) {
            const int tile_end = (u / geo.kb + 1) * geo.kb;
            const int seg_end = tile_end < u1 ? tile_end : u1;
            const int a = segc % NACC;
            const uint32_t use = (uint32_t)(segc / NACC);
            if (use > 0) {
              ok = mbar_wait_a(&acc_empty[a], (use - 1) & 1, p, 200);
              if (!ok) break;
              tc_fence_after();
            }
            const uint32_t acc_addr = tmem_base + a * BN;
            bool first = true;
            for (; u < seg_end; ++u, ++it) {
              const int s = (int)(it % stages);
              ok = mbar_wait_a(&full[s], (uint32_t)(it / stages) & 1, p, 201);
              if (!ok) break;
              tc_fence_after();
              const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
              const uint64_t da = umma_desc_sw128(st);
              const uint64_t db = umma_desc_sw128(st + W_TILE_BYTES);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                tc_mma_f16(acc_addr, da + 2 * k, db + 2 * k, IDESC, (first && k == 0) ? 0u : 1u);
              }
              first = false;
              tc_commit(&empty[s]);
            }
            if (ok) tc_commit(&acc_full[a]);
            ++segc;
          }
        }
      }
    }
  } else {
    // =============================== workers ===============================
    const int wtid = threadIdx.x - 64;
    const int ww = wtid >> 5;  // worker warp 0..7; warps 0..3 also run the epilogues
    AttnScratch& sc = *reinterpret_cast<AttnScratch*>(scratch);
    int segc = 0;
    bool ok = true;

    // Epilogue of GEMM g of the current layer: TMEM -> fp32 slab [slab][t][m]
    auto epilogue = [&](int g) {
      const GemmGeo& geo = p.geo[g];
      const int u0 = sk_start(cta, geo.U, G), u1 = sk_start(cta + 1, geo.U, G);
      int u = u0;
      while (u < u1) {
        const int m = u / geo.kb;
        const int tile_end = (m + 1) * geo.kb;
        const int seg_end = tile_end < u1 ? tile_end : u1;
        if (ww < 4) {
          const int a = segc % NACC;
          if (ok) ok = mbar_wait_a(&acc_full[a], (uint32_t)(segc / NACC) & 1, p, 300);
          // warp-wide TMEM access stays convergent: the wait result is the same for the whole
          // warp only after the vote
          ok = __all_sync(0xffffffffu, ok);
          if (ok) {
            tc_fence_after();
            const int q = (warp & 3);
            uint32_t r[16];
            tmem_ld16(tmem_base + a * BN + ((uint32_t)(q * 32) << 16), r);
            tmem_ld_wait();
            tc_fence_before();
            if (lane == 0) mbar_arrive(&acc_empty[a]);
            const int row = m * BM + q * 32 + lane;
            if (row < geo.M) {
              const int slab = cta - sk_owner(m * geo.kb, geo.U, G);
              float* dst = geo.part + (size_t)slab * geo.slab_stride + row;
#pragma unroll
              for (int t = 0; t < BN; ++t)
                if (t < p.T) __stcg(dst + (size_t)t * geo.M, __uint_as_float(r[t]));
            }
          }
        }
        ++segc;
        u = seg_end;
      }
    };

    for (int l = 0; l < p.n_layers && ok; ++l) {
      const LayerDesc& L = p.layers[l];
      // 1. reduce the previous projection into the residual; activation of the QKV GEMM
      reduce_phase(p, l == 0 ? nullptr : &p.geo[3], p.x0, L.norm_in, l > 0, p.ssq, false, wtid);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, l * 4 + 1))) break;
      // 2. QKV GEMM
      epilogue(0);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, 0))) break;
      // 3. q/k/v rows, KV store, attention
      load_rstd(p, p.ssq, sc.rstd, wtid);
      attn_phase<D>(p, L, sc, wtid);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, l * 4 + 2))) break;
      // 4. o_proj
      epilogue(1);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, 0))) break;
      // 5. reduce o_proj into the residual; activation of the gate/up GEMM
      reduce_phase(p, &p.geo[1], nullptr, L.norm_post, true, p.ssq + MAX_T * 32, false, wtid);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, l * 4 + 3))) break;
      // 6. gate/up GEMM
      epilogue(2);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, 0))) break;
      // 7. SwiGLU
      load_rstd(p, p.ssq + MAX_T * 32, sc.rstd, wtid);
      swiglu_phase(p, sc.rstd, wtid);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, l * 4 + 4))) break;
      // 8. down projection
      epilogue(3);
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, 0))) break;
    }
    if (ok) reduce_phase(p, &p.geo[3], nullptr, nullptr, true, nullptr, true, wtid);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

int g_sm_count = 0;
int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      g_sm_count = 148;
  }
  return g_sm_count;
}

}  // namespace

// Bytes of one layer descriptor; the caller owns an array of them in device memory.
PRISM_API int prism_decode_layer_desc_bytes() { return (int)sizeof(LayerDesc); }

// Fill one layer descriptor in HOST memory (the caller copies the array to the device once).
// Weights are row-major bf16: qkv [m_qkv, H], o [H, QD], gate_up [2 I, H], down [H, I].
PRISM_API int prism_decode_layer_desc(void* out, const void* w_qkv, int m_qkv, const void* w_o, const void* w_gate_up,
                                      const void* w_down, int H, int QD, int I, const void* norm_in, const void* norm_post,
                                      const void* q_norm, const void* k_norm, void* k_cache, void* v_cache, void* k_scale,
                                      void* v_scale) {
  LayerDesc d;
  int rc;
  if ((rc = prism_get_tensor_map(w_qkv, m_qkv, H, H, BM, &d.tm_w[0])) != 0) return rc;
  if ((rc = prism_get_tensor_map(w_o, H, QD, QD, BM, &d.tm_w[1])) != 0) return rc;
  if ((rc = prism_get_tensor_map(w_gate_up, 2ull * I, H, H, BM, &d.tm_w[2])) != 0) return rc;
  if ((rc = prism_get_tensor_map(w_down, H, I, I, BM, &d.tm_w[3])) != 0) return rc;
  d.norm_in = (const bf16*)norm_in;
  d.norm_post = (const bf16*)norm_post;
  d.q_norm = (const bf16*)q_norm;
  d.k_norm = (const bf16*)k_norm;
  d.k_cache = k_cache;
  d.v_cache = v_cache;
  d.k_scale = (float*)k_scale;
  d.v_scale = (float*)v_scale;
  memcpy(out, &d, sizeof(d));
  return 0;
}

// Grid size and slab counts for a model shape: out6 = {grid, P_qkv, P_o, P_gate_up, P_down, stages}.
PRISM_API int prism_decode_layers_plan(int H, int m_qkv, int QD, int I, int* out6) {
  if (H % 64 || QD % 64 || I % 64 || H <= 0 || m_qkv <= 0 || QD <= 0 || I <= 0) return -1;
  const long long M[4] = {m_qkv, H, 2ll * I, H};
  const long long K[4] = {H, QD, H, I};
  long long min_u = 1ll << 60;
  for (int g = 0; g < 4; ++g) {
    const long long U = ((M[g] + BM - 1) / BM) * (K[g] / BK);
    if (U < min_u) min_u = U;
    if (U * (sm_count() + 1) >= (1ll << 31)) return -2;
  }
  int G = sm_count();
  if ((long long)G > min_u) G = (int)min_u;
  out6[0] = G;
  for (int g = 0; g < 4; ++g) {
    const int kb = (int)(K[g] / BK), U = (int)((M[g] + BM - 1) / BM) * kb;
    int worst = 1;
    for (int m = 0; m * kb < U; ++m) {
      const int n = sk_owner(m * kb + kb - 1, U, G) - sk_owner(m * kb, U, G) + 1;
      if (n > worst) worst = n;
    }
    out6[1 + g] = worst;
  }
  int stages = (SMEM_LIMIT - 1024 - SCRATCH_BYTES - 512) / STAGE_BYTES;
  if (stages > 11) stages = 11;
  out6[5] = stages;
  return 0;
}

// One decode step through every layer.  `args` is a flat array of 64-bit words (pointers and
// integers; the three floats travel as their bit patterns), indexed by the enum below; see
// ops.decode_layers for the owner of every buffer.
enum DLArg {
  A_LAYERS, A_N_LAYERS, A_T, A_H, A_HQ, A_HKV, A_D, A_I, A_M_QKV, A_PAGE, A_MAX_BLOCKS, A_NUM_BLOCKS, A_KV_MODE,
  A_NSPLIT, A_EPS_BITS, A_SCALE_BITS, A_X0, A_POSITIONS, A_SLOTS, A_BLOCK_TABLES, A_CONTEXT_LENS, A_INV_FREQ, A_AXIS,
  A_RESIDUAL, A_XW, A_ATTN, A_ACT, A_SSQ, A_PART_O, A_PART_ML, A_ATTN_COUNTERS, A_GBAR, A_ABORT, A_PART_QKV, A_PART_OPROJ,
  A_PART_GU, A_PART_DOWN, A_GRID, A_COUNT
};

PRISM_API int prism_decode_layers(const long long* args, int n_args, void* stream_ptr) {
  if (n_args != A_COUNT) return -1;
  auto ptr = [&](int i) { return reinterpret_cast<void*>(static_cast<uintptr_t>(args[i])); };
  auto f32 = [&](int i) {
    const unsigned int bits = (unsigned int)args[i];
    float f;
    memcpy(&f, &bits, 4);
    return f;
  };
  DLParams p;
  memset(&p, 0, sizeof(p));
  p.layers = (const LayerDesc*)ptr(A_LAYERS);
  p.n_layers = (int)args[A_N_LAYERS];
  p.T = (int)args[A_T];
  p.H = (int)args[A_H];
  p.Hq = (int)args[A_HQ];
  p.Hkv = (int)args[A_HKV];
  const int D = (int)args[A_D];
  p.I = (int)args[A_I];
  const int m_qkv = (int)args[A_M_QKV];
  p.page = (int)args[A_PAGE];
  p.max_blocks = (int)args[A_MAX_BLOCKS];
  p.num_blocks = (int)args[A_NUM_BLOCKS];
  p.kv_mode = (int)args[A_KV_MODE];
  p.nsplit = (int)args[A_NSPLIT];
  p.eps = f32(A_EPS_BITS);
  p.attn_scale = f32(A_SCALE_BITS);
  if (p.T < 1 || p.T > MAX_T || p.n_layers < 1) return -2;
  if (D != 64 && D != 128) return -3;
  if (p.Hq <= 0 || p.Hkv <= 0 || p.Hq % p.Hkv) return -4;
  const int GQ = p.Hq / p.Hkv;
  if ((GQ != 1 && GQ != 2 && GQ != 4 && GQ != 8) || GQ * D > 512) return -5;
  if (m_qkv != (p.Hq + 2 * p.Hkv) * D) return -6;
  if (p.H % 64 || p.I % 64 || p.H > 8192) return -7;
  if (p.nsplit < 1 || p.nsplit > 32 || p.page <= 0 || p.max_blocks <= 0) return -8;
  int plan[6];
  if (prism_decode_layers_plan(p.H, m_qkv, p.Hq * D, p.I, plan) != 0) return -9;
  const int G = (int)args[A_GRID];
  if (G != plan[0]) return -10;  // slab buffers were sized for another grid
  p.stages = plan[5];
  const long long M[4] = {m_qkv, p.H, 2ll * p.I, p.H};
  const long long K[4] = {p.H, (long long)p.Hq * D, p.H, p.I};
  const int part_arg[4] = {A_PART_QKV, A_PART_OPROJ, A_PART_GU, A_PART_DOWN};
  for (int g = 0; g < 4; ++g) {
    p.geo[g].M = (int)M[g];
    p.geo[g].m_tiles = (int)((M[g] + BM - 1) / BM);
    p.geo[g].kb = (int)(K[g] / BK);
    p.geo[g].U = p.geo[g].m_tiles * p.geo[g].kb;
    p.geo[g].slab_stride = (long long)p.T * M[g];
    p.geo[g].part = (float*)ptr(part_arg[g]);
  }
  p.x0 = (const bf16*)ptr(A_X0);
  p.positions = (const int*)ptr(A_POSITIONS);
  p.slots = (const long long*)ptr(A_SLOTS);
  p.block_tables = (const int*)ptr(A_BLOCK_TABLES);
  p.context_lens = (const int*)ptr(A_CONTEXT_LENS);
  p.inv_freq = (const float*)ptr(A_INV_FREQ);
  p.axis = (const int*)ptr(A_AXIS);
  p.residual = (bf16*)ptr(A_RESIDUAL);
  p.xw = (bf16*)ptr(A_XW);
  p.attn = (bf16*)ptr(A_ATTN);
  p.act = (bf16*)ptr(A_ACT);
  p.ssq = (float*)ptr(A_SSQ);
  p.part_o = (float*)ptr(A_PART_O);
  p.part_ml = (float*)ptr(A_PART_ML);
  p.attn_counters = (int*)ptr(A_ATTN_COUNTERS);
  p.gbar = (unsigned long long*)ptr(A_GBAR);
  p.abort_flag = (int*)ptr(A_ABORT);

  CUtensorMap tm_xw, tm_attn, tm_act;
  int rc;
  if ((rc = prism_get_tensor_map(p.xw, p.T, p.H, p.H, BN, &tm_xw)) != 0) return rc;
  if ((rc = prism_get_tensor_map(p.attn, p.T, (unsigned long long)p.Hq * D, (unsigned long long)p.Hq * D, BN, &tm_attn)) != 0) return rc;
  if ((rc = prism_get_tensor_map(p.act, p.T, p.I, p.I, BN, &tm_act)) != 0) return rc;

  const size_t smem = (size_t)p.stages * STAGE_BYTES + SCRATCH_BYTES + 1024 + (2 * p.stages + 2 * NACC) * 8 + 64;
  auto kernel = (D == 128) ? decode_layers_kernel<128> : decode_layers_kernel<64>;
  static std::mutex mu;
  static bool configured[2] = {false, false};
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[D == 128]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
      if (e != cudaSuccess) return (int)e;
      configured[D == 128] = true;
    }
  }
  // all CTAs wait on one another: the launch must be cooperative (the driver refuses a grid that
  // cannot be co-resident instead of letting it deadlock)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, tm_xw, tm_attn, tm_act, p);
}
