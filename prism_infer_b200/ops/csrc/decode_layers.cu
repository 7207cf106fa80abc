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
#include <type_traits>

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
constexpr int SCRATCH_BYTES = 20 * 1024;
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
  int pf_depth;  // units the L2 prefetch cursor may run ahead of the ring (0: off)
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
  float* ssq;                // [2][MAX_T][SSQ_STRIDE]
  float* part_o;             // [T][Hq][nsplit][D]
  float* part_ml;            // [T][Hq][nsplit][2]
  int* attn_counters;        // [T*Hkv], zero, self-resetting
  unsigned long long* gbar;  // grid barrier ticket counter (monotonic)
  int* abort_flag;           // zero; set when a wait ran out
  int* tile_counters;        // [3][TILE_COUNTERS] zero, self-resetting: partials delivered per tile of o_proj / gate+up / down
  long long* timeline;       // optional [grid][n_layers][TL_STAMPS] SM clock stamps of the phase boundaries (null: off)
  // tensor parallel: every reduce phase is also the all-reduce of a row-parallel projection (or of
  // the vocabulary-sharded embedding).  xch[slot][r] is rank r's exchange buffer of that slot,
  // [tp][T][H] 8-byte words {fp32 value, sequence}; epoch is the step's sequence base.
  int tp, my_rank;
  const unsigned long long* epoch;
  unsigned long long* xch[2][8];
};
constexpr int TL_PHASES = 13;   // phase boundaries of a layer
constexpr int TL_STAMPS = 20;   // + 7 stamps inside the CTA's first attention item
constexpr int TILE_COUNTERS = 512;  // arrival counters per projection (weight tiles of 128 rows)

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

// Sum of up to n slabs, 8 consecutive floats each: every load is issued before the first add, so the
// sum costs one memory round trip whatever n is (a plain loop waits for each slab in turn).
constexpr int SLAB_UNROLL = 8;
__device__ __forceinline__ void sum_slabs8(const float* base, long long stride, int n, float (&out)[8]) {
  float4 v0[SLAB_UNROLL], v1[SLAB_UNROLL];
#pragma unroll
  for (int s = 0; s < SLAB_UNROLL; ++s) {
    v0[s] = make_float4(0.f, 0.f, 0.f, 0.f);
    v1[s] = v0[s];
    if (s < n) {
      v0[s] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * stride));
      v1[s] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * stride + 4));
    }
  }
  float4 a0 = v0[0], a1 = v1[0];
#pragma unroll
  for (int s = 1; s < SLAB_UNROLL; ++s) {
    a0.x += v0[s].x; a0.y += v0[s].y; a0.z += v0[s].z; a0.w += v0[s].w;
    a1.x += v1[s].x; a1.y += v1[s].y; a1.z += v1[s].z; a1.w += v1[s].w;
  }
  for (int s = SLAB_UNROLL; s < n; ++s) {
    const float4 w0 = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * stride));
    const float4 w1 = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * stride + 4));
    a0.x += w0.x; a0.y += w0.y; a0.z += w0.z; a0.w += w0.w;
    a1.x += w1.x; a1.y += w1.y; a1.z += w1.z; a1.w += w1.w;
  }
  out[0] = a0.x; out[1] = a0.y; out[2] = a0.z; out[3] = a0.w;
  out[4] = a1.x; out[5] = a1.y; out[6] = a1.z; out[7] = a1.w;
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

// Grid-wide barrier over the worker threads of every CTA.  A monotonic 64-bit counter: the k-th
// barrier since the buffer was created owns counts (k G, (k+1) G], so no reset and no
// launch-dependent base are needed.  The first barrier of a launch takes a ticket
// (atom.add.release) to learn k; later ones add with a fire-and-forget red.release and advance the
// target by G.  One thread arrives for the CTA after a CTA barrier (the release is cumulative
// over what the barrier ordered before it) and polls with ld.acquire.  Returns false when aborted.
__device__ __forceinline__ void st_release_cta(volatile int* addr, int v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(const_cast<int*>(addr))), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cta(volatile int* addr) {
  int v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(const_cast<int*>(addr))) : "memory");
  return v;
}
__device__ __forceinline__ bool grid_barrier(const DLParams& p, int wtid, volatile int* s_abort, volatile int* s_xphase,
                                             int xphase_value, unsigned long long& target) {
  named_bar_sync(1, NWT);
  if (wtid == 0) {
    const unsigned long long G = gridDim.x;
    bool ok = *s_abort == 0;  // after an abort nobody waits for anybody any more (peers' aborts are seen while polling)
    if (ok) {
      if (target == 0ull) {
        unsigned long long ticket;
        asm volatile("atom.add.release.gpu.global.u64 %0, [%1], 1;" : "=l"(ticket) : "l"(p.gbar) : "memory");
        target = (ticket / G + 1ull) * G;
      } else {
        target += G;
        asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(p.gbar) : "memory");
      }
    }
    const long long t0 = clock64();
    int polls = 0;
    while (ok) {
      unsigned long long v;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.gbar) : "memory");
      if (v >= target) break;
      if ((++polls & 15) == 0) {
        if (aborted(p)) ok = false;
        else if (clock64() - t0 > PRISM_WAIT_CYCLES) {
          raise_abort(p, PRISM_ERR_PEER_TIMEOUT, 900);
          ok = false;
        }
      }
    }
    if (!ok) *s_abort = 1;
    else if (xphase_value > 0) st_release_cta(s_xphase, xphase_value);  // the producer may now load this phase's activations
  }
  named_bar_sync(1, NWT);
  return *s_abort == 0;
}

// ---- reduce: slabs (+ residual) -> residual, xw = bf16(residual * weight), ssq ---------------------
constexpr int SSQ_STRIDE = 64;  // per-token partial sums of squares, one per 128-column tile (H <= 8192)

__device__ __forceinline__ float4 sum_slabs4(const float* base, long long stride, int n) {
  float4 v[SLAB_UNROLL];
#pragma unroll
  for (int s = 0; s < SLAB_UNROLL; ++s) {
    v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (s < n) v[s] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * stride));
  }
  float4 a = v[0];
#pragma unroll
  for (int s = 1; s < SLAB_UNROLL; ++s) {
    a.x += v[s].x; a.y += v[s].y; a.z += v[s].z; a.w += v[s].w;
  }
  for (int s = SLAB_UNROLL; s < n; ++s) {
    const float4 w = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * stride));
    a.x += w.x; a.y += w.y; a.z += w.z; a.w += w.w;
  }
  return a;
}

// Tensor-parallel all-reduce of 4 consecutive columns of one token, inside the reduce.  The lane
// stores its local sums into EVERY rank's exchange buffer as {value, sequence} words (an aligned
// 8-byte store is single-copy atomic: a reader that sees the sequence number sees the value), then
// polls its own buffer until all ranks' words of this exchange carry the sequence number and adds
// them in rank order, so every rank computes bit-identical rows.  No flag, fence or extra barrier;
// consecutive exchanges alternate between two buffers: a rank can only reach the next use of a
// buffer after all peers consumed the previous one, because the exchange in between needed every
// peer's data.
__device__ __forceinline__ void tp_exchange4(const DLParams& p, float (&d)[4], int t, int col, int point,
                                             unsigned long long epoch) {
  const unsigned long long seq = (epoch + (unsigned long long)point) & 0xffffffffull;
  const int slot = (int)(((epoch >> 7) + (unsigned long long)point) & 1ull);
  const size_t mine = ((size_t)p.my_rank * p.T + t) * p.H + col;
  for (int r = 0; r < p.tp; ++r) {
    unsigned long long* dst = p.xch[slot][r] + mine;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const unsigned long long w0 = (seq << 32) | (unsigned long long)__float_as_uint(d[2 * e]);
      const unsigned long long w1 = (seq << 32) | (unsigned long long)__float_as_uint(d[2 * e + 1]);
      asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst + 2 * e), "l"(w0), "l"(w1) : "memory");
    }
  }
  const unsigned long long* own = p.xch[slot][p.my_rank] + (size_t)t * p.H + col;
  const unsigned int want = (unsigned int)seq;
  const long long t0 = clock64();
  for (;;) {
    unsigned int stale = 0;
    d[0] = d[1] = d[2] = d[3] = 0.0f;
    for (int r = 0; r < p.tp; ++r) {
      const unsigned long long* q0 = own + (size_t)r * p.T * p.H;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        unsigned long long w0, w1;
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(q0 + 2 * e) : "memory");
        stale |= ((unsigned int)(w0 >> 32) ^ want) | ((unsigned int)(w1 >> 32) ^ want);
        d[2 * e] += __uint_as_float((unsigned int)w0);
        d[2 * e + 1] += __uint_as_float((unsigned int)w1);
      }
    }
    if (stale == 0) break;
    if (aborted(p)) break;
    if (clock64() - t0 > PRISM_WAIT_CYCLES) {
      raise_abort(p, PRISM_ERR_PEER_TIMEOUT, 700 + point);
      break;
    }
  }
}

// One (token, 128-column tile) on one warp; a lane owns 4 columns.  src: slabs of the projection
// that produced the delta (null: the embedding rows x0); weight null: only the residual is updated
// (the last layer's down projection leaves the pre-norm hidden state there).
__device__ __forceinline__ void reduce_tile(const DLParams& p, const GemmGeo* src, const bf16* x0, const bf16* weight,
                                            bool have_residual, float* ssq_out, int t, int m, int lane, int point,
                                            unsigned long long epoch) {
  const int H = p.H;
  const int col = m * BM + lane * 4;
  // residual and norm weight are requested together with the slabs: one memory round trip
  bf16* res = p.residual + (size_t)t * H + col;
  uint2 res_raw = make_uint2(0, 0), w_raw = make_uint2(0, 0), x_raw = make_uint2(0, 0);
  if (have_residual) res_raw = __ldcg(reinterpret_cast<const uint2*>(res));
  if (weight != nullptr) w_raw = __ldg(reinterpret_cast<const uint2*>(weight + col));
  float d[4];
  if (src != nullptr) {
    int first, n;
    sk_tile_slabs(*src, m, gridDim.x, first, n);
    const float4 a = sum_slabs4(src->part + (size_t)t * src->M + col, src->slab_stride, n);
    d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w;
  } else {
    x_raw = __ldcg(reinterpret_cast<const uint2*>(x0 + (size_t)t * H + col));
    const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&x_raw);
    d[0] = b2f(v[0].x); d[1] = b2f(v[0].y); d[2] = b2f(v[1].x); d[3] = b2f(v[1].y);
  }
  if (p.tp > 1) tp_exchange4(p, d, t, col, point, epoch);
#pragma unroll
  for (int e = 0; e < 4; ++e) d[e] = bf16_round(d[e]);
  if (have_residual) {
    const __nv_bfloat162* r = reinterpret_cast<const __nv_bfloat162*>(&res_raw);
    d[0] = bf16_round(b2f(r[0].x) + d[0]);
    d[1] = bf16_round(b2f(r[0].y) + d[1]);
    d[2] = bf16_round(b2f(r[1].x) + d[2]);
    d[3] = bf16_round(b2f(r[1].y) + d[3]);
  }
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(d[0], d[1]);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(d[2], d[3]);
  *reinterpret_cast<uint2*>(res) = o;
  if (weight != nullptr) {
    const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&w_raw);
    uint2 xo;
    *reinterpret_cast<__nv_bfloat162*>(&xo.x) = __floats2bfloat162_rn(d[0] * b2f(w[0].x), d[1] * b2f(w[0].y));
    *reinterpret_cast<__nv_bfloat162*>(&xo.y) = __floats2bfloat162_rn(d[2] * b2f(w[1].x), d[3] * b2f(w[1].y));
    *reinterpret_cast<uint2*>(p.xw + (size_t)t * H + col) = xo;
    const float ss = warp_sum(d[0] * d[0] + d[1] * d[1] + d[2] * d[2] + d[3] * d[3]);
    if (lane == 0) __stcg(ssq_out + t * SSQ_STRIDE + m, ss);
  }
}

// The embedding rows of a step (layer 0 has no projection before it): (token, tile) items over all
// worker warps of all CTAs.
__device__ __forceinline__ void reduce_phase_x0(const DLParams& p, const bf16* weight, float* ssq_out, int wtid,
                                                unsigned long long epoch) {
  const int G = gridDim.x, cta = blockIdx.x;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int tiles = p.H / BM;
  const int items = p.T * tiles;
  for (int it = cta + G * warp; it < items; it += G * NW)
    reduce_tile(p, nullptr, p.x0, weight, false, ssq_out, it / tiles, it % tiles, lane, 0, epoch);
  fence_proxy_async_global();  // xw is read by TMA (async proxy) after the barrier
}

// 1/rms of every token from the per-tile sums of squares -> shared memory
__device__ __forceinline__ void load_rstd(const DLParams& p, const float* ssq, float* s_rstd, int wtid) {
  const int warp = wtid >> 5, lane = wtid & 31;
  const int tiles = p.H / BM;
  for (int t = warp; t < p.T; t += NW) {
    float v = lane < tiles ? __ldcg(ssq + t * SSQ_STRIDE + lane) : 0.0f;
    if (lane + 32 < tiles) v += __ldcg(ssq + t * SSQ_STRIDE + lane + 32);
    v = warp_sum(v);
    if (lane == 0) s_rstd[t] = rsqrtf(v / (float)p.H + p.eps);
  }
  named_bar_sync(1, NWT);
}

// SwiGLU of one (token, 128-column tile of the activation) on one warp:
// act = bf16(bf16(silu(bf16(rstd * sum gate))) * bf16(rstd * sum up))
__device__ __forceinline__ void swiglu_tile(const DLParams& p, float rstd, int t, int m, int lane) {
  const GemmGeo& g = p.geo[2];
  const int I = p.I, G = gridDim.x;
  const int col = m * BM + lane * 4;
  int f0, n0, f1, n1;
  sk_tile_slabs(g, m, G, f0, n0);
  sk_tile_slabs(g, m + I / BM, G, f1, n1);
  const float4 ga = sum_slabs4(g.part + (size_t)t * g.M + col, g.slab_stride, n0);
  const float4 ua = sum_slabs4(g.part + (size_t)t * g.M + I + col, g.slab_stride, n1);
  const float gs[4] = {ga.x, ga.y, ga.z, ga.w}, us[4] = {ua.x, ua.y, ua.z, ua.w};
  float a[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) a[e] = bf16_round(silu(bf16_round(gs[e] * rstd))) * bf16_round(us[e] * rstd);
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(a[0], a[1]);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(a[2], a[3]);
  *reinterpret_cast<uint2*>(p.act + (size_t)t * I + col) = o;
}

// ---- attention phase ---------------------------------------------------------------------------
// Per-step inputs that every layer reads again: copied to shared memory once per launch.
constexpr int BT_CACHE = 1024;  // block-table entries kept in shared memory (T * max_blocks beyond that: global loads)
struct StepConst {
  long long slots[MAX_T];
  int ctx[MAX_T];
  int pos[3][MAX_T];
  int axis[64];
  float inv_freq[64];
  int bt_ok;
  int bt[BT_CACHE];
};
struct AttnScratch {
  float rstd[MAX_T];       // 1/rms of the layer input (QKV consumer)
  float rstd_post[MAX_T];  // 1/rms after attention (gate/up consumer)
  int tail_tile;           // tile whose pointwise tail this CTA runs (-1: none)
  float q[512];            // [GQ][D] bf16 values as floats
  float kn[128], vn[128];  // the new token's K / V as attention sees them (dequantised payload)
  float kv_scale[2];
  float m[NW / 2][8], l[NW / 2][8];
  float acc[(NW / 2) * 512];  // [NW/2][GQ][D]: warps merge in two rounds
  float coef[8][32];
  float inv[8];
  int last;
};
struct WorkerSmem {
  AttnScratch attn;
  StepConst step;
  long long* tl_attn;  // where the current layer's attention sub-stamps go (null: off)
};
static_assert(sizeof(WorkerSmem) <= SCRATCH_BYTES, "worker scratch");

// One (sequence, KV head, split) item on all worker warps.
template <int D, int GQ, bool KV8>
__device__ __noinline__ void attn_item(const DLParams& p, const LayerDesc& L, WorkerSmem& ws, int b, int kvh, int split,
                                       int wtid) {
  constexpr int EPL = 8;            // head-dimension elements per lane (8 bytes of FP8 or 16 bytes of bf16)
  constexpr int LPT = D / EPL;      // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp and load group
  constexpr int UNR = 4;
  constexpr int PER = D / 64;
  AttnScratch& sc = ws.attn;
  const StepConst& cst = ws.step;
  const int G = gridDim.x;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int slot_in_warp = lane / LPT, part = lane % LPT;
  long long* tla = ws.tl_attn;
  int tla_i = 0;
  auto sub_stamp = [&]() {
    if (tla != nullptr && wtid == 0 && tla_i < TL_STAMPS - TL_PHASES) tla[tla_i++] = clock64();
  };
  sub_stamp();
  int ctx = cst.ctx[b];
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
  const int j_stop = owner ? min(j_end, ctx - 1) : j_end;  // the new token comes from shared memory
  const float rstd = sc.rstd[b];
  const GemmGeo& gq = p.geo[0];
  const int* bt_g = p.block_tables + (size_t)b * p.max_blocks;
  const int* bt_s = cst.bt + b * p.max_blocks;
  const bool bt_cached = cst.bt_ok != 0;

  // One batch of cached tokens per warp: page-table entries, payload and scales of UNR token groups.
  // The loaded registers are not touched before the fold (any move of a loaded value would make the
  // warp wait for that load before it issues the next one).
  typedef typename std::conditional<KV8, uint2, uint4>::type KvVec;  // 8 elements: 8 bytes of FP8 / 16 of bf16
  KvVec kr[UNR], vr[UNR];
  float ks[UNR], vs[UNR];
  bool valid[UNR];
  auto load_batch = [&](int j0) {
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int j = j0 + u * TPW + slot_in_warp;
      int blk = -1;
      if (j < j_stop) {
        blk = bt_cached ? bt_s[j / p.page] : bt_g[j / p.page];
        if (p.num_blocks > 0 && blk >= p.num_blocks) {
          prism_report(PRISM_ERR_BOUNDS, 2);
          blk = -1;
        }
      }
      valid[u] = blk >= 0;
      ks[u] = 1.0f;
      vs[u] = 1.0f;
      if (valid[u]) {
        const size_t row = ((size_t)blk * p.Hkv + kvh) * p.page + (j % p.page);
        const size_t off = (row * D + (size_t)part * 8) * (KV8 ? 1 : 2);
        kr[u] = __ldcg(reinterpret_cast<const KvVec*>(reinterpret_cast<const uint8_t*>(L.k_cache) + off));
        vr[u] = __ldcg(reinterpret_cast<const KvVec*>(reinterpret_cast<const uint8_t*>(L.v_cache) + off));
        if (KV8 && p.kv_mode == 2) {
          ks[u] = __ldcg(L.k_scale + row);
          vs[u] = __ldcg(L.v_scale + row);
        }
      }
    }
  };
  // the first batch is requested before the q / k / v rows are built: it does not depend on them
  const int j_first = j_begin + warp * TPW * UNR;
  if (j_first < j_stop) load_batch(j_first);

  // ---- rows of the packed QKV projection this item needs: GQ query heads (+ K and V of the new token)
  const int nrows = GQ + (owner ? 2 : 0);
  for (int r = warp; r < nrows; r += NW) {
    const bool is_q = r < GQ, is_k = r == GQ;
    const int h = is_q ? kvh * GQ + r : (is_k ? p.Hq + kvh : p.Hq + p.Hkv + kvh);
    const int col0 = h * D;
    int first, n;
    sk_tile_slabs(gq, col0 / BM, G, first, n);
    const float* base = gq.part + (size_t)b * gq.M + col0;
    const bf16* nw = is_q ? L.q_norm : L.k_norm;
    bf16 wlo_raw[PER], whi_raw[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {  // norm weights travel together with the slabs (converted only when used)
      wlo_raw[j] = nw[lane + 32 * j];
      whi_raw[j] = nw[lane + 32 * j + D / 2];
    }
    float lo[PER], hi[PER];
    {
      float v0[SLAB_UNROLL][PER], v1[SLAB_UNROLL][PER];
#pragma unroll
      for (int s = 0; s < SLAB_UNROLL; ++s)
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          v0[s][j] = v1[s][j] = 0.0f;
          if (s < n) {
            v0[s][j] = __ldcg(base + (size_t)s * gq.slab_stride + lane + 32 * j);
            v1[s][j] = __ldcg(base + (size_t)s * gq.slab_stride + lane + 32 * j + D / 2);
          }
        }
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        float s0 = v0[0][j], s1 = v1[0][j];
#pragma unroll
        for (int s = 1; s < SLAB_UNROLL; ++s) {
          s0 += v0[s][j];
          s1 += v1[s][j];
        }
        for (int s = SLAB_UNROLL; s < n; ++s) {
          s0 += __ldcg(base + (size_t)s * gq.slab_stride + lane + 32 * j);
          s1 += __ldcg(base + (size_t)s * gq.slab_stride + lane + 32 * j + D / 2);
        }
        lo[j] = bf16_round(s0 * rstd);
        hi[j] = bf16_round(s1 * rstd);
      }
    }
    if (is_q || is_k) {
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < PER; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
      ss = warp_sum(ss);
      const float hr = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        lo[j] = bf16_round(bf16_round(lo[j] * hr) * b2f(wlo_raw[j]));
        hi[j] = bf16_round(bf16_round(hi[j] * hr) * b2f(whi_raw[j]));
      }
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + 32 * j;
        const float pos = (float)cst.pos[cst.axis[i]][b];
        float sn, cs;
        sincosf(pos * cst.inv_freq[i], &sn, &cs);
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
    const long long slot = cst.slots[b];
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
  sub_stamp();
  named_bar_sync(1, NWT);
  sub_stamp();

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

  auto fold = [&](const float (&kf)[EPL], const float (&vf)[EPL], float kscale, float vscale, bool ok) {
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      float sdot = 0.0f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) sdot += q[g][e] * kf[e];
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, o);
      if (ok) {
        sdot *= kscale;
        const float mn = fmaxf(m[g], sdot);
        const float corr = __expf(m[g] - mn);
        const float pr = __expf(sdot - mn);
        l[g] = l[g] * corr + pr;
        const float pv = pr * vscale;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + pv * vf[e];
        m[g] = mn;
      }
    }
  };

  for (int j0 = j_first; j0 < j_stop; j0 += TPW * NW * UNR) {
    if (j0 != j_first) load_batch(j0);
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      float kf[EPL], vf[EPL];
      if (KV8) {
        const unsigned short* kp = reinterpret_cast<const unsigned short*>(&kr[u]);
        const unsigned short* vp = reinterpret_cast<const unsigned short*>(&vr[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 kk = fp8x2_to_float2(kp[e]);
          const float2 vv = fp8x2_to_float2(vp[e]);
          kf[2 * e] = kk.x;
          kf[2 * e + 1] = kk.y;
          vf[2 * e] = vv.x;
          vf[2 * e + 1] = vv.y;
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
  sub_stamp();
  // merge the token slots of a warp (afterwards every lane of a slice holds the warp's result)
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
  // merge the warps in two rounds through NW / 2 shared-memory slots
  constexpr int HW = NW / 2;
  auto put = [&](int slotw) {
    if (slot_in_warp == 0) {
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        if (part == 0) {
          sc.m[slotw][g] = m[g];
          sc.l[slotw][g] = l[g];
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) sc.acc[(slotw * GQ + g) * D + part * EPL + e] = acc[g][e];
      }
    }
  };
  if (warp >= HW) put(warp - HW);
  named_bar_sync(1, NWT);
  if (warp < HW) {
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      const float mo = sc.m[warp][g], lo2 = sc.l[warp][g];
      const float mn = fmaxf(m[g], mo);
      const float c0 = (m[g] == -INFINITY) ? 0.0f : __expf(m[g] - mn);
      const float c1 = (mo == -INFINITY) ? 0.0f : __expf(mo - mn);
      l[g] = l[g] * c0 + lo2 * c1;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * c0 + sc.acc[(warp * GQ + g) * D + part * EPL + e] * c1;
      m[g] = mn;
    }
    __syncwarp();
    put(warp);
  }
  named_bar_sync(1, NWT);
  sub_stamp();
  const int ns = p.nsplit;
  for (int idx = wtid; idx < GQ * D; idx += NWT) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < HW; ++w) mm = fmaxf(mm, sc.m[w][g]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < HW; ++w) {
      const float c = (sc.m[w][g] == -INFINITY) ? 0.0f : __expf(sc.m[w][g] - mm);
      ll += sc.l[w][g] * c;
      oo += sc.acc[(w * GQ + g) * D + d] * c;
    }
    const int hq = kvh * GQ + g;
    if (ns == 1) {
      p.attn[((size_t)b * p.Hq + hq) * D + d] = __float2bfloat16_rn(ll > 0.0f ? oo / ll : 0.0f);
    } else {
      const size_t pidx = ((size_t)b * p.Hq + hq) * ns + split;
      __stcg(p.part_o + pidx * D + d, oo);
      if (d == 0) {
        __stcg(p.part_ml + pidx * 2, mm);
        __stcg(p.part_ml + pidx * 2 + 1, ll);
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
    sub_stamp();
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
        // all partial loads in flight at once (a serial loop would pay one round trip per split)
        float pv[32];
#pragma unroll
        for (int sidx = 0; sidx < 32; ++sidx) pv[sidx] = sidx < ns ? __ldcg(po + (size_t)sidx * D) : 0.0f;
        float oo = 0.0f;
#pragma unroll
        for (int sidx = 0; sidx < 32; ++sidx) oo += pv[sidx] * sc.coef[g][sidx];
        p.attn[bh * D + d] = __float2bfloat16_rn(oo * sc.inv[g]);
      }
    }
  }
  named_bar_sync(1, NWT);  // scratch is reused by the next item
  sub_stamp();
  if (wtid == 0) ws.tl_attn = nullptr;  // only the CTA's first item of a layer is recorded
}

template <int D>
__device__ __forceinline__ void attn_phase(const DLParams& p, const LayerDesc& L, WorkerSmem& ws, int wtid) {
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
    if (kv8) attn_item<D, GQ_, true>(p, L, ws, b, kvh, split, wtid);           \
    else attn_item<D, GQ_, false>(p, L, ws, b, kvh, split, wtid);              \
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

// ---- producer cursors ------------------------------------------------------------------------------
struct UnitCursor {
  int l, g;      // layer, GEMM (0 qkv, 1 o_proj, 2 gate/up, 3 down)
  int u, u1;     // unit and end of this CTA's run of the current GEMM
  int m, kb;     // weight tile and k-block of the unit
  int kbn;       // k-blocks per tile of the current GEMM
  bool done;
};
__device__ __forceinline__ void cursor_load(UnitCursor& c, const DLParams& p, int cta, int G) {
  const GemmGeo& geo = p.geo[c.g];
  c.u = sk_start(cta, geo.U, G);
  c.u1 = sk_start(cta + 1, geo.U, G);
  c.kbn = geo.kb;
  c.m = c.u / geo.kb;
  c.kb = c.u % geo.kb;
}
__device__ __forceinline__ void cursor_begin(UnitCursor& c, const DLParams& p, int cta, int G) {
  c.l = 0;
  c.g = 0;
  c.done = false;
  cursor_load(c, p, cta, G);
}
__device__ __forceinline__ void cursor_next(UnitCursor& c, const DLParams& p, int cta, int G) {
  ++c.u;
  if (++c.kb == c.kbn) {
    c.kb = 0;
    ++c.m;
  }
  if (c.u < c.u1) return;
  if (++c.g == 4) {
    c.g = 0;
    if (++c.l == p.n_layers) {
      c.done = true;
      return;
    }
  }
  cursor_load(c, p, cta, G);
}
// Request the box into L2 without a destination: a later TMA load of the same box hits.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y)
               : "memory");
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
      // Three cursors walk this CTA's units of every GEMM of every layer in order:
      //   P  requests weight tiles into L2 (a hint), up to pf_depth units ahead of W,
      //   W  issues the weight tile of a unit into the next free ring stage,
      //   X  issues the unit's activation tile once the phase that produces it has passed.
      // W runs ahead of X by at most the ring depth and across phase and layer boundaries, so the
      // HBM stream does not stop while the workers sit in a barrier or a pointwise phase.
      UnitCursor P, W, X;
      cursor_begin(P, p, cta, G);
      W = P;
      X = P;
      long long n_p = 0, n_w = 0, n_x = 0;  // units passed by each cursor
      int w_s = 0, x_s = 0;                  // ring stage of the next W / X issue
      uint32_t w_pass = 0;                   // times the W cursor wrapped the ring
      int xphase_seen = 0;
      const int pf_depth = p.pf_depth;
      long long t0 = clock64();
      int idle = 0;
      while (!X.done) {
        if (n_x < n_w) {
          const int need = X.l * 4 + X.g + 1;
          if (xphase_seen < need) {
            const int v = ld_acquire_cta(s_xphase);
            if (v > xphase_seen) {
              xphase_seen = v;
              fence_proxy_async_global();  // activations were written through the generic proxy
            }
          }
          if (xphase_seen >= need) {
            const CUtensorMap* tmX = (X.g == 1) ? &tmAttn : (X.g == 3 ? &tmAct : &tmXw);
            tma_load_2d(smem + (size_t)x_s * STAGE_BYTES + W_TILE_BYTES, tmX, &full[x_s], X.kb * BK, 0);
            if (++x_s == stages) x_s = 0;
            cursor_next(X, p, cta, G);
            ++n_x;
            idle = 0;
            continue;
          }
        }
        if (!W.done && (w_pass == 0 || mbar_try_wait(&empty[w_s], (w_pass - 1) & 1))) {
          mbar_expect_tx(&full[w_s], STAGE_BYTES);
          tma_load_2d(smem + (size_t)w_s * STAGE_BYTES, &p.layers[W.l].tm_w[W.g], &full[w_s], W.kb * BK, W.m * BM);
          if (++w_s == stages) {
            w_s = 0;
            ++w_pass;
          }
          cursor_next(W, p, cta, G);
          ++n_w;
          idle = 0;
          continue;
        }
        if (!P.done && n_p < n_w + pf_depth) {
          if (n_p >= n_w + stages / 2) tma_prefetch_2d(&p.layers[P.l].tm_w[P.g], P.kb * BK, P.m * BM);
          cursor_next(P, p, cta, G);
          ++n_p;
          idle = 0;
          continue;
        }
        if (idle == 0) t0 = clock64();
        if (++idle >= 64) {
          idle = 1;
          if (aborted(p)) break;
          if (clock64() - t0 > PRISM_WAIT_CYCLES) {
            raise_abort(p, PRISM_ERR_MBAR_TIMEOUT, 100 + X.g);
            break;
          }
        }
      }
      if (!X.done) {
        // unwinding: weight tiles in flight must land before the CTA's shared memory is released;
        // a stage whose activation tile was never issued cannot complete and only gets a short wait
        int s2 = w_s;
        uint32_t pass = w_pass;
        const int back = n_w < stages ? (int)n_w : stages;
        for (int i = 0; i < back; ++i) {
          if (s2 == 0) {
            s2 = stages;
            --pass;
          }
          --s2;
          (void)mbar_wait_short(&full[s2], pass & 1);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // =============================== MMA issuer ===============================
      int s_i = 0;            // ring stage
      uint32_t s_par = 0;     // its phase parity
      int a_i = 0;            // accumulator
      uint32_t a_use = 0;     // times the accumulator ring wrapped
      bool ok = true;
      for (int l = 0; l < p.n_layers && ok; ++l) {
        for (int g = 0; g < 4 && ok; ++g) {
          const GemmGeo& geo = p.geo[g];
          const int u0 = sk_start(cta, geo.U, G), u1 = sk_start(cta + 1, geo.U, G);
          int u = u0;
          int kb_in_tile = u0 % geo.kb;
          while (u < u1 && ok) {
            const int left = geo.kb - kb_in_tile;
            const int seg_end = (u + left < u1) ? u + left : u1;
            if (a_use > 0) {
              ok = mbar_wait_a(&acc_empty[a_i], (a_use - 1) & 1, p, 200);
              if (!ok) break;
              tc_fence_after();
            }
            const uint32_t acc_addr = tmem_base + a_i * BN;
            bool first = true;
            for (; u < seg_end; ++u) {
              ok = mbar_wait_a(&full[s_i], s_par, p, 201);
              if (!ok) break;
              tc_fence_after();
              const uint32_t st = smem_u32(smem + (size_t)s_i * STAGE_BYTES);
              const uint64_t da = umma_desc_sw128(st);
              const uint64_t db = umma_desc_sw128(st + W_TILE_BYTES);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                tc_mma_f16(acc_addr, da + 2 * k, db + 2 * k, IDESC, (first && k == 0) ? 0u : 1u);
              }
              first = false;
              tc_commit(&empty[s_i]);
              if (++s_i == stages) {
                s_i = 0;
                s_par ^= 1;
              }
            }
            if (ok) tc_commit(&acc_full[a_i]);
            if (++a_i == NACC) {
              a_i = 0;
              ++a_use;
            }
            kb_in_tile = 0;
          }
        }
      }
    }
  } else {
    // =============================== workers ===============================
    const int wtid = threadIdx.x - 64;
    const int ww = wtid >> 5;  // worker warp 0..7; warps 0..3 also run the epilogues
    WorkerSmem& ws = *reinterpret_cast<WorkerSmem*>(scratch);
    AttnScratch& sc = ws.attn;
    int segc = 0;
    bool ok = true;

    const unsigned long long epoch = (p.tp > 1 && p.epoch != nullptr) ? *p.epoch : 0ull;

    // Epilogue of GEMM g of layer l: TMEM -> fp32 slab [slab][t][m].  For o_proj, gate/up and down
    // the CTA that delivers the LAST partial of a weight tile (arrival counter per tile, the classic
    // fence / counter / fence hand-off) runs the pointwise step on that tile's 128 columns right
    // away: the reduce into the residual (+ the activation of the next GEMM and the sums of
    // squares), or SwiGLU once the gate tile and its up tile are both complete.  No grid barrier
    // stands between a projection and its consumer, and the tails of 32 to 96 tiles run on as many
    // CTAs in parallel instead of on the few that a separate phase would keep busy.
    auto epilogue = [&](int g, int l) {
      const GemmGeo& geo = p.geo[g];
      const int u0 = sk_start(cta, geo.U, G), u1 = sk_start(cta + 1, geo.U, G);
      const int pair = p.I / BM;  // gate tile m and up tile m + pair feed the same activation tile
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
          if (g != 0) {
            // all four epilogue warps take part, also after a failed wait (the barrier count is fixed)
            __threadfence();
            named_bar_sync(2, 128);
            if (wtid == 0) {
              int need, first;
              const int tile = (g == 2 && m >= pair) ? m - pair : m;
              sk_tile_slabs(geo, tile, G, first, need);
              if (g == 2) {
                int n_up;
                sk_tile_slabs(geo, tile + pair, G, first, n_up);
                need += n_up;
              }
              int* cnt = p.tile_counters + (g - 1) * TILE_COUNTERS + tile;
              const int old = atomicAdd(cnt, 1);
              const bool last = ok && old == need - 1;
              if (old == need - 1) *cnt = 0;  // self-resetting: the next layer's arrivals come after a grid barrier
              sc.tail_tile = last ? tile : -1;
            }
            named_bar_sync(2, 128);
            const int tile = sc.tail_tile;
            if (tile >= 0) {
              __threadfence();
              if (g == 2) {
                for (int t = ww; t < p.T; t += 4) swiglu_tile(p, sc.rstd_post[t], t, tile, lane);
              } else if (g == 1) {
                for (int t = ww; t < p.T; t += 4)
                  reduce_tile(p, &geo, nullptr, p.layers[l].norm_post, true, p.ssq + MAX_T * SSQ_STRIDE, t, tile, lane, 2 * l + 1, epoch);
              } else {
                const bf16* w_next = l + 1 < p.n_layers ? p.layers[l + 1].norm_in : nullptr;
                for (int t = ww; t < p.T; t += 4) reduce_tile(p, &geo, nullptr, w_next, true, p.ssq, t, tile, lane, 2 * l + 2, epoch);
              }
              fence_proxy_async_global();  // xw / act are read by TMA (async proxy) after the barrier
            }
          }
        }
        ++segc;
        u = seg_end;
      }
    };

    {  // per-step inputs every layer reads again
      StepConst& cst = ws.step;
      const int half = D / 2;
      for (int i = wtid; i < MAX_T; i += NWT) {
        cst.ctx[i] = i < p.T ? p.context_lens[i] : 0;
        cst.slots[i] = i < p.T ? p.slots[i] : -1;
        for (int a3 = 0; a3 < 3; ++a3) cst.pos[a3][i] = i < p.T ? p.positions[(size_t)a3 * p.T + i] : 0;
      }
      for (int i = wtid; i < 64; i += NWT) {
        cst.axis[i] = i < half ? min(2, max(0, p.axis[i])) : 0;
        cst.inv_freq[i] = i < half ? p.inv_freq[i] : 0.0f;
      }
      const int n_bt = p.T * p.max_blocks;
      if (wtid == 0) cst.bt_ok = n_bt <= BT_CACHE ? 1 : 0;
      if (n_bt <= BT_CACHE)
        for (int i = wtid; i < n_bt; i += NWT) cst.bt[i] = p.block_tables[i];
      named_bar_sync(1, NWT);
    }
    unsigned long long bar_target = 0ull;
    int stamp_i = 0;
    long long* tl = nullptr;
    auto stamp = [&]() {
      if (tl != nullptr && wtid == 0 && stamp_i < TL_PHASES) tl[stamp_i++] = clock64();
    };
    if (wtid == 0) ws.tl_attn = nullptr;
    for (int l = 0; l < p.n_layers && ok; ++l) {
      const LayerDesc& L = p.layers[l];
      if (p.timeline != nullptr) tl = p.timeline + ((size_t)cta * p.n_layers + l) * TL_STAMPS;
      stamp_i = 0;
      stamp();
      if (l == 0) {
        // the embedding rows become the residual and the activation of the first QKV GEMM
        reduce_phase_x0(p, L.norm_in, p.ssq, wtid, epoch);
        stamp();
        if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, 1, bar_target))) break;
        stamp();
      } else {
        stamp();
        stamp();
      }
      // 1. QKV GEMM
      epilogue(0, l);
      stamp();
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, 0, bar_target))) break;
      stamp();
      // 2. q/k/v rows, KV store, attention
      if (wtid == 0) ws.tl_attn = tl != nullptr ? tl + TL_PHASES : nullptr;
      load_rstd(p, p.ssq, sc.rstd, wtid);
      attn_phase<D>(p, L, ws, wtid);
      stamp();
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, l * 4 + 2, bar_target))) break;
      stamp();
      // 3. o_proj; tile tails: reduce into the residual, activation of the gate/up GEMM
      epilogue(1, l);
      stamp();
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, l * 4 + 3, bar_target))) break;
      stamp();
      // 4. gate/up GEMM; tile tails: SwiGLU (needs the post-attention 1/rms)
      load_rstd(p, p.ssq + MAX_T * SSQ_STRIDE, sc.rstd_post, wtid);
      epilogue(2, l);
      stamp();
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, l * 4 + 4, bar_target))) break;
      stamp();
      // 5. down projection; tile tails: reduce into the residual, activation of the next layer's QKV GEMM
      epilogue(3, l);
      stamp();
      if (!(ok = grid_barrier(p, wtid, s_abort, s_xphase, (l + 1) * 4 + 1, bar_target))) break;
      stamp();
    }
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
  A_PART_GU, A_PART_DOWN, A_GRID, A_TIMELINE, A_PF_DEPTH, A_TP, A_RANK, A_EPOCH, A_TILE_COUNTERS, A_XCH0, A_XCH1 = A_XCH0 + 8,
  A_COUNT = A_XCH1 + 8
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
  if (p.H % 128 || p.I % 128 || p.H > 8192 || p.H / BM > TILE_COUNTERS || p.I / BM > TILE_COUNTERS) return -7;
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
  p.tile_counters = (int*)ptr(A_TILE_COUNTERS);
  p.timeline = (long long*)ptr(A_TIMELINE);
  p.pf_depth = (int)args[A_PF_DEPTH];
  if (p.pf_depth < 0 || p.pf_depth > 256) return -11;
  p.tp = (int)args[A_TP];
  p.my_rank = (int)args[A_RANK];
  p.epoch = (const unsigned long long*)ptr(A_EPOCH);
  if (p.tp < 1 || p.tp > 8 || p.my_rank < 0 || p.my_rank >= p.tp) return -12;
  for (int r = 0; r < 8; ++r) {
    p.xch[0][r] = (unsigned long long*)ptr(A_XCH0 + r);
    p.xch[1][r] = (unsigned long long*)ptr(A_XCH1 + r);
    if (p.tp > 1 && r < p.tp && (p.xch[0][r] == nullptr || p.xch[1][r] == nullptr)) return -13;
  }
  if (p.tp > 1 && p.epoch == nullptr) return -13;
  if (p.tp > 1 && 2 * p.n_layers + 1 > 127) return -14;  // exchange points of a step share the epoch's 128 sequence numbers

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
