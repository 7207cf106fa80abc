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
constexpr int SCRATCH_BYTES = 26 * 1024;
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
  int page_shift;            // log2(page): pages are powers of two
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
struct WorkerSmem;
// What a worker thread carries through the phases (the phase functions are not inlined, so that
// each exists once in the instruction stream: a decode step runs every phase once per layer, and
// code that does not stay in the instruction cache is fetched again for every layer).
struct WorkerCtx {
  uint64_t* acc_full;
  uint64_t* acc_empty;
  uint32_t tmem_base;
  volatile int* s_abort;
  volatile int* s_xphase;
  WorkerSmem* ws;
  int wtid, ww, lane, warp;   // worker thread / worker warp / lane / warp index inside the CTA
  int segc;                   // accumulator segments consumed so far
  bool ok;
  unsigned long long epoch, bar_target;
};

__device__ __noinline__ bool grid_barrier(const DLParams& p, WorkerCtx& c, int xphase_value) {
  named_bar_sync(1, NWT);
  if (c.wtid == 0) {
    const unsigned long long G = gridDim.x;
    unsigned long long target = c.bar_target;
    bool ok = *c.s_abort == 0;  // after an abort nobody waits for anybody any more (peers' aborts are seen while polling)
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
    c.bar_target = target;
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
    if (!ok) *c.s_abort = 1;
    else if (xphase_value > 0) st_release_cta(c.s_xphase, xphase_value);  // the producer may now load this phase's activations
  }
  named_bar_sync(1, NWT);
  return *c.s_abort == 0;
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
#pragma unroll 1
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
  const size_t rank_stride = (size_t)p.T * p.H;
  const long long t0 = clock64();
  for (;;) {
    // every rank's words are requested before any is looked at: one round trip per attempt
    unsigned long long w[8][4];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < p.tp) {
        const unsigned long long* q0 = own + (size_t)r * rank_stride;
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w[r][0]), "=l"(w[r][1]) : "l"(q0) : "memory");
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w[r][2]), "=l"(w[r][3]) : "l"(q0 + 2) : "memory");
      }
    }
    unsigned int stale = 0;
    d[0] = d[1] = d[2] = d[3] = 0.0f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < p.tp) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          stale |= (unsigned int)(w[r][e] >> 32) ^ want;
          d[e] += __uint_as_float((unsigned int)w[r][e]);
        }
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
#pragma unroll 1
  for (int it = cta + G * warp; it < items; it += G * NW)
    reduce_tile(p, nullptr, p.x0, weight, false, ssq_out, it / tiles, it % tiles, lane, 0, epoch);
  fence_proxy_async_global();  // xw is read by TMA (async proxy) after the barrier
}

// 1/rms of every token from the per-tile sums of squares -> shared memory
__device__ __noinline__ void load_rstd(const DLParams& p, const float* ssq, float* s_rstd, int wtid) {
  const int warp = wtid >> 5, lane = wtid & 31;
  const int tiles = p.H / BM;
#pragma unroll 1
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
  // gate and up slabs are requested together (one memory round trip), then summed slab by slab
  constexpr int SU = 4;
  const float* gb = g.part + (size_t)t * g.M + col;
  const float* ub = gb + I;
  float4 gv[SU], uv[SU];
#pragma unroll
  for (int s2 = 0; s2 < SU; ++s2) {
    gv[s2] = make_float4(0.f, 0.f, 0.f, 0.f);
    uv[s2] = gv[s2];
    if (s2 < n0) gv[s2] = __ldcg(reinterpret_cast<const float4*>(gb + (size_t)s2 * g.slab_stride));
    if (s2 < n1) uv[s2] = __ldcg(reinterpret_cast<const float4*>(ub + (size_t)s2 * g.slab_stride));
  }
  float gs[4] = {gv[0].x, gv[0].y, gv[0].z, gv[0].w}, us[4] = {uv[0].x, uv[0].y, uv[0].z, uv[0].w};
#pragma unroll
  for (int s2 = 1; s2 < SU; ++s2) {
    gs[0] += gv[s2].x; gs[1] += gv[s2].y; gs[2] += gv[s2].z; gs[3] += gv[s2].w;
    us[0] += uv[s2].x; us[1] += uv[s2].y; us[2] += uv[s2].z; us[3] += uv[s2].w;
  }
#pragma unroll 1
  for (int s2 = SU; s2 < max(n0, n1); ++s2) {
    if (s2 < n0) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(gb + (size_t)s2 * g.slab_stride));
      gs[0] += v.x; gs[1] += v.y; gs[2] += v.z; gs[3] += v.w;
    }
    if (s2 < n1) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(ub + (size_t)s2 * g.slab_stride));
      us[0] += v.x; us[1] += v.y; us[2] += v.z; us[3] += v.w;
    }
  }
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
  float rope_cos[MAX_T][64];  // bf16-rounded cosine / sine of every token's rotary angles: the same for all layers
  float rope_sin[MAX_T][64];
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

// NB bytes (4, 8, 16 or 32) of a token row held exactly as the vector loads deliver them.  The
// loaded registers must not be copied before they are used: a move of a loaded value makes the
// warp wait for that load, and the loads of a batch would then complete one after another
// instead of together.  word(i) is resolved at compile time inside unrolled loops.
template <int NB>
struct KvReg;
template <>
struct KvReg<4> {
  uint32_t a;
  __device__ __forceinline__ void load(const uint8_t* src) { a = __ldcg(reinterpret_cast<const uint32_t*>(src)); }
  __device__ __forceinline__ uint32_t word(int) const { return a; }
};
template <>
struct KvReg<8> {
  uint2 a;
  __device__ __forceinline__ void load(const uint8_t* src) { a = __ldcg(reinterpret_cast<const uint2*>(src)); }
  __device__ __forceinline__ uint32_t word(int i) const { return i == 0 ? a.x : a.y; }
};
template <>
struct KvReg<16> {
  uint4 a;
  __device__ __forceinline__ void load(const uint8_t* src) { a = __ldcg(reinterpret_cast<const uint4*>(src)); }
  __device__ __forceinline__ uint32_t word(int i) const { return i == 0 ? a.x : (i == 1 ? a.y : (i == 2 ? a.z : a.w)); }
};
template <>
struct KvReg<32> {
  uint4 a, b;
  __device__ __forceinline__ void load(const uint8_t* src) {
    a = __ldcg(reinterpret_cast<const uint4*>(src));
    b = __ldcg(reinterpret_cast<const uint4*>(src) + 1);
  }
  __device__ __forceinline__ uint32_t word(int i) const {
    return i == 0 ? a.x : (i == 1 ? a.y : (i == 2 ? a.z : (i == 3 ? a.w : (i == 4 ? b.x : (i == 5 ? b.y : (i == 6 ? b.z : b.w))))));
  }
};
template <>
struct KvReg<64> {
  uint4 a, b, c, d;
  __device__ __forceinline__ void load(const uint8_t* src) {
    a = __ldcg(reinterpret_cast<const uint4*>(src));
    b = __ldcg(reinterpret_cast<const uint4*>(src) + 1);
    c = __ldcg(reinterpret_cast<const uint4*>(src) + 2);
    d = __ldcg(reinterpret_cast<const uint4*>(src) + 3);
  }
  __device__ __forceinline__ uint32_t word(int i) const {
    const uint4& v = i < 4 ? a : (i < 8 ? b : (i < 12 ? c : d));
    const int k = i & 3;
    return k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w));
  }
};

// One (sequence, KV head, split) item on all worker warps.
//
// Lane layout: the GQ query heads of the KV head sit side by side in a warp (32 / GQ lanes per
// head, D / (32 / GQ) head-dimension elements per lane), and a warp handles one cached token at a
// time: the token's K and V slices are loaded once per slice (lanes of different heads read the
// same address) and every head scores it in parallel.  The per-token body is a few dozen
// instructions, so the loop stays in the instruction cache; tokens go through in batches of UNR
// with all loads of a batch in flight together.
template <int D, int GQ, bool KV8>
__device__ __noinline__ void attn_item(const DLParams& p, const LayerDesc& L, WorkerSmem& ws, int b, int kvh, int split,
                                       int wtid) {
  constexpr int LPH = 32 / GQ;               // lanes per head
  constexpr int EPL = D / LPH;               // head-dimension elements per lane
  constexpr int KB = EPL * (KV8 ? 1 : 2);    // bytes of a token row per lane
  constexpr int NWORD = KB / 4;
  constexpr int UNR = 4;                     // tokens per warp with loads in flight together
  constexpr int PER = D / 64;
  static_assert(EPL >= 4 && KB >= 4, "lane slice too small");
  AttnScratch& sc = ws.attn;
  const StepConst& cst = ws.step;
  const int G = gridDim.x;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int g = lane / LPH, part = lane % LPH;
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
  constexpr int QUANT = NW * UNR;
  const int per_split = ((ctx + p.nsplit - 1) / p.nsplit + QUANT - 1) / QUANT * QUANT;
  const int j_begin = split * per_split;
  const int j_end = min(ctx, j_begin + per_split);
  const bool owner = ctx > 0 && ctx - 1 >= j_begin && ctx - 1 < j_begin + per_split;  // this split sees the new token
  const int j_stop = owner ? min(j_end, ctx - 1) : j_end;  // the new token comes from shared memory
  const float rstd = sc.rstd[b];
  const GemmGeo& gq = p.geo[0];
  const int* bt = (cst.bt_ok != 0) ? cst.bt + b * p.max_blocks : p.block_tables + (size_t)b * p.max_blocks;

  // One batch: tokens j0 + u * NW (u < UNR) of this warp.  The loaded registers are not touched
  // before they are used (a move of a loaded value would make the warp wait for that load).
  KvReg<KB> kw[UNR], vw[UNR];
  float ks[UNR], vs[UNR];
  bool valid[UNR];
  auto load_batch = [&](int j0) {
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int j = j0 + u * NW;
      int blk = -1;
      if (j < j_stop) {
        blk = bt[j >> p.page_shift];
        if (p.num_blocks > 0 && blk >= p.num_blocks) {
          if (lane == 0) prism_report(PRISM_ERR_BOUNDS, 2);
          blk = -1;
        }
      }
      valid[u] = blk >= 0;
      ks[u] = 1.0f;
      vs[u] = 1.0f;
      if (valid[u]) {
        const size_t row = ((size_t)blk * p.Hkv + kvh) * p.page + (j & (p.page - 1));
        const size_t off = row * D * (KV8 ? 1 : 2) + (size_t)part * KB;
        kw[u].load(reinterpret_cast<const uint8_t*>(L.k_cache) + off);
        vw[u].load(reinterpret_cast<const uint8_t*>(L.v_cache) + off);
        if (KV8 && p.kv_mode == 2) {
          ks[u] = __ldcg(L.k_scale + row);
          vs[u] = __ldcg(L.v_scale + row);
        }
      }
    }
  };
  // ---- split-KV attention over the cached tokens [j_begin, j_stop) ------------------------------------
  float q[EPL];
  float m = -INFINITY, l = 0.0f, acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc[e] = 0.0f;

  // one token for every head of the warp: kf / vf are this lane's slice of the token's K / V row
  auto fold = [&](const float (&kf)[EPL], const float (&vf)[EPL], float kscale, float vscale) {
    float sdot = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) sdot += q[e] * kf[e];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, o);
    sdot *= kscale;
    const float mn = fmaxf(m, sdot);
    const float corr = __expf(m - mn);
    const float pr = __expf(sdot - mn);
    l = l * corr + pr;
    const float pv = pr * vscale;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * corr + pv * vf[e];
    m = mn;
  };

  // The loads of a batch are in flight while the previous batch is folded; the q / k / v rows are
  // built inside the first pass, after the first batch (which does not depend on them) was requested.
  const int j_first = j_begin + warp;
  bool first_pass = true;
#pragma unroll 1
  for (int j0 = j_first;; j0 += NW * UNR) {
    const bool have = j0 < j_stop;
    if (have) load_batch(j0);
    if (first_pass) {
      first_pass = false;
  // ---- rows of the packed QKV projection this item needs: GQ query heads (+ K and V of the new token)
  const int nrows = GQ + (owner ? 2 : 0);
#pragma unroll 1
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
      constexpr int SU = 4;  // slabs whose loads are in flight together
      float v0[SU][PER], v1[SU][PER];
#pragma unroll
      for (int s = 0; s < SU; ++s)
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
        for (int s = 1; s < SU; ++s) {
          s0 += v0[s][j];
          s1 += v1[s][j];
        }
#pragma unroll 1
        for (int s = SU; s < n; ++s) {
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
        const float cs = cst.rope_cos[b][i], sn = cst.rope_sin[b][i];
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
#pragma unroll
      for (int e = 0; e < EPL; ++e) q[e] = sc.q[g * D + part * EPL + e] * p.attn_scale;
    }
    if (!have) break;
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      if (!valid[u]) continue;  // the same for every lane of the warp
      float kf[EPL], vf[EPL];
      if (KV8) {
#pragma unroll
        for (int w = 0; w < NWORD; ++w) {
          const uint32_t kword = kw[u].word(w), vword = vw[u].word(w);
          const float2 k0 = fp8x2_to_float2((unsigned short)(kword & 0xffffu)), k1 = fp8x2_to_float2((unsigned short)(kword >> 16));
          const float2 v0 = fp8x2_to_float2((unsigned short)(vword & 0xffffu)), v1 = fp8x2_to_float2((unsigned short)(vword >> 16));
          kf[4 * w] = k0.x; kf[4 * w + 1] = k0.y; kf[4 * w + 2] = k1.x; kf[4 * w + 3] = k1.y;
          vf[4 * w] = v0.x; vf[4 * w + 1] = v0.y; vf[4 * w + 2] = v1.x; vf[4 * w + 3] = v1.y;
        }
      } else {
#pragma unroll
        for (int w = 0; w < NWORD; ++w) {
          const uint32_t kword = kw[u].word(w), vword = vw[u].word(w);
          const float2 kk = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kword));
          const float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vword));
          kf[2 * w] = kk.x; kf[2 * w + 1] = kk.y;
          vf[2 * w] = vv.x; vf[2 * w + 1] = vv.y;
        }
      }
      fold(kf, vf, ks[u], vs[u]);
    }
  }
  if (owner && warp == 0) {  // the new token, from shared memory
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kf[e] = sc.kn[part * EPL + e];
      vf[e] = sc.vn[part * EPL + e];
    }
    fold(kf, vf, sc.kv_scale[0], sc.kv_scale[1]);
  }
  sub_stamp();
  // merge the warps in two rounds through NW / 2 shared-memory slots
  constexpr int HW = NW / 2;
  auto put = [&](int slotw) {
    if (part == 0) {
      sc.m[slotw][g] = m;
      sc.l[slotw][g] = l;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sc.acc[(slotw * GQ + g) * D + part * EPL + e] = acc[e];
  };
  if (warp >= HW) put(warp - HW);
  named_bar_sync(1, NWT);
  if (warp < HW) {
    const float mo = sc.m[warp][g], lo2 = sc.l[warp][g];
    const float mn = fmaxf(m, mo);
    const float c0 = (m == -INFINITY) ? 0.0f : __expf(m - mn);
    const float c1 = (mo == -INFINITY) ? 0.0f : __expf(mo - mn);
    l = l * c0 + lo2 * c1;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * c0 + sc.acc[(warp * GQ + g) * D + part * EPL + e] * c1;
    m = mn;
    __syncwarp();
    put(warp);
  }
  named_bar_sync(1, NWT);
  sub_stamp();
  const int ns = p.nsplit;
#pragma unroll 1
  for (int idx = wtid; idx < GQ * D; idx += NWT) {
    const int gg = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < HW; ++w) mm = fmaxf(mm, sc.m[w][gg]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < HW; ++w) {
      const float c = (sc.m[w][gg] == -INFINITY) ? 0.0f : __expf(sc.m[w][gg] - mm);
      ll += sc.l[w][gg] * c;
      oo += sc.acc[(w * GQ + gg) * D + d] * c;
    }
    const int hq = kvh * GQ + gg;
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
#pragma unroll 1
      for (int gg = warp; gg < GQ; gg += NW) {
        const size_t bh = (size_t)b * p.Hq + kvh * GQ + gg;
        const float ms = lane < ns ? __ldcg(&p.part_ml[(bh * ns + lane) * 2]) : -INFINITY;
        const float ls = lane < ns ? __ldcg(&p.part_ml[(bh * ns + lane) * 2 + 1]) : 0.0f;
        const float mm = warp_max(ms);
        const float c = (ms == -INFINITY) ? 0.0f : __expf(ms - mm);
        const float ll = warp_sum(ls * c);
        sc.coef[gg][lane] = c;
        if (lane == 0) sc.inv[gg] = ll > 0.0f ? 1.0f / ll : 0.0f;
      }
      named_bar_sync(1, NWT);
#pragma unroll 1
      for (int idx = wtid; idx < GQ * D; idx += NWT) {
        const int gg = idx / D, d = idx % D;
        const size_t bh = (size_t)b * p.Hq + kvh * GQ + gg;
        const float* po = p.part_o + bh * ns * D + d;
        // eight partial loads in flight at a time (a plain loop would pay one round trip per split)
        float oo = 0.0f;
#pragma unroll 1
        for (int s0 = 0; s0 < ns; s0 += 8) {
          float pv[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) pv[k] = s0 + k < ns ? __ldcg(po + (size_t)(s0 + k) * D) : 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) oo += pv[k] * sc.coef[gg][(s0 + k) & 31];
        }
        p.attn[bh * D + d] = __float2bfloat16_rn(oo * sc.inv[gg]);
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
#pragma unroll 1
  for (int it = blockIdx.x; it < items; it += G) {
    const int split = it % p.nsplit;
    const int kvh = (it / p.nsplit) % p.Hkv;
    const int b = it / (p.nsplit * p.Hkv);
#define PRISM_ATTN_CASE(GQ_)                                                   \
  case GQ_:                                                                    \
    if constexpr (D * GQ_ >= 128) { /* at least four elements per lane */      \
      if (kv8) attn_item<D, GQ_, true>(p, L, ws, b, kvh, split, wtid);         \
      else attn_item<D, GQ_, false>(p, L, ws, b, kvh, split, wtid);            \
    }                                                                          \
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

// ---- GEMM epilogue -------------------------------------------------------------------------------
// Epilogue of GEMM g of layer l: TMEM -> fp32 slab [slab][t][m].  For o_proj, gate/up and down the
// CTA that delivers the LAST partial of a weight tile (arrival counter per tile, the classic fence
// / counter / fence hand-off) runs the pointwise step on that tile's 128 columns right away: the
// reduce into the residual (+ the activation of the next GEMM and the sums of squares), or SwiGLU
// once the gate tile and its up tile are both complete.  No grid barrier stands between a
// projection and its consumer, and the tails of 32 to 96 tiles run on as many CTAs in parallel
// instead of on the few that a separate phase would keep busy.
__device__ __noinline__ void epilogue_gemm(const DLParams& p, WorkerCtx& c, int g, int l) {
  const GemmGeo& geo = p.geo[g];
  const int G = gridDim.x, cta = blockIdx.x;
  AttnScratch& sc = c.ws->attn;
  const int u0 = sk_start(cta, geo.U, G), u1 = sk_start(cta + 1, geo.U, G);
  const int pair = p.I / BM;  // gate tile m and up tile m + pair feed the same activation tile
  int u = u0;
  while (u < u1) {
    const int m = u / geo.kb;
    const int tile_end = (m + 1) * geo.kb;
    const int seg_end = tile_end < u1 ? tile_end : u1;
    if (c.ww < 4) {
      const int a = c.segc % NACC;
      if (c.ok) c.ok = mbar_wait_a(&c.acc_full[a], (uint32_t)(c.segc / NACC) & 1, p, 300);
      // warp-wide TMEM access stays convergent: the wait result is the same for the whole warp
      // only after the vote
      c.ok = __all_sync(0xffffffffu, c.ok);
      if (c.ok) {
        tc_fence_after();
        const int q = (c.warp & 3);
        uint32_t r[16];
        tmem_ld16(c.tmem_base + a * BN + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        tc_fence_before();
        if (c.lane == 0) mbar_arrive(&c.acc_empty[a]);
        const int row = m * BM + q * 32 + c.lane;
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
        if (c.wtid == 0) {
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
          const bool last = c.ok && old == need - 1;
          if (old == need - 1) *cnt = 0;  // self-resetting: the next layer's arrivals come after a grid barrier
          sc.tail_tile = last ? tile : -1;
        }
        named_bar_sync(2, 128);
        const int tile = sc.tail_tile;
        if (tile >= 0) {
          __threadfence();
          if (g == 2) {
#pragma unroll 1
            for (int t = c.ww; t < p.T; t += 4) swiglu_tile(p, sc.rstd_post[t], t, tile, c.lane);
          } else {
            // o_proj feeds the post-attention norm of this layer, down the input norm of the next one
            // (none after the last layer: only the residual, the pre-norm hidden state, is written)
            const bf16* w = g == 1 ? p.layers[l].norm_post : (l + 1 < p.n_layers ? p.layers[l + 1].norm_in : nullptr);
            float* ssq = g == 1 ? p.ssq + MAX_T * SSQ_STRIDE : p.ssq;
#pragma unroll 1
            for (int t = c.ww; t < p.T; t += 4) reduce_tile(p, &geo, nullptr, w, true, ssq, t, tile, c.lane, 2 * l + (g == 1 ? 1 : 2), c.epoch);
          }
          fence_proxy_async_global();  // xw / act are read by TMA (async proxy) after the barrier
        }
      }
    }
    ++c.segc;
    u = seg_end;
  }
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
                     const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ DLParams p) {
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
    WorkerSmem& ws = *reinterpret_cast<WorkerSmem*>(scratch);
    AttnScratch& sc = ws.attn;
    WorkerCtx c;
    c.acc_full = acc_full;
    c.acc_empty = acc_empty;
    c.tmem_base = tmem_base;
    c.s_abort = s_abort;
    c.s_xphase = s_xphase;
    c.ws = &ws;
    c.wtid = threadIdx.x - 64;
    c.ww = c.wtid >> 5;  // worker warp 0..7; warps 0..3 also run the epilogues
    c.lane = lane;
    c.warp = warp;
    c.segc = 0;
    c.ok = true;
    c.epoch = (p.tp > 1 && p.epoch != nullptr) ? *p.epoch : 0ull;
    c.bar_target = 0ull;
    const int wtid = c.wtid;

    {  // per-step inputs every layer reads again
      StepConst& cst = ws.step;
      const int half = D / 2;
      for (int i = wtid; i < MAX_T; i += NWT) {
        cst.ctx[i] = i < p.T ? p.context_lens[i] : 0;
        cst.slots[i] = i < p.T ? p.slots[i] : -1;
      }
      // rotary angles depend on the token and the frequency slot, not on the layer: evaluated once
      // per launch (position of the slot's axis times its inverse frequency; bf16 like the eager graph)
      for (int i = wtid; i < p.T * half; i += NWT) {
        const int t = i / half, f = i % half;
        const int ax = min(2, max(0, p.axis[f]));
        float sn, cs;
        sincosf((float)p.positions[(size_t)ax * p.T + t] * p.inv_freq[f], &sn, &cs);
        cst.rope_cos[t][f] = bf16_round(cs);
        cst.rope_sin[t][f] = bf16_round(sn);
      }
      const int n_bt = p.T * p.max_blocks;
      if (wtid == 0) {
        cst.bt_ok = n_bt <= BT_CACHE ? 1 : 0;
        ws.tl_attn = nullptr;
      }
      if (n_bt <= BT_CACHE)
        for (int i = wtid; i < n_bt; i += NWT) cst.bt[i] = p.block_tables[i];
      named_bar_sync(1, NWT);
    }
    int stamp_i = 0;
    long long* tl = nullptr;
    auto stamp = [&]() {
      if (tl != nullptr && wtid == 0 && stamp_i < TL_PHASES) tl[stamp_i++] = clock64();
    };
    bool ok = true;
    for (int l = 0; l < p.n_layers && ok; ++l) {
      const LayerDesc& L = p.layers[l];
      if (p.timeline != nullptr) tl = p.timeline + ((size_t)cta * p.n_layers + l) * TL_STAMPS;
      stamp_i = 0;
      stamp();
      if (l == 0) {
        // the embedding rows become the residual and the activation of the first QKV GEMM
        reduce_phase_x0(p, L.norm_in, p.ssq, wtid, c.epoch);
        stamp();
        if (!(ok = grid_barrier(p, c, 1))) break;
        stamp();
      } else {
        stamp();
        stamp();
      }
      // phases: 0 QKV GEMM | 1 q/k/v rows, KV store, attention | 2 o_proj (+ reduce tails) |
      // 3 gate/up (+ SwiGLU tails) | 4 down (+ reduce tails); a grid barrier after each
#pragma unroll 1
      for (int ph = 0; ph < 5 && ok; ++ph) {
        if (ph == 1) {
          if (wtid == 0) ws.tl_attn = tl != nullptr ? tl + TL_PHASES : nullptr;
          load_rstd(p, p.ssq, sc.rstd, wtid);
          attn_phase<D>(p, L, ws, wtid);
        } else {
          const int g = ph == 0 ? 0 : ph - 1;
          if (g == 2) load_rstd(p, p.ssq + MAX_T * SSQ_STRIDE, sc.rstd_post, wtid);  // the SwiGLU tails need the post-attention 1/rms
          epilogue_gemm(p, c, g, l);
        }
        stamp();
        // activations the producer may load after this barrier: o_proj's after attention, gate/up's
        // after the o_proj tails, down's after the SwiGLU tails, the next layer's QKV after the down tails
        const int xv = ph == 0 ? 0 : (ph < 4 ? l * 4 + ph + 1 : (l + 1) * 4 + 1);
        ok = grid_barrier(p, c, xv);
        stamp();
      }
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
  if ((GQ != 1 && GQ != 2 && GQ != 4 && GQ != 8) || GQ * D > 512 || GQ * D < 128) return -5;
  if (m_qkv != (p.Hq + 2 * p.Hkv) * D) return -6;
  if (p.H % 128 || p.I % 128 || p.H > 8192 || p.H / BM > TILE_COUNTERS || p.I / BM > TILE_COUNTERS) return -7;
  if (p.nsplit < 1 || p.nsplit > 32 || p.page <= 0 || (p.page & (p.page - 1)) || p.max_blocks <= 0) return -8;
  p.page_shift = 0;
  while ((1 << p.page_shift) < p.page) ++p.page_shift;
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
