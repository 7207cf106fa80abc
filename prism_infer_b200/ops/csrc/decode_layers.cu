// Persistent decode kernel: every decoder layer of one decode step (at most 4 tokens) in ONE
// launch, organised as a dataflow over the SMs.
//
// The per-layer chain of the reference (prism_infer/models/qwen3_vl.py:925-1022 under
// prism_infer/engine/model_runner.py:1219-1313) is add+RMSNorm -> QKV GEMM -> QK-norm + M-RoPE +
// KV store -> paged attention -> o_proj -> add+RMSNorm -> gate/up GEMM + SwiGLU -> down_proj: eight
// launches per layer even when every op is one kernel.  A decode step of a few tokens is one pass
// over the weights plus a chain of tiny all-to-all hand-offs; a kernel boundary (or a grid-wide
// barrier, which costs the same few microseconds: fence, atomic, poll) at each of them is what
// bounds the step once the weights stream at full rate.  Here one CTA per SM stays resident for
// the whole step and NOTHING synchronises globally:
//
//   * every value that crosses CTAs travels as one 8-byte word {fp32 value, sequence number}.  An
//     aligned 8-byte store is single-copy atomic, so a consumer that polls the word and sees this
//     hand-off's sequence number also has the value: no fence, no flag, no atomic, no barrier;
//     one memory round trip after the producer's store.  Sequence numbers grow with (launch,
//     layer, hand-off), buffers are reused every layer, and a slow reader can never meet a word
//     of a later hand-off: every hand-off is followed by a GEMM that needs ALL CTAs' units before
//     its buffer is written again.
//   * warp 0 is the producer: one lane issues the TMA loads of the CTA's weight tiles (stream-K
//     run of (tile, k-block) units of every GEMM of every layer, through a shared-memory ring);
//     the activation tile of a stage is copied by the warp from the CTA's own shared-memory copy
//     of the activation vector.  Weight loads run ahead across hand-offs and layers.
//   * warp 1 issues tcgen05.mma into rotating TMEM accumulators.
//   * warps 2..9 (workers) poll the activations the CTA's units need into shared memory, run the
//     epilogues (TMEM -> fp32 partial words) and the pointwise work the CTA OWNS: each 128-column
//     tile of the residual stream has one owner CTA that sums the partials of o_proj / down,
//     keeps that slice of the residual in shared memory, and publishes residual * norm weight
//     and the slice's sum of squares (the row's 1/rms is a scalar the consumers apply); each
//     activation tile has an owner that applies SwiGLU; each (sequence, KV head, split) has a CTA
//     that builds its q / k / v rows, stores the new token's K / V and attends over cached tokens
//     that bulk copies stage in shared memory, the first chunks one layer ahead; split 0 merges
//     the splits.
//
// One GPU only: tensor-parallel ranks run the per-layer chain, whose exchanges are fused into its
// kernels.
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
typedef unsigned long long u64;

constexpr int BM = 128, BK = 64, BN = 16, UMMA_K = 16;
constexpr int W_TILE_BYTES = BM * BK * 2;   // 16 KB
constexpr int X_TILE_BYTES = BN * BK * 2;   // 2 KB
constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
constexpr int NW = 8;                        // worker warps
constexpr int NWT = NW * 32;                 // worker threads
constexpr int NTHREADS = 64 + NWT;
constexpr int NACC = 4;                      // TMEM accumulators (16 fp32 columns each)
constexpr int TMEM_COLS = 64;
constexpr int TMAX = 4;                      // tokens per step
constexpr int KV_SLOTS = 2;                  // staged chunks of cached tokens in flight
constexpr int KV_SLOT_BYTES = 16 * 1024;     // K rows in the first half, V rows in the second
constexpr int KV_CHUNK_MAX = 64;             // tokens per chunk at most
constexpr int BT_CACHE = 512;                // block-table entries kept in shared memory
constexpr int SMEM_LIMIT = 232448;
constexpr int MAX_STAGES = 12;
constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN);
constexpr float FP8_MAX = 448.0f;
constexpr float FP8_SCALE_FLOOR = 1.0e-6f;
constexpr long long UNWIND_CYCLES = 4000000ll;  // in-flight copies land within microseconds
constexpr int SEQ_PER_LAYER = 16;
constexpr int SLAB_UNROLL = 8;               // slabs polled together

// hand-offs of a layer (sequence number = launch base + layer * SEQ_PER_LAYER + id); HO_XW_IN of
// layer l is produced at the end of layer l - 1 (or from the embedding rows)
enum : int { HO_XW_IN = 0, HO_QKV = 1, HO_ATTN_PART = 2, HO_ATTN = 3, HO_OPROJ = 4, HO_XW_POST = 5, HO_GATE_UP = 6, HO_ACT = 7, HO_DOWN = 8 };

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
  long long slab_stride;  // words between slabs (T * M)
  u64* part;     // [P][T][M] packed words
};

struct DLParams {
  const LayerDesc* layers;
  int n_layers;
  int T;
  int H, Hq, Hkv, I;
  int page, page_shift, max_blocks, num_blocks, kv_mode;
  int nsplit;
  int stages;
  int xslots;                // k-blocks of activations a CTA keeps per token
  int pf_depth;              // units the L2 prefetch cursor may run ahead of the ring (0: off)
  float eps, attn_scale;
  GemmGeo geo[4];
  const u64* state;          // device words {sequence base of this launch, wrap generation}: advanced before every launch
  const bf16* x0;            // [T][H] embedding rows
  const int* positions;      // [3][T]
  const long long* slots;    // [T]
  const int* block_tables;   // [T][max_blocks]
  const int* context_lens;   // [T]
  const float* inv_freq;     // [D/2]
  const int* axis;           // [D/2]
  bf16* out;                 // [T][H] hidden state before the final norm
  u64* xw_in;                // [T][H]   residual * input-norm weight
  u64* xw_post;              // [T][H]   residual * post-attention-norm weight
  u64* ssq_in;               // [T][64]  sums of squares per residual tile
  u64* ssq_post;             // [T][64]
  u64* attn_part;            // [T][Hq][nsplit][D + 2]  split partials (o, max, sum)
  u64* attn;                 // [T][Hq * D]
  u64* act;                  // [T][I]
  int* abort_flag;           // zero; set when a wait ran out
  long long* timeline;       // optional [grid][n_layers][TL_STAMPS] nanosecond stamps of the GPU-wide timer (null: off)
};
constexpr int TL_STAMPS = 16;

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
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
// number of partial slabs of weight tile m (one per contributing CTA)
__device__ __forceinline__ int sk_tile_slabs(const GemmGeo& g, int m, int G) {
  const int u0 = m * g.kb;
  return sk_owner(u0 + g.kb - 1, g.U, G) - sk_owner(u0, g.U, G) + 1;
}
// Owner CTA of tile m out of n tiles (n <= G): spread over the grid.
__host__ __device__ __forceinline__ int tile_owner(int m, int n, int G) { return (int)((long long)m * G / n); }
// The k-blocks of activations CTA `cta` needs for its units of a GEMM: kb0, kb0 + 1, ... (cyclic), `count` of them.
__host__ __device__ __forceinline__ void gemm_window(int U, int kb, int cta, int G, int& kb0, int& count) {
  const int u0 = sk_start(cta, U, G), u1 = sk_start(cta + 1, U, G);
  if (u1 - u0 >= kb) {
    kb0 = 0;
    count = kb;
  } else {
    kb0 = u0 % kb;
    count = u1 - u0;
  }
}

// ---- packed words --------------------------------------------------------------------------------
__device__ __forceinline__ u64 pack(uint32_t seq, float v) { return ((u64)seq << 32) | (u64)__float_as_uint(v); }
__device__ __forceinline__ uint32_t seq_of_word(u64 w) { return (uint32_t)(w >> 32); }
__device__ __forceinline__ float val_of_word(u64 w) { return __uint_as_float((uint32_t)w); }
__device__ __forceinline__ void st_word(u64* dst, u64 w) { asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(dst), "l"(w) : "memory"); }
__device__ __forceinline__ void st_word2(u64* dst, u64 w0, u64 w1) {
  asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(w0), "l"(w1) : "memory");
}
__device__ __forceinline__ void ld_word2(const u64* src, u64& w0, u64& w1) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(src) : "memory");
}
__device__ __forceinline__ u64 ld_word(const u64* src) {
  u64 w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
  return w;
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
// Poll bookkeeping: `spins` counts failed attempts of one wait; every 64 of them the abort word
// and the clock are looked at.  Returns false when the wait must be given up.
// The rare part of a wait (every 64 failed attempts) exists once in the instruction stream.
__device__ __noinline__ bool poll_check(const DLParams& p, long long t0, int tag) {
  if (aborted(p)) return false;
  if (clock64() - t0 > PRISM_WAIT_CYCLES) {
    raise_abort(p, PRISM_ERR_PEER_TIMEOUT, tag);
    return false;
  }
  return true;
}
struct PollGuard {
  long long t0;
  int spins;
  __device__ __forceinline__ PollGuard() : t0(0), spins(0) {}
  __device__ __forceinline__ bool keep_waiting(const DLParams& p, int tag) {
    if (spins == 0) t0 = clock64();
    if ((++spins & 63) == 0) return poll_check(p, t0, tag);
    return true;
  }
  // for loops whose exit is a warp vote: every lane takes the same decision
  __device__ __forceinline__ bool keep_waiting_warp(const DLParams& p, int tag) {
    return __all_sync(0xffffffffu, keep_waiting(p, tag));
  }
};
__device__ __forceinline__ void st_release_cta(volatile int* addr, int v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(const_cast<int*>(addr))), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cta(volatile int* addr) {
  int v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(const_cast<int*>(addr))) : "memory");
  return v;
}

// Sum of the n slabs of 4 consecutive words: every load of an attempt is in flight together (one
// round trip per attempt); repeated until all words carry `want`.
__device__ __forceinline__ bool poll_slabs4(const DLParams& p, const u64* base, long long stride, int n, uint32_t want,
                                            float (&out)[4], int tag) {
  PollGuard guard;
  for (;;) {
    u64 w[SLAB_UNROLL][4];
#pragma unroll
    for (int s = 0; s < SLAB_UNROLL; ++s) {
      if (s < n) {
        ld_word2(base + (size_t)s * stride, w[s][0], w[s][1]);
        ld_word2(base + (size_t)s * stride + 2, w[s][2], w[s][3]);
      }
    }
    uint32_t stale = 0;
    out[0] = out[1] = out[2] = out[3] = 0.0f;
#pragma unroll
    for (int s = 0; s < SLAB_UNROLL; ++s) {
      if (s < n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          stale |= seq_of_word(w[s][e]) ^ want;
          out[e] += val_of_word(w[s][e]);
        }
      }
    }
#pragma unroll 1
    for (int s = SLAB_UNROLL; s < n; ++s) {  // more contributors than the unrolled window (never at the shapes in use)
      u64 a[4];
      ld_word2(base + (size_t)s * stride, a[0], a[1]);
      ld_word2(base + (size_t)s * stride + 2, a[2], a[3]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        stale |= seq_of_word(a[e]) ^ want;
        out[e] += val_of_word(a[e]);
      }
    }
    if (stale == 0) return true;
    if (!guard.keep_waiting(p, tag)) return false;
  }
}

// ---- shared memory of the workers ----------------------------------------------------------------------
struct WorkerSmem {
  // per launch
  float rope_cos[TMAX][64];    // bf16-rounded cosine / sine of every token's rotary angles: the same for all layers
  float rope_sin[TMAX][64];
  long long slots[TMAX];
  int ctx[TMAX];
  int bt_ok;
  int bt[BT_CACHE];
  // per hand-off
  float rstd[TMAX];            // 1/rms of the layer input (QKV consumer)
  float rstd_post[TMAX];       // 1/rms after attention (gate/up consumer)
  alignas(16) bf16 res_tile[TMAX][BM];        // the residual tile this CTA owns
  // attention
  alignas(128) uint8_t kv[KV_SLOTS][KV_SLOT_BYTES];
  alignas(16) float kscale[KV_SLOTS][KV_CHUNK_MAX];
  alignas(16) float vscale[KV_SLOTS][KV_CHUNK_MAX];
  float q[512];                // [GQ][D] bf16 values as floats
  float kn[128], vn[128];      // the new token's K / V as attention sees them (dequantised payload)
  float kv_scale[2];
  float m[NW / 2][8], l[NW / 2][8];
  float acc[(NW / 2) * 512];   // [NW/2][GQ][D]: warps merge in two rounds
  float coef[8][32];
  float inv[8];
  long long* tl;               // where the current layer's stamps go (null: off)
  int tl_i;
};
// followed by xbuf: bf16 [T][xslots][64], the activation columns the CTA's units of the current GEMM need
constexpr int WS_BYTES = (sizeof(WorkerSmem) + 127) / 128 * 128;

// What a worker thread carries through the steps (the step functions are not inlined: each exists
// once in the instruction stream).
struct WorkerCtx {
  uint64_t* acc_full;
  uint64_t* acc_empty;
  uint64_t* kv_full;           // [KV_SLOTS] staged-chunk barriers
  uint32_t tmem_base;
  volatile int* s_xphase;
  WorkerSmem* ws;
  bf16* xbuf;
  int wtid, ww, lane, warp;    // worker thread / worker warp / lane / warp index inside the CTA
  int segc;                    // accumulator segments consumed so far
  int xphase;                  // activation vectors handed to the producer so far
  int kv_req, kv_done;         // staged chunks requested / consumed so far (slot = count & 1)
  bool ok;
  uint32_t base;               // sequence base of this launch
};
__device__ __forceinline__ uint32_t seq_of(const WorkerCtx& c, int layer, int handoff) {
  return c.base + (uint32_t)(layer * SEQ_PER_LAYER + handoff);
}
__device__ __forceinline__ void stamp(WorkerCtx& c) {
  WorkerSmem& ws = *c.ws;
  if (c.wtid == 0 && ws.tl != nullptr && ws.tl_i < TL_STAMPS) {
    long long ns;  // the GPU-wide timer: stamps of different SMs share one axis
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
    ws.tl[ws.tl_i++] = ns;
  }
}

// ---- owner of a residual tile: delta -> residual, publish residual * weight and the sum of squares -----------
// One warp per token; a lane owns 4 of the tile's 128 columns.  src: the projection whose slabs
// hold the delta (null: the embedding rows x0).  weight null: last layer, the residual is the
// output.
__device__ __noinline__ void reduce_tile(const DLParams& p, WorkerCtx& c, const GemmGeo* src, uint32_t src_seq, const bf16* weight,
                                         u64* xw_out, u64* ssq_out, uint32_t out_seq, int m) {
  WorkerSmem& ws = *c.ws;
  const int H = p.H;
  const int col = m * BM + c.lane * 4;
  const int n = src != nullptr ? sk_tile_slabs(*src, m, gridDim.x) : 0;
#pragma unroll 1
  for (int t = c.ww; t < p.T; t += NW) {
    uint2 w_raw = make_uint2(0, 0);
    if (weight != nullptr) w_raw = __ldg(reinterpret_cast<const uint2*>(weight + col));
    float d[4];
    if (src != nullptr) {
      if (!poll_slabs4(p, src->part + (size_t)t * src->M + col, src->slab_stride, n, src_seq, d, 710)) c.ok = false;
    } else {
      const uint2 x_raw = __ldg(reinterpret_cast<const uint2*>(p.x0 + (size_t)t * H + col));
      const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&x_raw);
      d[0] = b2f(v[0].x); d[1] = b2f(v[0].y); d[2] = b2f(v[1].x); d[3] = b2f(v[1].y);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) d[e] = bf16_round(d[e]);
    bf16* res = &ws.res_tile[t][c.lane * 4];
    if (src != nullptr) {  // the embedding rows start the residual; every later delta is added to it
      const uint2 res_raw = *reinterpret_cast<const uint2*>(res);
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
      u64* dst = xw_out + (size_t)t * H + col;
      st_word2(dst, pack(out_seq, bf16_round(d[0] * b2f(w[0].x))), pack(out_seq, bf16_round(d[1] * b2f(w[0].y))));
      st_word2(dst + 2, pack(out_seq, bf16_round(d[2] * b2f(w[1].x))), pack(out_seq, bf16_round(d[3] * b2f(w[1].y))));
      const float ss = warp_sum(d[0] * d[0] + d[1] * d[1] + d[2] * d[2] + d[3] * d[3]);
      if (c.lane == 0) st_word(ssq_out + t * 64 + m, pack(out_seq, ss));
    } else {
      *reinterpret_cast<uint2*>(p.out + (size_t)t * H + col) = o;
    }
  }
}

// ---- owner of an activation tile: SwiGLU of the gate and up tiles ------------------------------------------------
// act = bf16(bf16(silu(bf16(rstd * sum gate))) * bf16(rstd * sum up)); one warp per token.
__device__ __noinline__ void swiglu_tile(const DLParams& p, WorkerCtx& c, uint32_t src_seq, uint32_t out_seq, int m) {
  WorkerSmem& ws = *c.ws;
  const GemmGeo& g = p.geo[2];
  const int I = p.I, G = gridDim.x;
  const int col = m * BM + c.lane * 4;
  const int n0 = sk_tile_slabs(g, m, G), n1 = sk_tile_slabs(g, m + I / BM, G);
  const int nmax = max(n0, n1);
#pragma unroll 1
  for (int t = c.ww; t < p.T; t += NW) {
    const float rstd = ws.rstd_post[t];
    const u64* gb = g.part + (size_t)t * g.M + col;
    const u64* ub = gb + I;
    float gs[4], us[4];
    // gate and up slabs of the tile are polled together: one round trip per attempt
    constexpr int SU = 4;
    PollGuard guard;
    for (;;) {
      u64 gw[SU][4], uw[SU][4];
#pragma unroll
      for (int s = 0; s < SU; ++s) {
        if (s < n0) {
          ld_word2(gb + (size_t)s * g.slab_stride, gw[s][0], gw[s][1]);
          ld_word2(gb + (size_t)s * g.slab_stride + 2, gw[s][2], gw[s][3]);
        }
        if (s < n1) {
          ld_word2(ub + (size_t)s * g.slab_stride, uw[s][0], uw[s][1]);
          ld_word2(ub + (size_t)s * g.slab_stride + 2, uw[s][2], uw[s][3]);
        }
      }
      uint32_t stale = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) gs[e] = us[e] = 0.0f;
#pragma unroll
      for (int s = 0; s < SU; ++s) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (s < n0) {
            stale |= seq_of_word(gw[s][e]) ^ src_seq;
            gs[e] += val_of_word(gw[s][e]);
          }
          if (s < n1) {
            stale |= seq_of_word(uw[s][e]) ^ src_seq;
            us[e] += val_of_word(uw[s][e]);
          }
        }
      }
#pragma unroll 1
      for (int s = SU; s < nmax; ++s) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (s < n0) {
            const u64 w = ld_word(gb + (size_t)s * g.slab_stride + e);
            stale |= seq_of_word(w) ^ src_seq;
            gs[e] += val_of_word(w);
          }
          if (s < n1) {
            const u64 w = ld_word(ub + (size_t)s * g.slab_stride + e);
            stale |= seq_of_word(w) ^ src_seq;
            us[e] += val_of_word(w);
          }
        }
      }
      if (stale == 0) break;
      if (!guard.keep_waiting(p, 720)) {
        c.ok = false;
        break;
      }
    }
    float a[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) a[e] = bf16_round(bf16_round(silu(bf16_round(gs[e] * rstd))) * bf16_round(us[e] * rstd));
    u64* dst = p.act + (size_t)t * I + col;
    st_word2(dst, pack(out_seq, a[0]), pack(out_seq, a[1]));
    st_word2(dst + 2, pack(out_seq, a[2]), pack(out_seq, a[3]));
  }
}

// ---- activation vector -> shared memory ------------------------------------------------------------------
// Slot s of xbuf holds k-block (kb0 + s) % kb of the CTA's window of GEMM g.  The words are polled
// with eight 16-byte loads in flight per lane; afterwards the producer warp is told (x-phase
// counter) that it may copy activation tiles for this GEMM.  Also fetches the rows' 1/rms when the
// vector is a normalised one (ssq != null).
__device__ __noinline__ void fill_xbuf(const DLParams& p, WorkerCtx& c, int g, const u64* vec, int K, uint32_t seq, const u64* ssq,
                                       float* rstd_out) {
  const GemmGeo& geo = p.geo[g];
  int kb0, count;
  gemm_window(geo.U, geo.kb, blockIdx.x, gridDim.x, kb0, count);
  // items: (token, slot); a lane moves 2 words (columns 2 * lane, 2 * lane + 1 of the slot)
  const int items = p.T * count;
  constexpr int UN = 8;
#pragma unroll 1
  for (int it0 = c.ww * UN; it0 < items; it0 += NW * UN) {
    const u64* src[UN];
    bf16* dst[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int it = min(it0 + u, items - 1);
      const int t = it / count, s = it - t * count;
      int kb = kb0 + s;
      if (kb >= geo.kb) kb -= geo.kb;
      src[u] = vec + (size_t)t * K + kb * BK + c.lane * 2;
      dst[u] = c.xbuf + ((size_t)t * p.xslots + s) * BK + c.lane * 2;
    }
    PollGuard guard;
    for (;;) {
      u64 w[UN][2];
#pragma unroll
      for (int u = 0; u < UN; ++u)
        if (it0 + u < items) ld_word2(src[u], w[u][0], w[u][1]);
      uint32_t stale = 0;
#pragma unroll
      for (int u = 0; u < UN; ++u)
        if (it0 + u < items) stale |= (seq_of_word(w[u][0]) ^ seq) | (seq_of_word(w[u][1]) ^ seq);
      if (!__any_sync(0xffffffffu, stale != 0)) {
#pragma unroll
        for (int u = 0; u < UN; ++u)
          if (it0 + u < items)
            *reinterpret_cast<__nv_bfloat162*>(dst[u]) = __floats2bfloat162_rn(val_of_word(w[u][0]), val_of_word(w[u][1]));
        break;
      }
      if (!guard.keep_waiting_warp(p, 730 + g)) {
        c.ok = false;
        break;
      }
    }
  }
  if (ssq != nullptr && c.ww == NW - 1) {  // one warp fetches the 1/rms of every token
    const int tiles = p.H / BM;
#pragma unroll 1
    for (int t = 0; t < p.T; ++t) {
      PollGuard guard;
      for (;;) {
        u64 a = pack(seq, 0.0f), b = a;
        if (c.lane < tiles) a = ld_word(ssq + t * 64 + c.lane);
        if (c.lane + 32 < tiles) b = ld_word(ssq + t * 64 + c.lane + 32);
        const bool stale = (seq_of_word(a) != seq) || (seq_of_word(b) != seq);
        if (!__any_sync(0xffffffffu, stale)) {
          const float v = warp_sum(val_of_word(a) + val_of_word(b));
          if (c.lane == 0) rstd_out[t] = rsqrtf(v / (float)p.H + p.eps);
          break;
        }
        if (!guard.keep_waiting_warp(p, 740)) {
          c.ok = false;
          break;
        }
      }
    }
  }
  named_bar_sync(1, NWT);
  ++c.xphase;
  if (c.wtid == 0) st_release_cta(c.s_xphase, c.xphase);  // the producer may now copy this GEMM's activation tiles
}

// ---- GEMM epilogue: TMEM -> partial words [slab][t][m] ---------------------------------------------------------
__device__ __noinline__ void epilogue_gemm(const DLParams& p, WorkerCtx& c, int g, uint32_t seq) {
  const GemmGeo& geo = p.geo[g];
  const int G = gridDim.x, cta = blockIdx.x;
  const int u0 = sk_start(cta, geo.U, G), u1 = sk_start(cta + 1, geo.U, G);
  int u = u0;
  while (u < u1) {
    const int m = u / geo.kb;
    const int tile_end = (m + 1) * geo.kb;
    const int seg_end = tile_end < u1 ? tile_end : u1;
    if (c.ww < 4) {
      const int a = c.segc % NACC;
      if (c.ok) c.ok = mbar_wait_a(&c.acc_full[a], (uint32_t)(c.segc / NACC) & 1, p, 300);
      c.ok = __all_sync(0xffffffffu, c.ok);  // the TMEM load is warp-wide
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
          u64* dst = geo.part + (size_t)slab * geo.slab_stride + row;
#pragma unroll
          for (int t = 0; t < TMAX; ++t)
            if (t < p.T) st_word(dst + (size_t)t * geo.M, ((u64)seq << 32) | (u64)r[t]);
        }
      }
    }
    ++c.segc;
    u = seg_end;
  }
}

// ---- attention ---------------------------------------------------------------------------------------
// Geometry of one (sequence, KV head, split) item; the same for every layer (the context is fixed).
struct AttnItem {
  int b, kvh, split;
  int j_begin, j_stop;  // cached tokens this split reads from the pages
  bool owner;           // this split sees the new token (kept in shared memory, never read back)
};
__device__ __forceinline__ AttnItem attn_item_of(const DLParams& p, const WorkerSmem& ws, int it) {
  AttnItem a;
  a.split = it % p.nsplit;
  a.kvh = (it / p.nsplit) % p.Hkv;
  a.b = it / (p.nsplit * p.Hkv);
  int ctx = ws.ctx[a.b];
  const long long reach = (long long)p.max_blocks * p.page;
  if ((long long)ctx > reach) ctx = (int)reach;
  if (ctx < 0) ctx = 0;
  const int per_split = ((ctx + p.nsplit - 1) / p.nsplit + 31) / 32 * 32;
  a.j_begin = a.split * per_split;
  const int j_end = min(ctx, a.j_begin + per_split);
  a.owner = ctx > 0 && ctx - 1 >= a.j_begin && ctx - 1 < a.j_begin + per_split;
  a.j_stop = a.owner ? min(j_end, ctx - 1) : j_end;
  if (a.j_stop < a.j_begin) a.j_stop = a.j_begin;
  return a;
}
template <int D, bool KV8>
struct KvGeo {
  static constexpr int ROW = D * (KV8 ? 1 : 2);  // bytes of a cached row
  static constexpr int CAP = (KV_SLOT_BYTES / 2 / ROW) < KV_CHUNK_MAX ? (KV_SLOT_BYTES / 2 / ROW) : KV_CHUNK_MAX;  // tokens per chunk
  static constexpr int VOFF = KV_SLOT_BYTES / 2;
};
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Bulk copies of the cached tokens [j0, j1) of an item into a slot (K rows, V rows, scales), page
// by page; one thread.  Token offsets inside a page are multiples of 4 (ranges start at multiples
// of 32, chunks and pages are multiples of 4 tokens), so every address and size is a multiple of
// 16 bytes.  Returns the bytes the copies deliver; issues them only when `issue`.
template <int D, bool KV8>
__device__ __forceinline__ uint32_t stage_kv(const DLParams& p, const LayerDesc& L, WorkerSmem& ws, const AttnItem& a, int j0, int j1,
                                             int slot, uint64_t* bar, bool issue) {
  typedef KvGeo<D, KV8> KG;
  const int* bt = (ws.bt_ok != 0) ? ws.bt + a.b * p.max_blocks : p.block_tables + (size_t)a.b * p.max_blocks;
  const bool scaled = KV8 && p.kv_mode == 2;
  uint32_t bytes = 0;
  int j = j0;
  while (j < j1) {
    const int pg = j >> p.page_shift, off = j & (p.page - 1);
    const int n = min(j1 - j, p.page - off);
    const int blk = bt[pg];
    const int n4 = (n + 3) & ~3;  // whole 16-byte groups of scales; stays inside the page
    if (blk >= 0 && (p.num_blocks <= 0 || blk < p.num_blocks)) {
      const size_t row = ((size_t)blk * p.Hkv + a.kvh) * p.page + off;
      const int local = j - j0;
      if (issue) {
        bulk_g2s(ws.kv[slot] + (size_t)local * KG::ROW, reinterpret_cast<const uint8_t*>(L.k_cache) + row * KG::ROW, n * KG::ROW, bar);
        bulk_g2s(ws.kv[slot] + KG::VOFF + (size_t)local * KG::ROW, reinterpret_cast<const uint8_t*>(L.v_cache) + row * KG::ROW, n * KG::ROW,
                 bar);
        if (scaled) {
          bulk_g2s(&ws.kscale[slot][local], L.k_scale + row, n4 * 4, bar);
          bulk_g2s(&ws.vscale[slot][local], L.v_scale + row, n4 * 4, bar);
        }
      }
      bytes += 2u * (uint32_t)(n * KG::ROW);
      if (scaled) bytes += 2u * (uint32_t)(n4 * 4);
    }
    j += n;
  }
  return bytes;
}
// Request chunk k of the item's range for layer l into the next slot.  Thread 0 issues; every
// thread counts.
template <int D, bool KV8>
__device__ __forceinline__ void request_chunk(const DLParams& p, WorkerCtx& c, int l, const AttnItem& a, int k) {
  typedef KvGeo<D, KV8> KG;
  if (c.wtid == 0) {
    const int slot = c.kv_req & (KV_SLOTS - 1);
    const int j0 = a.j_begin + k * KG::CAP, j1 = min(a.j_stop, j0 + KG::CAP);
    const LayerDesc& L = p.layers[l];
    const uint32_t bytes = stage_kv<D, KV8>(p, L, *c.ws, a, j0, j1, slot, &c.kv_full[slot], false);
    mbar_expect_tx(&c.kv_full[slot], bytes);  // one arrival; the phase completes when the bytes have landed (at once if none)
    (void)stage_kv<D, KV8>(p, L, *c.ws, a, j0, j1, slot, &c.kv_full[slot], true);
  }
  ++c.kv_req;
}
template <int D>
__device__ __forceinline__ void request_first_chunks(const DLParams& p, WorkerCtx& c, int l, const AttnItem& a) {
  const int span = a.j_stop - a.j_begin;
  if (p.kv_mode != 0) {
    const int n_ch = (span + KvGeo<D, true>::CAP - 1) / KvGeo<D, true>::CAP;
    for (int k = 0; k < min(KV_SLOTS, n_ch); ++k) request_chunk<D, true>(p, c, l, a, k);
  } else {
    const int n_ch = (span + KvGeo<D, false>::CAP - 1) / KvGeo<D, false>::CAP;
    for (int k = 0; k < min(KV_SLOTS, n_ch); ++k) request_chunk<D, false>(p, c, l, a, k);
  }
}

// One (sequence, KV head, split) item on all worker warps.
//
// Lane layout: the GQ query heads of the KV head sit side by side in a warp (32 / GQ lanes per
// head, D / (32 / GQ) head-dimension elements per lane), and a warp handles one cached token at a
// time from the staged rows: lanes of different heads read the same shared-memory words and
// every head scores the token in parallel.
template <int D, int GQ, bool KV8>
__device__ __noinline__ void attn_item(const DLParams& p, WorkerCtx& c, int l, const AttnItem& a) {
  typedef KvGeo<D, KV8> KG;
  constexpr int LPH = 32 / GQ;               // lanes per head
  constexpr int EPL = D / LPH;               // head-dimension elements per lane
  constexpr int ROW = KG::ROW;
  constexpr int KB = EPL * (KV8 ? 1 : 2);    // bytes of a row per lane
  constexpr int CAP = KG::CAP;
  constexpr int PER = D / 64;
  static_assert(EPL >= 4, "lane slice too small");
  WorkerSmem& ws = *c.ws;
  const LayerDesc& L = p.layers[l];
  const int G = gridDim.x;
  const int wtid = c.wtid, warp = c.ww, lane = c.lane;
  const int g = lane / LPH, part = lane % LPH;
  const int b = a.b, kvh = a.kvh;
  const float rstd = ws.rstd[b];
  const GemmGeo& gq = p.geo[0];
  const uint32_t seq_qkv = seq_of(c, l, HO_QKV);

  // ---- rows of the packed QKV projection this item needs: GQ query heads (+ K and V of the new token)
  const int nrows = GQ + (a.owner ? 2 : 0);
#pragma unroll 1
  for (int r = warp; r < nrows; r += NW) {
    const bool is_q = r < GQ, is_k = r == GQ;
    const int h = is_q ? kvh * GQ + r : (is_k ? p.Hq + kvh : p.Hq + p.Hkv + kvh);
    const int col0 = h * D;
    const int n = sk_tile_slabs(gq, col0 / BM, G);
    const u64* base = gq.part + (size_t)b * gq.M + col0;
    const bf16* nw = is_q ? L.q_norm : L.k_norm;
    bf16 wlo_raw[PER], whi_raw[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {  // norm weights travel together with the slabs (converted only when used)
      wlo_raw[j] = nw[lane + 32 * j];
      whi_raw[j] = nw[lane + 32 * j + D / 2];
    }
    float lo[PER], hi[PER];
    {
      constexpr int SU = 4;  // slabs polled together
      PollGuard guard;
      for (;;) {
        u64 v0[SU][PER], v1[SU][PER];
#pragma unroll
        for (int s = 0; s < SU; ++s)
#pragma unroll
          for (int j = 0; j < PER; ++j)
            if (s < n) {
              v0[s][j] = ld_word(base + (size_t)s * gq.slab_stride + lane + 32 * j);
              v1[s][j] = ld_word(base + (size_t)s * gq.slab_stride + lane + 32 * j + D / 2);
            }
        uint32_t stale = 0;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
          for (int s = 0; s < SU; ++s)
            if (s < n) {
              stale |= (seq_of_word(v0[s][j]) ^ seq_qkv) | (seq_of_word(v1[s][j]) ^ seq_qkv);
              s0 += val_of_word(v0[s][j]);
              s1 += val_of_word(v1[s][j]);
            }
#pragma unroll 1
          for (int s = SU; s < n; ++s) {
            const u64 a0 = ld_word(base + (size_t)s * gq.slab_stride + lane + 32 * j);
            const u64 a1 = ld_word(base + (size_t)s * gq.slab_stride + lane + 32 * j + D / 2);
            stale |= (seq_of_word(a0) ^ seq_qkv) | (seq_of_word(a1) ^ seq_qkv);
            s0 += val_of_word(a0);
            s1 += val_of_word(a1);
          }
          lo[j] = bf16_round(s0 * rstd);
          hi[j] = bf16_round(s1 * rstd);
        }
        if (!__any_sync(0xffffffffu, stale != 0)) break;
        if (!guard.keep_waiting_warp(p, 750)) {
          c.ok = false;
          break;
        }
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
        const float cs = ws.rope_cos[b][i], sn = ws.rope_sin[b][i];
        const float x0 = lo[j], x1 = hi[j];
        lo[j] = bf16_round(bf16_round(x0 * cs) + bf16_round(-x1 * sn));
        hi[j] = bf16_round(bf16_round(x1 * cs) + bf16_round(x0 * sn));
      }
    }
    if (is_q) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        ws.q[r * D + lane + 32 * j] = lo[j];
        ws.q[r * D + lane + 32 * j + D / 2] = hi[j];
      }
      continue;
    }
    // K or V of the new token: quantise as the cache stores it, keep what attention will see
    float* keep = is_k ? ws.kn : ws.vn;
    const long long slot = ws.slots[b];
    long long blk = slot >= 0 ? slot >> p.page_shift : -1;
    if (blk >= 0 && p.num_blocks > 0 && blk >= p.num_blocks) {
      if (lane == 0) prism_report(PRISM_ERR_BOUNDS, 3);
      blk = -1;
    }
    const size_t row = blk >= 0 ? ((size_t)blk * p.Hkv + kvh) * p.page + (size_t)(slot & (p.page - 1)) : 0;
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
      if (lane == 0) ws.kv_scale[is_k ? 0 : 1] = 1.0f;
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
      if (lane == 0) ws.kv_scale[is_k ? 0 : 1] = scale;
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
  stamp(c);

  // ---- split-KV attention over the cached tokens [j_begin, j_stop), chunk by chunk from shared memory ----
  float q[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) q[e] = ws.q[g * D + part * EPL + e] * p.attn_scale;
  float m = -INFINITY, lsum = 0.0f, acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc[e] = 0.0f;
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
    lsum = lsum * corr + pr;
    const float pv = pr * vscale;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * corr + pv * vf[e];
    m = mn;
  };
  const int* bt = (ws.bt_ok != 0) ? ws.bt + b * p.max_blocks : p.block_tables + (size_t)b * p.max_blocks;
  const int n_ch = (a.j_stop - a.j_begin + CAP - 1) / CAP;
  const bool scaled = KV8 && p.kv_mode == 2;
#pragma unroll 1
  for (int k = 0; k < n_ch; ++k) {
    const int j0 = a.j_begin + k * CAP, j1 = min(a.j_stop, j0 + CAP);
    const int slot = c.kv_done & (KV_SLOTS - 1);
    if (c.ok) {
      c.ok = mbar_wait_a(&c.kv_full[slot], (uint32_t)(c.kv_done / KV_SLOTS) & 1, p, 760);
      if (c.ok) ++c.kv_done;
    }
    const uint8_t* kslot = ws.kv[slot];
#pragma unroll 2
    for (int j = j0 + warp; j < j1; j += NW) {
      const int blk = bt[j >> p.page_shift];
      if (blk < 0 || (p.num_blocks > 0 && blk >= p.num_blocks)) continue;  // a hole: not staged, not scored
      const int local = j - j0;
      const uint8_t* kp = kslot + (size_t)local * ROW + part * KB;
      const uint8_t* vp = kp + KG::VOFF;
      uint32_t kw[KB / 4], vw[KB / 4];
      if constexpr (KB % 16 == 0) {
#pragma unroll
        for (int w = 0; w < KB / 16; ++w) {
          const uint4 k4 = *reinterpret_cast<const uint4*>(kp + 16 * w), v4 = *reinterpret_cast<const uint4*>(vp + 16 * w);
          kw[4 * w] = k4.x; kw[4 * w + 1] = k4.y; kw[4 * w + 2] = k4.z; kw[4 * w + 3] = k4.w;
          vw[4 * w] = v4.x; vw[4 * w + 1] = v4.y; vw[4 * w + 2] = v4.z; vw[4 * w + 3] = v4.w;
        }
      } else if constexpr (KB % 8 == 0) {
#pragma unroll
        for (int w = 0; w < KB / 8; ++w) {
          const uint2 k2 = *reinterpret_cast<const uint2*>(kp + 8 * w), v2 = *reinterpret_cast<const uint2*>(vp + 8 * w);
          kw[2 * w] = k2.x; kw[2 * w + 1] = k2.y;
          vw[2 * w] = v2.x; vw[2 * w + 1] = v2.y;
        }
      } else {
#pragma unroll
        for (int w = 0; w < KB / 4; ++w) {
          kw[w] = *reinterpret_cast<const uint32_t*>(kp + 4 * w);
          vw[w] = *reinterpret_cast<const uint32_t*>(vp + 4 * w);
        }
      }
      float kf[EPL], vf[EPL];
      if constexpr (KV8) {
#pragma unroll
        for (int w = 0; w < KB / 4; ++w) {
          const float2 k0 = fp8x2_to_float2((unsigned short)(kw[w] & 0xffffu)), k1 = fp8x2_to_float2((unsigned short)(kw[w] >> 16));
          const float2 v0 = fp8x2_to_float2((unsigned short)(vw[w] & 0xffffu)), v1 = fp8x2_to_float2((unsigned short)(vw[w] >> 16));
          kf[4 * w] = k0.x; kf[4 * w + 1] = k0.y; kf[4 * w + 2] = k1.x; kf[4 * w + 3] = k1.y;
          vf[4 * w] = v0.x; vf[4 * w + 1] = v0.y; vf[4 * w + 2] = v1.x; vf[4 * w + 3] = v1.y;
        }
      } else {
#pragma unroll
        for (int w = 0; w < KB / 4; ++w) {
          const float2 kk = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kw[w]));
          const float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vw[w]));
          kf[2 * w] = kk.x; kf[2 * w + 1] = kk.y;
          vf[2 * w] = vv.x; vf[2 * w + 1] = vv.y;
        }
      }
      fold(kf, vf, scaled ? ws.kscale[slot][local] : 1.0f, scaled ? ws.vscale[slot][local] : 1.0f);
    }
    if (k + KV_SLOTS < n_ch) {
      named_bar_sync(1, NWT);  // every warp is done with this slot
      request_chunk<D, KV8>(p, c, l, a, k + KV_SLOTS);
    }
  }
  if (a.owner && warp == 0) {  // the new token, from shared memory
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kf[e] = ws.kn[part * EPL + e];
      vf[e] = ws.vn[part * EPL + e];
    }
    fold(kf, vf, ws.kv_scale[0], ws.kv_scale[1]);
  }
  stamp(c);
  // merge the warps in two rounds through NW / 2 shared-memory slots
  constexpr int HW = NW / 2;
  auto put = [&](int slotw) {
    if (part == 0) {
      ws.m[slotw][g] = m;
      ws.l[slotw][g] = lsum;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) ws.acc[(slotw * GQ + g) * D + part * EPL + e] = acc[e];
  };
  if (warp >= HW) put(warp - HW);
  named_bar_sync(1, NWT);  // also: every warp is done with the staged rows
  // The next layer's first chunks are requested now: they depend on nothing this step computes
  // (the new token's row is outside the staged range) and land while the other GEMMs run.
  if (l + 1 < p.n_layers)
    for (int k = 0; k < min(KV_SLOTS, n_ch); ++k) request_chunk<D, KV8>(p, c, l + 1, a, k);
  if (warp < HW) {
    const float mo = ws.m[warp][g], lo2 = ws.l[warp][g];
    const float mn = fmaxf(m, mo);
    const float c0 = (m == -INFINITY) ? 0.0f : __expf(m - mn);
    const float c1 = (mo == -INFINITY) ? 0.0f : __expf(mo - mn);
    lsum = lsum * c0 + lo2 * c1;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * c0 + ws.acc[(warp * GQ + g) * D + part * EPL + e] * c1;
    m = mn;
    __syncwarp();
    put(warp);
  }
  named_bar_sync(1, NWT);
  // the split's result: (o[D], max, sum) per head, as words
  const int ns = p.nsplit;
  const uint32_t seq_part = seq_of(c, l, HO_ATTN_PART), seq_attn = seq_of(c, l, HO_ATTN);
  constexpr int PW = D + 2;  // words per (head, split)
#pragma unroll 1
  for (int idx = wtid; idx < GQ * PW; idx += NWT) {
    const int gg = idx / PW, d = idx % PW;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < HW; ++w) mm = fmaxf(mm, ws.m[w][gg]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < HW; ++w) {
      const float cf = (ws.m[w][gg] == -INFINITY) ? 0.0f : __expf(ws.m[w][gg] - mm);
      ll += ws.l[w][gg] * cf;
      if (d < D) oo += ws.acc[(w * GQ + gg) * D + d] * cf;
    }
    const int hq = kvh * GQ + gg;
    if (ns == 1) {
      if (d < D) st_word(p.attn + ((size_t)b * p.Hq + hq) * D + d, pack(seq_attn, bf16_round(ll > 0.0f ? oo / ll : 0.0f)));
    } else {
      const float v = d < D ? oo : (d == D ? mm : ll);
      st_word(p.attn_part + (((size_t)b * p.Hq + hq) * ns + a.split) * PW + d, pack(seq_part, v));
    }
  }
  stamp(c);
  if (ns > 1 && a.split == 0) {
    // split 0 merges all splits of this (sequence, KV head): first the (max, sum) words of every
    // split, then the outputs, each polled with all loads of an attempt in flight
#pragma unroll 1
    for (int gg = warp; gg < GQ; gg += NW) {
      const u64* src = p.attn_part + ((size_t)b * p.Hq + kvh * GQ + gg) * ns * PW;
      PollGuard guard;
      for (;;) {
        u64 wm = pack(seq_part, -INFINITY), wl = pack(seq_part, 0.0f);
        if (lane < ns) ld_word2(src + (size_t)lane * PW + D, wm, wl);
        const bool stale = (seq_of_word(wm) != seq_part) || (seq_of_word(wl) != seq_part);
        if (!__any_sync(0xffffffffu, stale)) {
          const float ms = val_of_word(wm), ls = val_of_word(wl);
          const float mm = warp_max(ms);
          const float cf = (ms == -INFINITY) ? 0.0f : __expf(ms - mm);
          const float ll = warp_sum(ls * cf);
          ws.coef[gg][lane] = cf;
          if (lane == 0) ws.inv[gg] = ll > 0.0f ? 1.0f / ll : 0.0f;
          break;
        }
        if (!guard.keep_waiting_warp(p, 770)) {
          c.ok = false;
          break;
        }
      }
    }
    named_bar_sync(1, NWT);
#pragma unroll 1
    for (int idx = wtid; idx < GQ * D; idx += NWT) {
      const int gg = idx / D, d = idx % D;
      const size_t bh = (size_t)b * p.Hq + kvh * GQ + gg;
      const u64* po = p.attn_part + bh * ns * PW + d;
      float oo = 0.0f;
#pragma unroll 1
      for (int s0 = 0; s0 < ns; s0 += 8) {
        PollGuard guard;
        for (;;) {
          u64 pv[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) pv[k] = s0 + k < ns ? ld_word(po + (size_t)(s0 + k) * PW) : pack(seq_part, 0.0f);
          uint32_t stale = 0;
          float part_sum = 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            stale |= seq_of_word(pv[k]) ^ seq_part;
            part_sum += val_of_word(pv[k]) * ws.coef[gg][(s0 + k) & 31];
          }
          if (stale == 0) {
            oo += part_sum;
            break;
          }
          if (!guard.keep_waiting(p, 780)) {
            c.ok = false;
            break;
          }
        }
      }
      st_word(p.attn + bh * D + d, pack(seq_attn, bf16_round(oo * ws.inv[gg])));
    }
  }
  named_bar_sync(1, NWT);  // scratch is reused
}

template <int D>
__device__ __forceinline__ void attn_dispatch(const DLParams& p, WorkerCtx& c, int l, const AttnItem& a) {
  const int GQ = p.Hq / p.Hkv;
  const bool kv8 = p.kv_mode != 0;
#define PRISM_ATTN_CASE(GQ_)                                                   \
  case GQ_:                                                                    \
    if constexpr (D * GQ_ >= 128) { /* at least four elements per lane */      \
      if (kv8) attn_item<D, GQ_, true>(p, c, l, a);                            \
      else attn_item<D, GQ_, false>(p, c, l, a);                               \
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

// ---- producer cursors ------------------------------------------------------------------------------
struct UnitCursor {
  int l, g;      // layer, GEMM (0 qkv, 1 o_proj, 2 gate/up, 3 down)
  int u, u1;     // unit and end of this CTA's run of the current GEMM
  int m, kb;     // weight tile and k-block of the unit
  int kbn;       // k-blocks per tile of the current GEMM
  int kb0;       // first k-block of the CTA's activation window of the current GEMM
  bool done;
};
__device__ __forceinline__ void cursor_load(UnitCursor& c, const DLParams& p, int cta, int G) {
  const GemmGeo& geo = p.geo[c.g];
  c.u = sk_start(cta, geo.U, G);
  c.u1 = sk_start(cta + 1, geo.U, G);
  c.kbn = geo.kb;
  c.m = c.u / geo.kb;
  c.kb = c.u % geo.kb;
  c.kb0 = (c.u1 - c.u >= geo.kb) ? 0 : c.kb;
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
__global__ void __launch_bounds__(NTHREADS, 1) decode_layers_kernel(const __grid_constant__ DLParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint8_t* scratch = smem + (size_t)stages * STAGE_BYTES;
  WorkerSmem& ws = *reinterpret_cast<WorkerSmem*>(scratch);
  bf16* xbuf = reinterpret_cast<bf16*>(scratch + WS_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(scratch + WS_BYTES + (((size_t)p.T * p.xslots * BK * 2 + 127) & ~(size_t)127));
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;
  uint64_t* acc_empty = acc_full + NACC;
  uint64_t* kv_full = acc_empty + NACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_full + KV_SLOTS);
  volatile int* s_xphase = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, cta = blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 2);  // the weight tile (arrival of the issuing thread + its bytes) and the activation tile copied by the warp
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    for (int s = 0; s < KV_SLOTS; ++s) mbar_init(&kv_full[s], 1);
    *s_xphase = 0;
    fence_barrier_init();
  }
  // rows of the activation tiles beyond the step's tokens stay zero for the whole launch
  for (int i = threadIdx.x; i < stages * (X_TILE_BYTES / 16); i += NTHREADS) {
    const int s = i / (X_TILE_BYTES / 16), k = i % (X_TILE_BYTES / 16);
    *reinterpret_cast<uint4*>(smem + (size_t)s * STAGE_BYTES + W_TILE_BYTES + k * 16) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async();
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =============================== producer warp ===============================
    // Three cursors walk this CTA's units of every GEMM of every layer in order:
    //   P  requests weight tiles into L2 (a hint), up to pf_depth units ahead of W,
    //   W  issues the weight tile of a unit into the next free ring stage (lane 0),
    //   X  copies the unit's activation tile from the CTA's activation vector into the stage (the
    //      whole warp, one 16-byte chunk per lane) once the workers have that vector.
    // W runs ahead of X by at most the ring depth and across hand-offs and layers, so the HBM
    // stream does not stop while the activations of the next GEMM are still being produced.
    UnitCursor P, W, X;
    cursor_begin(P, p, cta, G);
    W = P;
    X = P;
    long long n_p = 0, n_w = 0, n_x = 0;  // units passed by each cursor
    int w_s = 0, x_s = 0;                  // ring stage of the next W / X issue
    uint32_t w_pass = 0;                   // times the W cursor wrapped the ring
    int xphase_seen = 0;
    const int pf_depth = p.pf_depth;
    const int xt = lane >> 3, xc = lane & 7;  // token row and 16-byte chunk this lane copies
    long long t0 = clock64();
    int idle = 0;
    while (!X.done) {
      if (n_x < n_w) {
        const int need = X.l * 4 + X.g + 1;
        if (xphase_seen < need) xphase_seen = ld_acquire_cta(s_xphase);
        if (xphase_seen >= need) {
          if (xt < p.T) {
            int slot = X.kb - X.kb0;
            if (slot < 0) slot += X.kbn;
            const uint4 v = *reinterpret_cast<const uint4*>(xbuf + ((size_t)xt * p.xslots + slot) * BK + xc * 8);
            uint8_t* dst = smem + (size_t)x_s * STAGE_BYTES + W_TILE_BYTES;
            *reinterpret_cast<uint4*>(dst + xt * 128 + ((xc ^ (xt & 7)) << 4)) = v;  // 128-byte swizzle of the operand tile
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[x_s]);
          if (++x_s == stages) x_s = 0;
          cursor_next(X, p, cta, G);
          ++n_x;
          idle = 0;
          continue;
        }
      }
      int did = 0;
      if (lane == 0) {
        if (!W.done && n_w - n_x < stages && (w_pass == 0 || mbar_try_wait(&empty[w_s], (w_pass - 1) & 1))) {
          mbar_expect_tx(&full[w_s], W_TILE_BYTES);
          tma_load_2d(smem + (size_t)w_s * STAGE_BYTES, &p.layers[W.l].tm_w[W.g], &full[w_s], W.kb * BK, W.m * BM);
          did = 1;
        } else if (!P.done && n_p < n_w + pf_depth) {
          if (n_p >= n_w + stages / 2) tma_prefetch_2d(&p.layers[P.l].tm_w[P.g], P.kb * BK, P.m * BM);
        }
      }
      did = __shfl_sync(0xffffffffu, did, 0);
      if (did) {
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
        cursor_next(P, p, cta, G);
        ++n_p;
        idle = 0;
        continue;
      }
      if (idle == 0) t0 = clock64();
      if (++idle >= 64) {
        idle = 1;
        int stop = 0;
        if (lane == 0) {
          if (aborted(p)) stop = 1;
          else if (clock64() - t0 > PRISM_WAIT_CYCLES) {
            raise_abort(p, PRISM_ERR_MBAR_TIMEOUT, 100 + X.g);
            stop = 1;
          }
        }
        if (__shfl_sync(0xffffffffu, stop, 0)) break;
      }
    }
    if (!X.done && lane == 0) {
      // unwinding: weight tiles in flight must land before the CTA's shared memory is released.
      // Stages whose activation tile was never copied get that arrival now; then every stage
      // issued within the last ring pass is awaited (briefly: the copies are microseconds away).
      int s2 = x_s;
      for (long long i = n_x; i < n_w; ++i) {
        mbar_arrive(&full[s2]);
        if (++s2 == stages) s2 = 0;
      }
      s2 = w_s;
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
    WorkerCtx c;
    c.acc_full = acc_full;
    c.acc_empty = acc_empty;
    c.kv_full = kv_full;
    c.tmem_base = tmem_base;
    c.s_xphase = s_xphase;
    c.ws = &ws;
    c.xbuf = xbuf;
    c.wtid = threadIdx.x - 64;
    c.ww = c.wtid >> 5;  // worker warp 0..7; warps 0..3 also run the epilogues
    c.lane = lane;
    c.warp = warp;
    c.segc = 0;
    c.xphase = 0;
    c.kv_req = 0;
    c.kv_done = 0;
    c.ok = true;
    c.base = (uint32_t)p.state[0];
    const int wtid = c.wtid;
    const int r_tiles = p.H / BM, a_tiles = p.I / BM;

    {  // per-launch constants
      const int half = D / 2;
      for (int i = wtid; i < TMAX; i += NWT) {
        ws.ctx[i] = i < p.T ? p.context_lens[i] : 0;
        ws.slots[i] = i < p.T ? p.slots[i] : -1;
      }
      // rotary angles depend on the token and the frequency slot, not on the layer
      for (int i = wtid; i < p.T * half; i += NWT) {
        const int t = i / half, f = i % half;
        const int ax = min(2, max(0, p.axis[f]));
        float sn, cs;
        sincosf((float)p.positions[(size_t)ax * p.T + t] * p.inv_freq[f], &sn, &cs);
        ws.rope_cos[t][f] = bf16_round(cs);
        ws.rope_sin[t][f] = bf16_round(sn);
      }
      const int n_bt = p.T * p.max_blocks;
      if (wtid == 0) {
        ws.bt_ok = n_bt <= BT_CACHE ? 1 : 0;
        ws.tl = nullptr;
        ws.tl_i = 0;
      }
      if (n_bt <= BT_CACHE)
        for (int i = wtid; i < n_bt; i += NWT) ws.bt[i] = p.block_tables[i];
      named_bar_sync(1, NWT);
    }
    // this CTA's duties: owner of at most one residual tile and one activation tile, at most one attention item
    int my_rtile = -1, my_atile = -1;
    for (int m = 0; m < r_tiles; ++m)
      if (tile_owner(m, r_tiles, G) == cta) my_rtile = m;
    for (int m = 0; m < a_tiles; ++m)
      if (tile_owner(m, a_tiles, G) == cta) my_atile = m;
    const int n_items = p.T * p.Hkv * p.nsplit;
    const bool has_item = cta < n_items;
    const AttnItem item = attn_item_of(p, ws, has_item ? cta : 0);
    if (has_item) {
      // detail: the context length that exceeds the block table's reach
      if (wtid == 0 && (long long)ws.ctx[item.b] > (long long)p.max_blocks * p.page) prism_report(PRISM_ERR_BOUNDS, ws.ctx[item.b]);
      request_first_chunks<D>(p, c, 0, item);  // later layers' first chunks are requested from inside the previous layer's item
    }

    // the embedding rows start the residual and are the first QKV GEMM's input
    if (my_rtile >= 0)
      reduce_tile(p, c, nullptr, 0u, p.layers[0].norm_in, p.xw_in, p.ssq_in, seq_of(c, 0, HO_XW_IN), my_rtile);

#pragma unroll 1
    for (int l = 0; l < p.n_layers; ++l) {
      if (wtid == 0) {
        ws.tl = p.timeline != nullptr ? p.timeline + ((size_t)cta * p.n_layers + l) * TL_STAMPS : nullptr;
        ws.tl_i = 0;
      }
      stamp(c);
      // QKV: activation = residual * input-norm weight; 1/rms for the attention step
      fill_xbuf(p, c, 0, p.xw_in, p.H, seq_of(c, l, HO_XW_IN), p.ssq_in, ws.rstd);
      stamp(c);
      epilogue_gemm(p, c, 0, seq_of(c, l, HO_QKV));
      stamp(c);
      if (has_item) attn_dispatch<D>(p, c, l, item);
      else {
        stamp(c);
        stamp(c);
        stamp(c);
      }
      stamp(c);
      // o_proj: activation = attention output
      fill_xbuf(p, c, 1, p.attn, p.Hq * D, seq_of(c, l, HO_ATTN), nullptr, nullptr);
      stamp(c);
      epilogue_gemm(p, c, 1, seq_of(c, l, HO_OPROJ));
      stamp(c);
      if (my_rtile >= 0)
        reduce_tile(p, c, &p.geo[1], seq_of(c, l, HO_OPROJ), p.layers[l].norm_post, p.xw_post, p.ssq_post, seq_of(c, l, HO_XW_POST),
                    my_rtile);
      stamp(c);
      // gate / up: activation = residual * post-attention-norm weight; 1/rms for the SwiGLU owners
      fill_xbuf(p, c, 2, p.xw_post, p.H, seq_of(c, l, HO_XW_POST), p.ssq_post, ws.rstd_post);
      stamp(c);
      epilogue_gemm(p, c, 2, seq_of(c, l, HO_GATE_UP));
      stamp(c);
      if (my_atile >= 0) swiglu_tile(p, c, seq_of(c, l, HO_GATE_UP), seq_of(c, l, HO_ACT), my_atile);
      stamp(c);
      // down: activation = SwiGLU output
      fill_xbuf(p, c, 3, p.act, p.I, seq_of(c, l, HO_ACT), nullptr, nullptr);
      stamp(c);
      epilogue_gemm(p, c, 3, seq_of(c, l, HO_DOWN));
      stamp(c);
      if (my_rtile >= 0) {
        const bool last = l + 1 == p.n_layers;
        reduce_tile(p, c, &p.geo[3], seq_of(c, l, HO_DOWN), last ? nullptr : p.layers[l + 1].norm_in, p.xw_in, p.ssq_in,
                    seq_of(c, l + 1, HO_XW_IN), my_rtile);
      }
      stamp(c);
    }
    // unwinding after a failed wait: staged chunks still in flight must land before the shared memory is released
    if (wtid == 0) {
      while (c.kv_done < c.kv_req) {
        if (!mbar_wait_short(&kv_full[c.kv_done & (KV_SLOTS - 1)], (uint32_t)(c.kv_done / KV_SLOTS) & 1)) break;
        ++c.kv_done;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- sequence base ---------------------------------------------------------------------------------
// Runs before every launch of the kernel above.  state = {base, generation} may be shared by
// several plans: base += step.  Sequence numbers are 32 bits wide; before they would wrap, the
// base starts over and the generation grows.  A plan whose own generation word differs from the
// state's zeroes its word buffers (one arena) first, so no word of an earlier pass over the number
// space survives.
struct AdvanceArgs {
  u64* state;
  u64* plan_generation;
  u64 step;
  uint4* arena;
  size_t arena_vec;
};
__global__ void advance_seq_kernel(const __grid_constant__ AdvanceArgs a) {
  __shared__ int wrap, stale;
  if (threadIdx.x == 0) {
    wrap = (a.state[0] + 2 * a.step > 0xffffffffull) ? 1 : 0;
    stale = (*a.plan_generation != a.state[1] + (u64)wrap) ? 1 : 0;
  }
  __syncthreads();
  if (stale)
    for (size_t i = threadIdx.x; i < a.arena_vec; i += blockDim.x) a.arena[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (threadIdx.x == 0) {
    a.state[0] = wrap ? a.step : a.state[0] + a.step;
    a.state[1] += (u64)wrap;
    *a.plan_generation = a.state[1];
  }
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

constexpr int TAIL_BYTES = (2 * MAX_STAGES + 2 * NACC + KV_SLOTS) * 8 + 64;
size_t xbuf_bytes(int T, int xslots) { return ((size_t)T * xslots * BK * 2 + 127) & ~(size_t)127; }
int smem_stages(int T, int xslots) {
  const long long room = (long long)SMEM_LIMIT - 1024 - WS_BYTES - (long long)xbuf_bytes(T, xslots) - TAIL_BYTES;
  const int stages = (int)(room / STAGE_BYTES);
  return stages > MAX_STAGES ? MAX_STAGES : stages;
}

}  // namespace

// Bytes of one layer descriptor; the caller owns an array of them in device memory.
PRISM_API int prism_decode_layer_desc_bytes() { return (int)sizeof(LayerDesc); }
PRISM_API int prism_decode_layers_max_tokens() { return TMAX; }
PRISM_API int prism_decode_layers_timeline_stamps() { return TL_STAMPS; }
// Sequence numbers one launch consumes (the step of the sequence base).
PRISM_API int prism_decode_layers_seq_step(int n_layers) { return (n_layers + 1) * SEQ_PER_LAYER; }

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

// Grid size, slab counts and shared-memory plan for a model shape:
// out8 = {grid, P_qkv, P_o, P_gate_up, P_down, xslots, ring stages at 1 token, ring stages at 4 tokens}.
// A negative return: the shape is outside what the kernel handles.
PRISM_API int prism_decode_layers_plan(int H, int m_qkv, int QD, int I, int* out8) {
  if (H % 128 || QD % 64 || I % 128 || H <= 0 || m_qkv <= 0 || QD <= 0 || I <= 0 || H > 8192) return -1;
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
  // every residual tile and every activation tile has its own owner CTA
  if (H / BM > G || I / BM > G) return -3;
  out8[0] = G;
  int xslots = 1;
  for (int g = 0; g < 4; ++g) {
    const int kb = (int)(K[g] / BK), U = (int)((M[g] + BM - 1) / BM) * kb;
    int worst = 1;
    for (int m = 0; m * kb < U; ++m) {
      const int n = sk_owner(m * kb + kb - 1, U, G) - sk_owner(m * kb, U, G) + 1;
      if (n > worst) worst = n;
    }
    out8[1 + g] = worst;
    for (int c = 0; c < G; ++c) {
      int kb0, count;
      gemm_window(U, kb, c, G, kb0, count);
      if (count > xslots) xslots = count;
    }
  }
  out8[5] = xslots;
  out8[6] = smem_stages(1, xslots);
  out8[7] = smem_stages(TMAX, xslots);
  if (out8[7] < 4) return -5;
  return 0;
}

// One decode step through every layer.  `args` is a flat array of 64-bit words (pointers and
// integers; the two floats travel as their bit patterns), indexed by the enum below; see
// ops.decode_layers for the owner of every buffer.  Two launches: the sequence base, the layers.
enum DLArg {
  A_LAYERS, A_N_LAYERS, A_T, A_H, A_HQ, A_HKV, A_D, A_I, A_M_QKV, A_PAGE, A_MAX_BLOCKS, A_NUM_BLOCKS, A_KV_MODE,
  A_NSPLIT, A_EPS_BITS, A_SCALE_BITS, A_STATE, A_PLAN_GENERATION, A_ARENA, A_ARENA_BYTES, A_X0, A_POSITIONS, A_SLOTS, A_BLOCK_TABLES,
  A_CONTEXT_LENS, A_INV_FREQ, A_AXIS, A_OUT, A_XW_IN, A_XW_POST, A_SSQ_IN, A_SSQ_POST, A_ATTN_PART, A_ATTN, A_ACT, A_ABORT,
  A_PART_QKV, A_PART_OPROJ, A_PART_GU, A_PART_DOWN, A_GRID, A_TIMELINE, A_PF_DEPTH, A_COUNT
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
  if (p.T < 1 || p.T > TMAX || p.n_layers < 1 || p.n_layers > 4096) return -2;
  if (D != 64 && D != 128) return -3;
  if (p.Hq <= 0 || p.Hkv <= 0 || p.Hq % p.Hkv) return -4;
  const int GQ = p.Hq / p.Hkv;
  if ((GQ != 1 && GQ != 2 && GQ != 4 && GQ != 8) || GQ * D > 512 || GQ * D < 128) return -5;
  if (m_qkv != (p.Hq + 2 * p.Hkv) * D) return -6;
  if (p.nsplit < 1 || p.nsplit > 32 || p.page < 4 || (p.page & (p.page - 1)) || p.max_blocks <= 0) return -8;
  p.page_shift = 0;
  while ((1 << p.page_shift) < p.page) ++p.page_shift;
  if (p.kv_mode < 0 || p.kv_mode > 2) return -8;
  int plan[8];
  if (prism_decode_layers_plan(p.H, m_qkv, p.Hq * D, p.I, plan) != 0) return -9;
  const int G = (int)args[A_GRID];
  if (G != plan[0]) return -10;  // slab buffers were sized for another grid
  if (p.T * p.Hkv * p.nsplit > G) return -15;  // one attention item per CTA
  p.xslots = plan[5];
  p.stages = smem_stages(p.T, p.xslots);
  if (p.stages < 4) return -16;
  const long long M[4] = {m_qkv, p.H, 2ll * p.I, p.H};
  const long long K[4] = {p.H, (long long)p.Hq * D, p.H, p.I};
  const int part_arg[4] = {A_PART_QKV, A_PART_OPROJ, A_PART_GU, A_PART_DOWN};
  for (int g = 0; g < 4; ++g) {
    p.geo[g].M = (int)M[g];
    p.geo[g].m_tiles = (int)((M[g] + BM - 1) / BM);
    p.geo[g].kb = (int)(K[g] / BK);
    p.geo[g].U = p.geo[g].m_tiles * p.geo[g].kb;
    p.geo[g].slab_stride = (long long)p.T * M[g];
    p.geo[g].part = (u64*)ptr(part_arg[g]);
  }
  p.state = (const u64*)ptr(A_STATE);
  p.x0 = (const bf16*)ptr(A_X0);
  p.positions = (const int*)ptr(A_POSITIONS);
  p.slots = (const long long*)ptr(A_SLOTS);
  p.block_tables = (const int*)ptr(A_BLOCK_TABLES);
  p.context_lens = (const int*)ptr(A_CONTEXT_LENS);
  p.inv_freq = (const float*)ptr(A_INV_FREQ);
  p.axis = (const int*)ptr(A_AXIS);
  p.out = (bf16*)ptr(A_OUT);
  p.xw_in = (u64*)ptr(A_XW_IN);
  p.xw_post = (u64*)ptr(A_XW_POST);
  p.ssq_in = (u64*)ptr(A_SSQ_IN);
  p.ssq_post = (u64*)ptr(A_SSQ_POST);
  p.attn_part = (u64*)ptr(A_ATTN_PART);
  p.attn = (u64*)ptr(A_ATTN);
  p.act = (u64*)ptr(A_ACT);
  p.abort_flag = (int*)ptr(A_ABORT);
  p.timeline = (long long*)ptr(A_TIMELINE);
  p.pf_depth = (int)args[A_PF_DEPTH];
  if (p.pf_depth < 0 || p.pf_depth > 256) return -11;
  if (p.state == nullptr || ptr(A_PLAN_GENERATION) == nullptr || (args[A_ARENA_BYTES] & 15) || (args[A_ARENA] & 15)) return -14;

  const size_t smem = (size_t)p.stages * STAGE_BYTES + WS_BYTES + xbuf_bytes(p.T, p.xslots) + TAIL_BYTES + 1024;
  if (smem > (size_t)SMEM_LIMIT) return -16;
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
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  AdvanceArgs adv;
  memset(&adv, 0, sizeof(adv));
  adv.state = (u64*)ptr(A_STATE);
  adv.plan_generation = (u64*)ptr(A_PLAN_GENERATION);
  adv.step = (u64)prism_decode_layers_seq_step(p.n_layers);
  adv.arena = (uint4*)ptr(A_ARENA);
  adv.arena_vec = (size_t)args[A_ARENA_BYTES] / 16;
  advance_seq_kernel<<<1, 1024, 0, stream>>>(adv);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  // the CTAs wait on one another's words: the launch must be cooperative (the driver refuses a
  // grid that cannot be co-resident instead of letting it deadlock)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, p);
}
