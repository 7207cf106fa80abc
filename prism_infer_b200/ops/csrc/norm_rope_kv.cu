// Pointwise / row-wise kernels around the GEMMs:
//   * residual add + RMSNorm that also folds split-K / tensor-parallel fp32 partial slabs
//     and the DeepStack visual add (reference prism_infer/ops/add_rmsnorm.py:32-230 and
//     prism_infer/models/qwen3_vl.py:1148-1162),
//   * per-head QK-RMSNorm + interleaved M-RoPE + paged KV store with optional scaled-FP8
//     quantisation (reference prism_infer/ops/qk_rmsnorm.py:190-548 and
//     prism_infer/ops/kv_cache_store.py:57-167),
//   * SwiGLU (reference prism_infer/ops/swiglu.py:27-99),
//   * token embedding gather with visual-embedding scatter,
//   * the vision tower's LayerNorm, 2-D rotary and position-embedding interpolation
//     (reference prism_infer/vision/vision_encoder.py:243-262,546-653).
// bf16 rounding points follow the eager bf16 graph: after every add, after norm, after
// the weight multiply, after silu, after each rotary product.
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(norm)

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float b2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2b(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}

// ---------------------------------------------------------------------------------
// add + RMSNorm.  One CTA per token row.
//   delta   = bf16( sum_p partial[p][t][:] )            (P >= 1)   or  x_in[t][:]  (P == 0)
//   added   = residual ? bf16(residual[t] + delta) : delta
//   added   = extra ? bf16(added + extra[extra_index[t]])  (only rows with index >= 0)
//   residual[t] = added (when residual_out != null);  out[t] = bf16(bf16(added * rstd) * w)
// ---------------------------------------------------------------------------------
struct AddNormArgs {
  const float* partials;
  long long slab_stride;
  int P;
  const bf16* x_in;
  const bf16* residual_in;
  bf16* residual_out;
  const bf16* extra;
  const int* extra_index;
  const bf16* weight;
  bf16* out;
  int H;
  float eps;
  // tensor-parallel consumer side of the fused GEMM -> exchange: wait until every source
  // rank's flag reached *epoch + point before reading the partial slabs
  const unsigned long long* wait_flags;  // [n_wait] local flags written by the peers
  int n_wait;
  const unsigned long long* epoch;
  int point;
  int T;
  int packed;  // 1: partials are 8-byte {fp32 value, sequence} words polled until sequence == *epoch + point
};

// Bounded acquire-spin on a flag another GPU writes.  Returns false after
// PRISM_WAIT_CYCLES and records PRISM_ERR_PEER_TIMEOUT: the caller continues with whatever
// data is there, the host sees the status word, nothing hangs.
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long want, int tag) {
  const long long t0 = clock64();
  for (;;) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
    if (v >= want) return true;
    if (clock64() - t0 > PRISM_WAIT_CYCLES) break;
  }
  prism_report(PRISM_ERR_PEER_TIMEOUT, tag);
  return false;
}

__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(const AddNormArgs a) {
  extern __shared__ float row[];  // H floats
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int H = a.H;
  pdl_launch_dependents();
  pdl_wait();
  if (a.n_wait > 0) {
    if ((int)threadIdx.x < a.n_wait) wait_flag_ge(a.wait_flags + threadIdx.x, *a.epoch + (unsigned long long)a.point, threadIdx.x);
    __syncthreads();
  }
  const size_t base = (size_t)t * H;
  int ex = -1;
  if (a.extra != nullptr) ex = a.extra_index[t];
  float ss = 0.0f;
  // Four elements per thread and iteration; all partial-slab loads of an iteration are
  // independent, so a single small-batch row keeps P * 16 bytes per thread in flight.
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float d[4];
    if (a.P > 0 && a.packed) {
      // Packed exchange slabs: sum optimistically with every load in flight, and repeat the
      // pass while any word still carries an older sequence number (bounded).
      const unsigned long long* q0 = reinterpret_cast<const unsigned long long*>(a.partials) + base + i;
      const unsigned int want = (unsigned int)((*a.epoch + (unsigned long long)a.point) & 0xffffffffull);
      const long long t0 = clock64();
      float4 acc;
      for (;;) {
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
        unsigned int stale = 0;
#pragma unroll 8
        for (int p = 0; p < a.P; ++p) {
          unsigned long long w0, w1, w2, w3;
          const unsigned long long* src = q0 + (size_t)p * a.slab_stride;
          asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(src) : "memory");
          asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w2), "=l"(w3) : "l"(src + 2) : "memory");
          stale |= ((unsigned int)(w0 >> 32) ^ want) | ((unsigned int)(w1 >> 32) ^ want) |
                   ((unsigned int)(w2 >> 32) ^ want) | ((unsigned int)(w3 >> 32) ^ want);
          acc.x += __uint_as_float((unsigned int)w0);
          acc.y += __uint_as_float((unsigned int)w1);
          acc.z += __uint_as_float((unsigned int)w2);
          acc.w += __uint_as_float((unsigned int)w3);
        }
        if (stale == 0) break;
        if (clock64() - t0 > PRISM_WAIT_CYCLES) {
          prism_report(PRISM_ERR_PEER_TIMEOUT, (int)threadIdx.x);
          break;
        }
      }
      d[0] = bf16_round(acc.x);
      d[1] = bf16_round(acc.y);
      d[2] = bf16_round(acc.z);
      d[3] = bf16_round(acc.w);
    } else if (a.P > 0) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const float* p0 = a.partials + base + i;
#pragma unroll 8
      for (int p = 0; p < a.P; ++p) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(p0 + (size_t)p * a.slab_stride));
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      d[0] = bf16_round(acc.x);
      d[1] = bf16_round(acc.y);
      d[2] = bf16_round(acc.z);
      d[3] = bf16_round(acc.w);
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(a.x_in + base + i);
      const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
      d[0] = b2f(v[0].x);
      d[1] = b2f(v[0].y);
      d[2] = b2f(v[1].x);
      d[3] = b2f(v[1].y);
    }
    if (a.residual_in != nullptr) {
      const uint2 raw = *reinterpret_cast<const uint2*>(a.residual_in + base + i);
      const __nv_bfloat162* r = reinterpret_cast<const __nv_bfloat162*>(&raw);
      d[0] = bf16_round(b2f(r[0].x) + d[0]);
      d[1] = bf16_round(b2f(r[0].y) + d[1]);
      d[2] = bf16_round(b2f(r[1].x) + d[2]);
      d[3] = bf16_round(b2f(r[1].y) + d[3]);
    }
    if (ex >= 0) {
      const uint2 raw = *reinterpret_cast<const uint2*>(a.extra + (size_t)ex * H + i);
      const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
      d[0] = bf16_round(d[0] + b2f(e[0].x));
      d[1] = bf16_round(d[1] + b2f(e[0].y));
      d[2] = bf16_round(d[2] + b2f(e[1].x));
      d[3] = bf16_round(d[3] + b2f(e[1].y));
    }
    if (a.residual_out != nullptr) {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(d[0], d[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(d[2], d[3]);
      *reinterpret_cast<uint2*>(a.residual_out + base + i) = o;
    }
    *reinterpret_cast<float4*>(row + i) = make_float4(d[0], d[1], d[2], d[3]);
    ss += d[0] * d[0] + d[1] * d[1] + d[2] * d[2] + d[3] * d[3];
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)H + a.eps);
  if (a.out != nullptr) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      const uint2 raw = *reinterpret_cast<const uint2*>(a.weight + i);
      const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float4 r = *reinterpret_cast<const float4*>(row + i);
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) =
          __floats2bfloat162_rn(bf16_round(r.x * rstd) * b2f(w[0].x), bf16_round(r.y * rstd) * b2f(w[0].y));
      *reinterpret_cast<__nv_bfloat162*>(&o.y) =
          __floats2bfloat162_rn(bf16_round(r.z * rstd) * b2f(w[1].x), bf16_round(r.w * rstd) * b2f(w[1].y));
      *reinterpret_cast<uint2*>(a.out + base + i) = o;
    }
  }
}

// ---------------------------------------------------------------------------------
// Prefill form of add+RMSNorm (bf16 delta rows, hidden size at most 8192): one warp per row,
// the pre-norm row lives in registers as 16-byte vectors, no shared memory or block barrier.
// Same rounding points as add_rmsnorm_kernel.
// ---------------------------------------------------------------------------------
constexpr int RN_VEC = 32;  // vectors of 8 bf16 per lane (8192 / 32 / 8)
template <int NV>
__global__ void __launch_bounds__(256) add_rmsnorm_rows_kernel(const AddNormArgs a) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (t >= a.T) return;
  const int H = a.H, nvec = H >> 3;
  const size_t base = (size_t)t * H;
  const int ex = a.extra != nullptr ? a.extra_index[t] : -1;
  uint4 v[NV];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = lane + 32 * k;
    if (i < nvec) {
      uint4 x = reinterpret_cast<const uint4*>(a.x_in + base)[i];
      __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&x);
      float2 d[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) d[e] = __bfloat1622float2(xp[e]);
      if (a.residual_in != nullptr) {
        const uint4 r = reinterpret_cast<const uint4*>(a.residual_in + base)[i];
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(rp[e]);
          d[e].x = bf16_round(f.x + d[e].x);
          d[e].y = bf16_round(f.y + d[e].y);
        }
      }
      if (ex >= 0) {
        const uint4 r = reinterpret_cast<const uint4*>(a.extra + (size_t)ex * H)[i];
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(rp[e]);
          d[e].x = bf16_round(d[e].x + f.x);
          d[e].y = bf16_round(d[e].y + f.y);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ss += d[e].x * d[e].x + d[e].y * d[e].y;
        xp[e] = __floats2bfloat162_rn(d[e].x, d[e].y);  // exact: the sums are already bf16 values
      }
      v[k] = x;
      if (a.residual_out != nullptr) reinterpret_cast<uint4*>(a.residual_out + base)[i] = x;
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)H + a.eps);
  if (a.out == nullptr) return;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = lane + 32 * k;
    if (i < nvec) {
      const uint4 w = reinterpret_cast<const uint4*>(a.weight)[i];
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(xp[e]), wf = __bfloat1622float2(wp[e]);
        op[e] = __floats2bfloat162_rn(bf16_round(f.x * rstd) * wf.x, bf16_round(f.y * rstd) * wf.y);
      }
      reinterpret_cast<uint4*>(a.out + base)[i] = o;
    }
  }
}

// ---------------------------------------------------------------------------------
// Consumer of prism_gemm_wx_scatter (tensor-parallel prefill): this rank owns `rows` token
// rows.  For each of them (one CTA per row): wait for every rank's partial (bounded), sum the
// tp bf16 partial rows in rank order, add the residual shard (and a DeepStack row), write the
// new residual shard, RMSNorm, and store the normalised row into EVERY rank's activation
// buffer at its global row index (the all-gather).  The last CTA then raises flag[my_rank]
// on every rank.  Residuals stay sharded by token row between layers.
// ---------------------------------------------------------------------------------
struct RnaArgs {
  const bf16* rs;                       // local [tp][rows_per_owner][H]
  const unsigned long long* rs_flags;   // local [tp]
  unsigned long long rs_seq;
  int tp, my_rank, rows_per_owner, rows, row0, H;
  const bf16* residual_in;              // first owned row, row stride ld_res (may be null)
  long long ld_res;
  bf16* residual_out;                   // [rows][H]
  const bf16* extra;                    // DeepStack rows (may be null)
  const int* extra_index;               // [T] global row -> row of extra, or < 0
  const bf16* weight;
  float eps;
  bf16* peer_x[8];                      // [T][H] on every rank
  unsigned long long* peer_flag[8];     // [tp] on every rank
  unsigned long long ag_seq;
  const unsigned long long* epoch;      // when set, both sequence numbers are offsets from *epoch
  int* cta_counter;
};

// Split-K partial rows of a row-parallel projection -> the ranks that own the rows.  One CTA per
// token row: sum the P local fp32 slabs, round to bf16 and store the row into slab [my_rank] of
// its owner (rows_per_owner consecutive rows per rank); the last CTA raises flag[my_rank] on
// every rank.  Together with reduce_norm_allgather_kernel this is an all-reduce in which every
// rank sends T rows of bf16 once (the one-shot exchange of 8-byte words sends tp x splits x T).
struct ScatterRowsArgs {
  const float* partials;   // [P][T][H]
  long long slab_stride;
  int P, T, H, rows_per_owner, tp, my_rank;
  bf16* peer_rs[8];                   // [tp][rows_per_owner][H] on every rank
  unsigned long long* peer_flag[8];   // [tp] on every rank
  const unsigned long long* epoch;
  unsigned long long seq;
  int* cta_counter;
};
__global__ void __launch_bounds__(128) scatter_rows_kernel(const ScatterRowsArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int owner = t / a.rows_per_owner, local = t - owner * a.rows_per_owner;
  bf16* dst = a.peer_rs[owner] + ((size_t)a.my_rank * a.rows_per_owner + local) * a.H;
  const float* src = a.partials + (size_t)t * a.H;
  for (int c = threadIdx.x * 8; c < a.H; c += 128 * 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
    for (int p = 0; p < a.P; ++p) {
      const float4 lo = __ldcg(reinterpret_cast<const float4*>(src + (size_t)p * a.slab_stride + c));
      const float4 hi = __ldcg(reinterpret_cast<const float4*>(src + (size_t)p * a.slab_stride + c + 4));
      acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
      acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
    }
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) op[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(dst + c) = o;
  }
  __threadfence_system();  // the row is visible on its owner before the flag can be
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(a.cta_counter, 1);
    if (old == (int)gridDim.x - 1) {
      *a.cta_counter = 0;
      __threadfence_system();
      const unsigned long long seq = (a.epoch ? *a.epoch : 0ull) + a.seq;
      for (int p = 0; p < a.tp; ++p)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.peer_flag[p] + a.my_rank), "l"(seq) : "memory");
    }
  }
}

// One CTA of 128 threads per owned row (a rank owns only T / tp rows, so a warp per row would
// leave most SMs idle); NV 16-byte vectors per thread.
template <int NV>
__global__ void __launch_bounds__(128) reduce_norm_allgather_kernel(const RnaArgs a) {
  __shared__ float red[4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int H = a.H, nvec = H >> 3;
  const unsigned long long base = a.epoch ? *a.epoch : 0ull;
  if (i < a.rows) {
    if ((int)threadIdx.x < a.tp) wait_flag_ge(a.rs_flags + threadIdx.x, base + a.rs_seq, threadIdx.x);
    __syncthreads();
    const int g_row = a.row0 + i;
    const int ex = a.extra != nullptr ? a.extra_index[g_row] : -1;
    uint4 v[NV];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = threadIdx.x + 128 * k;
      if (c < nvec) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll 8
        for (int r = 0; r < a.tp; ++r) {
          const uint4 p = __ldcg(reinterpret_cast<const uint4*>(a.rs + ((size_t)r * a.rows_per_owner + i) * H) + c);
          const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&p);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(pp[e]);
            acc[2 * e] += f.x;
            acc[2 * e + 1] += f.y;
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = bf16_round(acc[e]);
        if (a.residual_in != nullptr) {
          const uint4 rv = reinterpret_cast<const uint4*>(a.residual_in + (size_t)i * a.ld_res)[c];
          const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(rp[e]);
            acc[2 * e] = bf16_round(f.x + acc[2 * e]);
            acc[2 * e + 1] = bf16_round(f.y + acc[2 * e + 1]);
          }
        }
        if (ex >= 0) {
          const uint4 rv = reinterpret_cast<const uint4*>(a.extra + (size_t)ex * H)[c];
          const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(rp[e]);
            acc[2 * e] = bf16_round(acc[2 * e] + f.x);
            acc[2 * e + 1] = bf16_round(acc[2 * e + 1] + f.y);
          }
        }
        uint4 x;
        __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          ss += acc[2 * e] * acc[2 * e] + acc[2 * e + 1] * acc[2 * e + 1];
          xp[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        }
        v[k] = x;
        reinterpret_cast<uint4*>(a.residual_out + (size_t)i * H)[c] = x;
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    const float rstd = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)H + a.eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = threadIdx.x + 128 * k;
      if (c < nvec) {
        const uint4 w = reinterpret_cast<const uint4*>(a.weight)[c];
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(xp[e]), wf = __bfloat1622float2(wp[e]);
          op[e] = __floats2bfloat162_rn(bf16_round(f.x * rstd) * wf.x, bf16_round(f.y * rstd) * wf.y);
        }
        for (int p = 0; p < a.tp; ++p) reinterpret_cast<uint4*>(a.peer_x[p] + (size_t)g_row * H)[c] = o;
      }
    }
    __threadfence_system();  // this row is visible on every rank before the flag can be
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(a.cta_counter, 1);
    if (old == (int)gridDim.x - 1) {
      *a.cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < a.tp; ++p)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.peer_flag[p] + a.my_rank), "l"(base + a.ag_seq) : "memory");
    }
  }
}

// ---------------------------------------------------------------------------------
// LayerNorm with bias (vision tower), one CTA per row, fp32 statistics.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) layernorm_kernel(const bf16* x, const bf16* w, const bf16* b, bf16* out, int H,
                                                        float eps) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * H;
  pdl_launch_dependents();
  pdl_wait();
  float s = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = b2f(x[base + i]);
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / (float)H;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row[i] - mean;
    ss += d * d;
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    out[base + i] = f2b((row[i] - mean) * rstd * b2f(w[i]) + b2f(b[i]));
  }
}

// Rows of at most 2048 elements (the vision tower: 1152 and 4608): one warp per row, the row
// lives in registers as 16-byte vectors, statistics with shuffles only.
constexpr int LN_VEC = 8;  // vectors of 8 bf16 per lane
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const bf16* x, const bf16* w, const bf16* b, bf16* out, int T,
                                                             int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (row >= T) return;
  const int nvec = H >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * H);
  uint4 v[LN_VEC];
  float s = 0.0f;
#pragma unroll
  for (int k = 0; k < LN_VEC; ++k) {
    const int i = lane + 32 * k;
    v[k] = i < nvec ? src[i] : make_uint4(0, 0, 0, 0);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(p[e]);
      s += f.x + f.y;
    }
  }
  const float mean = warp_sum(s) / (float)H;
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < LN_VEC; ++k) {
    if (lane + 32 * k < nvec) {
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        ss += (f.x - mean) * (f.x - mean) + (f.y - mean) * (f.y - mean);
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)H + eps);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * H);
#pragma unroll
  for (int k = 0; k < LN_VEC; ++k) {
    const int i = lane + 32 * k;
    if (i < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[i], bv = reinterpret_cast<const uint4*>(b)[i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
      const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bv);
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]), wf = __bfloat1622float2(wp[e]), bf = __bfloat1622float2(bp[e]);
        op[e] = __floats2bfloat162_rn((f.x - mean) * rstd * wf.x + bf.x, (f.y - mean) * rstd * wf.y + bf.y);
      }
      dst[i] = o;
    }
  }
}

// ---------------------------------------------------------------------------------
// QK-RMSNorm + M-RoPE + KV store.  One warp per (token, head); heads are ordered
// [q heads | k heads | v heads] exactly like the packed QKV projection row.
// ---------------------------------------------------------------------------------
struct QkvArgs {
  const bf16* qkv;          // [T][row_stride] bf16, or null when partials are given
  const float* partials;    // [P][T][row_stride] fp32 split-K slabs
  long long slab_stride;
  int P;
  long long row_stride;     // elements per token in the source
  const int* positions;     // [3][T] (T, H, W axes)
  const bf16* q_weight;     // [D]
  const bf16* k_weight;     // [D]
  const float* inv_freq;    // [D/2]
  const int* axis;          // [D/2] in {0,1,2}
  bf16* q_out;              // [T][Hq][D] (may be null)
  long long q_stride;       // elements per token in q_out
  const long long* slots;   // [T] flat slot (block * page + offset), < 0 = skip
  void* k_cache;            // [blocks][Hkv][page][D]
  void* v_cache;
  float* k_scale;           // [blocks][Hkv][page]
  float* v_scale;
  int T, Hq, Hkv, page;
  int kv_mode;              // 0 bf16, 1 fp8 unit scale, 2 fp8 + per-token-per-head scale
  int apply_norm, apply_rope;
  float eps;
  int k_writeback;          // 1: the normalised, rotated K also replaces its source in qkv (bf16 source only)
};

constexpr float FP8_MAX = 448.0f;
constexpr float FP8_SCALE_FLOOR = 1.0e-6f;

template <int D>
__global__ void __launch_bounds__(256) qk_norm_rope_store_kernel(const QkvArgs a) {
  constexpr int PER = D / 64;  // rotary pairs per lane
  const int warps_per_block = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = a.Hq + 2 * a.Hkv;
  pdl_launch_dependents();
  pdl_wait();
  if (gw >= a.T * heads) return;
  const int t = gw / heads;
  const int h = gw % heads;
  const bool is_q = h < a.Hq;
  const bool is_k = !is_q && h < a.Hq + a.Hkv;
  const size_t src = (size_t)t * a.row_stride + (size_t)h * D;

  float lo[PER], hi[PER];  // element i and element i + D/2
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    if (a.P > 0) {
      float s0 = 0.0f, s1 = 0.0f;
      for (int p = 0; p < a.P; ++p) {
        const float* row = a.partials + (size_t)p * a.slab_stride + src;
        s0 += row[i];
        s1 += row[i + D / 2];
      }
      lo[j] = bf16_round(s0);
      hi[j] = bf16_round(s1);
    } else {
      lo[j] = b2f(a.qkv[src + i]);
      hi[j] = b2f(a.qkv[src + i + D / 2]);
    }
  }
  if (is_q || is_k) {
    if (a.apply_norm) {
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < PER; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / (float)D + a.eps);
      const bf16* w = is_q ? a.q_weight : a.k_weight;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + 32 * j;
        lo[j] = bf16_round(bf16_round(lo[j] * rstd) * b2f(w[i]));
        hi[j] = bf16_round(bf16_round(hi[j] * rstd) * b2f(w[i + D / 2]));
      }
    }
    if (a.apply_rope) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + 32 * j;
        const int ax = a.axis[i];
        const float pos = (float)a.positions[(size_t)ax * a.T + t];
        float sn, cs;
        sincosf(pos * a.inv_freq[i], &sn, &cs);
        sn = bf16_round(sn);
        cs = bf16_round(cs);
        const float x0 = lo[j], x1 = hi[j];
        lo[j] = bf16_round(bf16_round(x0 * cs) + bf16_round(-x1 * sn));
        hi[j] = bf16_round(bf16_round(x1 * cs) + bf16_round(x0 * sn));
      }
    }
  }
  if (is_q) {
    if (a.q_out != nullptr) {
      bf16* dst = a.q_out + (size_t)t * a.q_stride + (size_t)h * D;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        dst[lane + 32 * j] = f2b(lo[j]);
        dst[lane + 32 * j + D / 2] = f2b(hi[j]);
      }
    }
    return;
  }
  if (is_k && a.k_writeback && a.qkv != nullptr) {
    // prefill without history attends over these bf16 rows directly instead of the paged copy
    bf16* dst = const_cast<bf16*>(a.qkv) + src;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      dst[lane + 32 * j] = f2b(lo[j]);
      dst[lane + 32 * j + D / 2] = f2b(hi[j]);
    }
  }
  const long long slot = a.slots[t];
  if (slot < 0) return;
  const int kvh = is_k ? h - a.Hq : h - a.Hq - a.Hkv;
  const long long blk = slot / a.page;
  const int off = (int)(slot % a.page);
  const size_t row = ((size_t)blk * a.Hkv + kvh) * a.page + off;  // token row inside [blocks][Hkv][page]
  void* cache = is_k ? a.k_cache : a.v_cache;
  if (a.kv_mode == 0) {
    bf16* dst = reinterpret_cast<bf16*>(cache) + row * D;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      dst[lane + 32 * j] = f2b(lo[j]);
      dst[lane + 32 * j + D / 2] = f2b(hi[j]);
    }
  } else {
    float scale = 1.0f;
    if (a.kv_mode == 2) {
      float am = 0.0f;
#pragma unroll
      for (int j = 0; j < PER; ++j) am = fmaxf(am, fmaxf(fabsf(lo[j]), fabsf(hi[j])));
      am = warp_max(am);
      scale = fmaxf(am / FP8_MAX, FP8_SCALE_FLOOR);
      if (lane == 0) (is_k ? a.k_scale : a.v_scale)[row] = scale;
    }
    __nv_fp8_storage_t* dst = reinterpret_cast<__nv_fp8_storage_t*>(cache) + row * D;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const float q0 = fminf(fmaxf(lo[j] / scale, -FP8_MAX), FP8_MAX);
      const float q1 = fminf(fmaxf(hi[j] / scale, -FP8_MAX), FP8_MAX);
      dst[lane + 32 * j] = __nv_cvt_float_to_fp8(q0, __NV_SATFINITE, __NV_E4M3);
      dst[lane + 32 * j + D / 2] = __nv_cvt_float_to_fp8(q1, __NV_SATFINITE, __NV_E4M3);
    }
  }
}

// ---------------------------------------------------------------------------------
// Prefill form of the kernel above (bf16 source rows, head dimension 128): one CTA per token.
// The 64 rotary angles of the token are evaluated once into shared memory instead of once
// per head, and every lane moves adjacent element pairs (4-byte accesses).  Same rounding
// points as the per-head kernel.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) qk_norm_rope_store_token_kernel(const QkvArgs a) {
  constexpr int D = 128, HALF = 64;
  __shared__ float cs_s[HALF], sn_s[HALF];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.Hq + 2 * a.Hkv;
  pdl_launch_dependents();
  pdl_wait();
  if ((int)threadIdx.x < HALF && a.apply_rope) {
    const int i = threadIdx.x;
    const float pos = (float)a.positions[(size_t)a.axis[i] * a.T + t];
    float sn, cs;
    sincosf(pos * a.inv_freq[i], &sn, &cs);
    sn_s[i] = bf16_round(sn);
    cs_s[i] = bf16_round(cs);
  }
  __syncthreads();
  const long long slot = a.slots[t];
  const int i0 = 2 * lane;  // this lane's elements: i0, i0 + 1 and i0 + 64, i0 + 65
  for (int h = warp; h < heads; h += 8) {
    const bool is_q = h < a.Hq;
    const bool is_k = !is_q && h < a.Hq + a.Hkv;
    bf16* src = const_cast<bf16*>(a.qkv) + (size_t)t * a.row_stride + (size_t)h * D;
    const float2 lo2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i0));
    const float2 hi2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i0 + HALF));
    float lo[2] = {lo2.x, lo2.y}, hi[2] = {hi2.x, hi2.y};
    if (is_q || is_k) {
      if (a.apply_norm) {
        float ss = lo[0] * lo[0] + lo[1] * lo[1] + hi[0] * hi[0] + hi[1] * hi[1];
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / (float)D + a.eps);
        const bf16* w = is_q ? a.q_weight : a.k_weight;
        const float2 wl = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + i0));
        const float2 wh = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + i0 + HALF));
        lo[0] = bf16_round(bf16_round(lo[0] * rstd) * wl.x);
        lo[1] = bf16_round(bf16_round(lo[1] * rstd) * wl.y);
        hi[0] = bf16_round(bf16_round(hi[0] * rstd) * wh.x);
        hi[1] = bf16_round(bf16_round(hi[1] * rstd) * wh.y);
      }
      if (a.apply_rope) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float cs = cs_s[i0 + e], sn = sn_s[i0 + e];
          const float x0 = lo[e], x1 = hi[e];
          lo[e] = bf16_round(bf16_round(x0 * cs) + bf16_round(-x1 * sn));
          hi[e] = bf16_round(bf16_round(x1 * cs) + bf16_round(x0 * sn));
        }
      }
    }
    const __nv_bfloat162 lo_b = __floats2bfloat162_rn(lo[0], lo[1]), hi_b = __floats2bfloat162_rn(hi[0], hi[1]);
    if (is_q) {
      if (a.q_out != nullptr) {
        bf16* dst = a.q_out + (size_t)t * a.q_stride + (size_t)h * D;
        *reinterpret_cast<__nv_bfloat162*>(dst + i0) = lo_b;
        *reinterpret_cast<__nv_bfloat162*>(dst + i0 + HALF) = hi_b;
      }
      continue;
    }
    if (is_k && a.k_writeback) {
      *reinterpret_cast<__nv_bfloat162*>(src + i0) = lo_b;
      *reinterpret_cast<__nv_bfloat162*>(src + i0 + HALF) = hi_b;
    }
    if (slot < 0) continue;
    const int kvh = is_k ? h - a.Hq : h - a.Hq - a.Hkv;
    const long long blk = slot / a.page;
    const int off = (int)(slot % a.page);
    const size_t row = ((size_t)blk * a.Hkv + kvh) * a.page + off;
    void* cache = is_k ? a.k_cache : a.v_cache;
    if (a.kv_mode == 0) {
      bf16* dst = reinterpret_cast<bf16*>(cache) + row * D;
      *reinterpret_cast<__nv_bfloat162*>(dst + i0) = lo_b;
      *reinterpret_cast<__nv_bfloat162*>(dst + i0 + HALF) = hi_b;
    } else {
      float scale = 1.0f;
      if (a.kv_mode == 2) {
        float am = fmaxf(fmaxf(fabsf(lo[0]), fabsf(lo[1])), fmaxf(fabsf(hi[0]), fabsf(hi[1])));
        am = warp_max(am);
        scale = fmaxf(am / FP8_MAX, FP8_SCALE_FLOOR);
        if (lane == 0) (is_k ? a.k_scale : a.v_scale)[row] = scale;
      }
      __nv_fp8_storage_t* dst = reinterpret_cast<__nv_fp8_storage_t*>(cache) + row * D;
      unsigned short lo8 = 0, hi8 = 0;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float q0 = fminf(fmaxf(lo[e] / scale, -FP8_MAX), FP8_MAX);
        const float q1 = fminf(fmaxf(hi[e] / scale, -FP8_MAX), FP8_MAX);
        lo8 |= (unsigned short)__nv_cvt_float_to_fp8(q0, __NV_SATFINITE, __NV_E4M3) << (8 * e);
        hi8 |= (unsigned short)__nv_cvt_float_to_fp8(q1, __NV_SATFINITE, __NV_E4M3) << (8 * e);
      }
      *reinterpret_cast<unsigned short*>(dst + i0) = lo8;
      *reinterpret_cast<unsigned short*>(dst + i0 + HALF) = hi8;
    }
  }
}

// ---------------------------------------------------------------------------------
// SwiGLU on a packed [T][2I] row (gate | up), bf16 source or fp32 split-K slabs.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_kernel(const bf16* gu, const float* partials, long long slab_stride, int P,
                                                     bf16* out, int T, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)T * I;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I, i = idx % I;
    float g, u;
    if (P > 0) {
      float sg = 0.0f, su = 0.0f;
      for (int p = 0; p < P; ++p) {
        const float* row = partials + (size_t)p * slab_stride + t * 2 * I;
        sg += row[i];
        su += row[I + i];
      }
      g = bf16_round(sg);
      u = bf16_round(su);
    } else {
      g = b2f(gu[t * 2 * I + i]);
      u = b2f(gu[t * 2 * I + I + i]);
    }
    out[idx] = f2b(bf16_round(silu(g)) * u);
  }
}

// ---------------------------------------------------------------------------------
// Token embedding gather with vocabulary shard window and visual-embedding scatter.
// vis_index[t] >= 0 selects row vis_index[t] of `visual` instead of the table.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_kernel(const long long* ids, const bf16* table, const bf16* visual,
                                                    const int* vis_index, bf16* out, int H, long long vocab_start,
                                                    long long vocab_end) {
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const long long id = ids[t];
  const int vi = (visual != nullptr && vis_index != nullptr) ? vis_index[t] : -1;
  const bf16* src = nullptr;
  if (vi >= 0) src = visual + (size_t)vi * H;
  else if (id >= vocab_start && id < vocab_end) src = table + (size_t)(id - vocab_start) * H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (src != nullptr) v = *reinterpret_cast<const uint4*>(src + i);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + i) = v;
  }
}

// hidden[t] += extra[index[t]] for rows with index >= 0 (DeepStack on an explicit tensor).
__global__ void __launch_bounds__(256) indexed_add_kernel(bf16* hidden, const bf16* extra, const int* index, int H) {
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int e = index[t];
  if (e < 0) return;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    hidden[(size_t)t * H + i] = f2b(b2f(hidden[(size_t)t * H + i]) + b2f(extra[(size_t)e * H + i]));
  }
}

// ---------------------------------------------------------------------------------
// Vision: x[n] += bf16( sum_k w[k][n] * table[idx[k][n]] )   (4-corner bilinear plan)
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pos_embed_add_kernel(bf16* x, const bf16* table, const long long* idx,
                                                            const float* wt, int N, int H) {
  const int n = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  long long id[4];
  float w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    id[k] = idx[(size_t)k * N + n];
    w[k] = wt[(size_t)k * N + n];
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) s += w[k] * b2f(table[(size_t)id[k] * H + i]);
    x[(size_t)n * H + i] = f2b(b2f(x[(size_t)n * H + i]) + bf16_round(s));
  }
}

// Vision 2-D rotary on q and k inside the packed [N][3][heads][hd] projection, in place.
// angle[n][i] for i < hd/2: first hd/4 slots use the row coordinate, next hd/4 the column.
__global__ void __launch_bounds__(256) vit_rope_kernel(bf16* qkv, const int* coords, const float* inv_freq, int N,
                                                       int heads, int hd) {
  // The angle depends on (patch, i) only: 36 sin/cos pairs per patch are computed once into
  // shared memory, then every (q|k, head) row is rotated with 4-byte accesses.
  __shared__ float sn_s[128], cs_s[128];
  const int n = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int half = hd / 2, quarter = hd / 4;
  if ((int)threadIdx.x < half) {
    const int i = threadIdx.x;
    const float pos = (float)coords[2 * n + (i < quarter ? 0 : 1)];
    sincosf(pos * inv_freq[i % quarter], &sn_s[i], &cs_s[i]);
  }
  __syncthreads();
  const int pairs = half / 2;  // two adjacent i per thread and step
  const int work = 2 * heads * pairs;
  for (int w = threadIdx.x; w < work; w += blockDim.x) {
    const int i = (w % pairs) * 2;
    const int h = (w / pairs) % heads;
    const int which = w / (pairs * heads);  // 0 = q, 1 = k
    bf16* p = qkv + ((size_t)n * 3 + which) * heads * hd + (size_t)h * hd;
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + i));
    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + i + half));
    const float c0 = cs_s[i], c1 = cs_s[i + 1], s0 = sn_s[i], s1 = sn_s[i + 1];
    *reinterpret_cast<__nv_bfloat162*>(p + i) = __floats2bfloat162_rn(x0.x * c0 - x1.x * s0, x0.y * c1 - x1.y * s1);
    *reinterpret_cast<__nv_bfloat162*>(p + i + half) = __floats2bfloat162_rn(x1.x * c0 + x0.x * s0, x1.y * c1 + x0.y * s1);
  }
}

}  // namespace

#define STREAM(p) reinterpret_cast<cudaStream_t>(p)

static int add_rmsnorm_impl(const void* partials, long long slab_stride, int P, const void* x_in,
                            const void* residual_in, void* residual_out, const void* extra, const void* extra_index,
                            const void* weight, void* out, int T, int H, float eps, void* stream, int pdl,
                            const void* wait_flags, int n_wait, const void* epoch, int point, int packed = 0) {
  if (T <= 0) return 0;
  if (H % 4) return -1;
  if (packed && (epoch == nullptr || P <= 0)) return -3;
  AddNormArgs a;
  a.packed = packed;
  a.partials = (const float*)partials;
  a.slab_stride = slab_stride;
  a.P = P;
  a.x_in = (const bf16*)x_in;
  a.residual_in = (const bf16*)residual_in;
  a.residual_out = (bf16*)residual_out;
  a.extra = (const bf16*)extra;
  a.extra_index = (const int*)extra_index;
  a.weight = (const bf16*)weight;
  a.out = (bf16*)out;
  a.H = H;
  a.eps = eps;
  a.wait_flags = (const unsigned long long*)wait_flags;
  a.n_wait = n_wait;
  a.epoch = (const unsigned long long*)epoch;
  a.point = point;
  a.T = T;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  {
    const unsigned long long addr = reinterpret_cast<unsigned long long>(x_in) | reinterpret_cast<unsigned long long>(residual_in) |
                                    reinterpret_cast<unsigned long long>(residual_out) | reinterpret_cast<unsigned long long>(extra) |
                                    reinterpret_cast<unsigned long long>(weight) | reinterpret_cast<unsigned long long>(out);
    if (T >= 64 && P == 0 && x_in != nullptr && n_wait == 0 && H % 8 == 0 && H <= 8192 && (addr & 15ull) == 0) {
      dim3 grid((T + 7) / 8), block(256);
      if (H <= 2048) return (int)prism_launch(add_rmsnorm_rows_kernel<8>, grid, block, 0, STREAM(stream), pdl != 0, a);
      if (H <= 4096) return (int)prism_launch(add_rmsnorm_rows_kernel<16>, grid, block, 0, STREAM(stream), pdl != 0, a);
      return (int)prism_launch(add_rmsnorm_rows_kernel<RN_VEC>, grid, block, 0, STREAM(stream), pdl != 0, a);
    }
  }
  // few rows: one wide CTA per row so every element has its own thread; many rows: 256 threads
  int threads = T <= 64 ? 1024 : 256;
  while (threads > 32 && threads * 4 > H * 2) threads >>= 1;
  return (int)prism_launch(add_rmsnorm_kernel, dim3(T), dim3(threads), smem, STREAM(stream), pdl != 0, a);
}

PRISM_API int prism_add_rmsnorm(const void* partials, long long slab_stride, int P, const void* x_in,
                                const void* residual_in, void* residual_out, const void* extra, const void* extra_index,
                                const void* weight, void* out, int T, int H, float eps, void* stream, int pdl) {
  return add_rmsnorm_impl(partials, slab_stride, P, x_in, residual_in, residual_out, extra, extra_index, weight, out, T, H,
                          eps, stream, pdl, nullptr, 0, nullptr, 0);
}

// Same, but first waits (bounded) until wait_flags[0..n_wait) >= *epoch + point: the
// consumer of prism_gemm_wx_push.  partials must be the local slab buffer of that slot.
PRISM_API int prism_add_rmsnorm_wait(const void* partials, long long slab_stride, int P, const void* residual_in,
                                     void* residual_out, const void* extra, const void* extra_index, const void* weight,
                                     void* out, int T, int H, float eps, const void* wait_flags, int n_wait,
                                     const void* epoch, int point, void* stream, int pdl) {
  return add_rmsnorm_impl(partials, slab_stride, P, nullptr, residual_in, residual_out, extra, extra_index, weight, out, T,
                          H, eps, stream, pdl, wait_flags, n_wait, epoch, point);
}

// Consumer of prism_gemm_wx_push: partials are 8-byte {fp32 value, sequence} words (strides in
// 8-byte elements) that are polled (bounded) until every sequence equals the low 32 bits of
// *epoch + point, then summed in slab order.
PRISM_API int prism_add_rmsnorm_packed(const void* partials, long long slab_stride, int P, const void* residual_in,
                                       void* residual_out, const void* extra, const void* extra_index,
                                       const void* weight, void* out, int T, int H, float eps, const void* epoch,
                                       int point, void* stream, int pdl) {
  return add_rmsnorm_impl(partials, slab_stride, P, nullptr, residual_in, residual_out, extra, extra_index, weight, out, T,
                          H, eps, stream, pdl, nullptr, 0, epoch, point, 1);
}

PRISM_API int prism_reduce_norm_allgather(const void* rs, const void* rs_flags, long long rs_seq, int tp, int my_rank,
                                          int rows_per_owner, int rows, int row0, int H, const void* residual_in,
                                          long long ld_res, void* residual_out, const void* extra, const void* extra_index,
                                          const void* weight, float eps, const void* const* peer_x,
                                          const void* const* peer_flag, long long ag_seq, const void* epoch,
                                          void* cta_counter, void* stream, int pdl) {
  if (tp < 1 || tp > 8 || rows < 0 || rows > rows_per_owner) return -20;
  if (H % 8 || H > 8192) return -21;
  RnaArgs a;
  a.rs = (const bf16*)rs;
  a.rs_flags = (const unsigned long long*)rs_flags;
  a.rs_seq = (unsigned long long)rs_seq;
  a.tp = tp;
  a.my_rank = my_rank;
  a.rows_per_owner = rows_per_owner;
  a.rows = rows;
  a.row0 = row0;
  a.H = H;
  a.residual_in = (const bf16*)residual_in;
  a.ld_res = ld_res;
  a.residual_out = (bf16*)residual_out;
  a.extra = (const bf16*)extra;
  a.extra_index = (const int*)extra_index;
  a.weight = (const bf16*)weight;
  a.eps = eps;
  for (int p = 0; p < 8; ++p) {
    a.peer_x[p] = p < tp ? (bf16*)const_cast<void*>(peer_x[p]) : nullptr;
    a.peer_flag[p] = p < tp ? (unsigned long long*)const_cast<void*>(peer_flag[p]) : nullptr;
  }
  a.ag_seq = (unsigned long long)ag_seq;
  a.epoch = (const unsigned long long*)epoch;
  a.cta_counter = (int*)cta_counter;
  dim3 grid(rows > 0 ? rows : 1), block(128);
  if (H <= 2048) return (int)prism_launch(reduce_norm_allgather_kernel<2>, grid, block, 0, STREAM(stream), pdl != 0, a);
  if (H <= 4096) return (int)prism_launch(reduce_norm_allgather_kernel<4>, grid, block, 0, STREAM(stream), pdl != 0, a);
  return (int)prism_launch(reduce_norm_allgather_kernel<8>, grid, block, 0, STREAM(stream), pdl != 0, a);
}

PRISM_API int prism_scatter_rows(const void* partials, long long slab_stride, int P, int T, int H, int rows_per_owner,
                                 const void* const* peer_rs, const void* const* peer_flag, int tp, int my_rank, long long seq,
                                 const void* epoch, void* cta_counter, void* stream, int pdl) {
  if (T <= 0) return 0;
  if (tp < 1 || tp > 8 || P < 1 || rows_per_owner < 1 || (long long)rows_per_owner * tp < T) return -20;
  if (H % 8 || cta_counter == nullptr) return -21;
  ScatterRowsArgs a;
  a.partials = (const float*)partials;
  a.slab_stride = slab_stride;
  a.P = P;
  a.T = T;
  a.H = H;
  a.rows_per_owner = rows_per_owner;
  a.tp = tp;
  a.my_rank = my_rank;
  for (int p = 0; p < 8; ++p) {
    a.peer_rs[p] = p < tp ? (bf16*)const_cast<void*>(peer_rs[p]) : nullptr;
    a.peer_flag[p] = p < tp ? (unsigned long long*)const_cast<void*>(peer_flag[p]) : nullptr;
  }
  a.epoch = (const unsigned long long*)epoch;
  a.seq = (unsigned long long)seq;
  a.cta_counter = (int*)cta_counter;
  return (int)prism_launch(scatter_rows_kernel, dim3(T), dim3(128), 0, STREAM(stream), pdl != 0, a);
}

PRISM_API int prism_layernorm(const void* x, const void* w, const void* b, void* out, int T, int H, float eps,
                              void* stream, int pdl) {
  if (T <= 0) return 0;
  const unsigned long long addr = reinterpret_cast<unsigned long long>(x) | reinterpret_cast<unsigned long long>(w) |
                                  reinterpret_cast<unsigned long long>(b) | reinterpret_cast<unsigned long long>(out);
  if (H % 8 == 0 && H <= 32 * 8 * LN_VEC && (addr & 15ull) == 0) {
    return (int)prism_launch(layernorm_rows_kernel, dim3((T + 7) / 8), dim3(256), 0, STREAM(stream), pdl != 0, (const bf16*)x,
                             (const bf16*)w, (const bf16*)b, (bf16*)out, T, H, eps);
  }
  const size_t smem = (size_t)H * sizeof(float);
  return (int)prism_launch(layernorm_kernel, dim3(T), dim3(256), smem, STREAM(stream), pdl != 0, (const bf16*)x,
                           (const bf16*)w, (const bf16*)b, (bf16*)out, H, eps);
}

PRISM_API int prism_qk_norm_rope_store(const void* qkv, const void* partials, long long slab_stride, int P,
                                       long long row_stride, const void* positions, const void* q_weight,
                                       const void* k_weight, const void* inv_freq, const void* axis, void* q_out,
                                       long long q_stride, const void* slots, void* k_cache, void* v_cache,
                                       void* k_scale, void* v_scale, int T, int Hq, int Hkv, int D, int page,
                                       int kv_mode, int apply_norm, int apply_rope, float eps, int k_writeback,
                                       void* stream, int pdl) {
  if (T <= 0) return 0;
  QkvArgs a;
  a.qkv = (const bf16*)qkv;
  a.partials = (const float*)partials;
  a.slab_stride = slab_stride;
  a.P = P;
  a.row_stride = row_stride;
  a.positions = (const int*)positions;
  a.q_weight = (const bf16*)q_weight;
  a.k_weight = (const bf16*)k_weight;
  a.inv_freq = (const float*)inv_freq;
  a.axis = (const int*)axis;
  a.q_out = (bf16*)q_out;
  a.q_stride = q_stride;
  a.slots = (const long long*)slots;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.k_scale = (float*)k_scale;
  a.v_scale = (float*)v_scale;
  a.T = T;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.page = page;
  a.kv_mode = kv_mode;
  a.apply_norm = apply_norm;
  a.apply_rope = apply_rope;
  a.eps = eps;
  a.k_writeback = k_writeback;
  const int warps = T * (Hq + 2 * Hkv);
  const int wpb = 8;
  dim3 grid((warps + wpb - 1) / wpb), block(wpb * 32);
  if (D == 128 && qkv != nullptr && T >= 64 && (row_stride % 2) == 0 && (q_stride % 2) == 0 &&
      ((reinterpret_cast<unsigned long long>(qkv) | reinterpret_cast<unsigned long long>(q_out)) & 3ull) == 0) {
    return (int)prism_launch(qk_norm_rope_store_token_kernel, dim3(T), dim3(256), 0, STREAM(stream), pdl != 0, a);
  }
  if (D == 128) return (int)prism_launch(qk_norm_rope_store_kernel<128>, grid, block, 0, STREAM(stream), pdl != 0, a);
  if (D == 64) return (int)prism_launch(qk_norm_rope_store_kernel<64>, grid, block, 0, STREAM(stream), pdl != 0, a);
  return -2;
}

PRISM_API int prism_swiglu(const void* gu, const void* partials, long long slab_stride, int P, void* out, int T, int I,
                           void* stream, int pdl) {
  if (T <= 0) return 0;
  const size_t total = (size_t)T * I;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  return (int)prism_launch(swiglu_kernel, dim3(blocks), dim3(256), 0, STREAM(stream), pdl != 0, (const bf16*)gu,
                           (const float*)partials, slab_stride, P, (bf16*)out, T, I);
}

PRISM_API int prism_embed(const void* ids, const void* table, const void* visual, const void* vis_index, void* out,
                          int T, int H, long long vocab_start, long long vocab_end, void* stream, int pdl) {
  if (T <= 0) return 0;
  if (H % 8) return -1;
  return (int)prism_launch(embed_kernel, dim3(T), dim3(256), 0, STREAM(stream), pdl != 0, (const long long*)ids,
                           (const bf16*)table, (const bf16*)visual, (const int*)vis_index, (bf16*)out, H, vocab_start,
                           vocab_end);
}

PRISM_API int prism_indexed_add(void* hidden, const void* extra, const void* index, int T, int H, void* stream, int pdl) {
  if (T <= 0) return 0;
  return (int)prism_launch(indexed_add_kernel, dim3(T), dim3(256), 0, STREAM(stream), pdl != 0, (bf16*)hidden,
                           (const bf16*)extra, (const int*)index, H);
}

PRISM_API int prism_pos_embed_add(void* x, const void* table, const void* idx, const void* wt, int N, int H,
                                  void* stream, int pdl) {
  if (N <= 0) return 0;
  return (int)prism_launch(pos_embed_add_kernel, dim3(N), dim3(256), 0, STREAM(stream), pdl != 0, (bf16*)x,
                           (const bf16*)table, (const long long*)idx, (const float*)wt, N, H);
}

PRISM_API int prism_vit_rope(void* qkv, const void* coords, const void* inv_freq, int N, int heads, int hd, void* stream,
                             int pdl) {
  if (N <= 0) return 0;
  if (hd % 4 || hd > 256) return -1;
  return (int)prism_launch(vit_rope_kernel, dim3(N), dim3(256), 0, STREAM(stream), pdl != 0, (bf16*)qkv,
                           (const int*)coords, (const float*)inv_freq, N, heads, hd);
}
