// Weight-streaming matrix-vector products for decode steps of at most four tokens.
//
// With one to four tokens a projection has no operand reuse: it is a pure stream of the
// weight matrix, and what matters besides bandwidth is the fixed latency of the kernel,
// because a decode step is a chain of ~250 dependent launches.  This kernel has no tensor
// map, TMEM allocation or mbarrier ring to set up: every warp owns whole weight rows, keeps
// two register buffers of 16-byte loads in flight, reduces with shuffles and writes the
// finished outputs (no split-K partial slabs for the consumer to sum).  The first buffer of
// weights is requested before griddepcontrol.wait, so under programmatic dependent launch
// the stream starts while the previous kernel is still draining.  The tcgen05 GEMM
// (gemm_tcgen05.cu) takes over from five tokens.
//
// Output forms: fp32 out[t][m]; dual = bf16 silu(Wg x) * (Wu x) with the rounding points of
// the separate kernels; push = the tensor-parallel exchange form of prism_gemm_wx_push
// (8-byte {value, sequence} words into slab `my_rank` of every rank's buffer).
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(gemv)

namespace {

constexpr int GEMV_WARPS = 16;
// 16-byte loads in flight per lane, buffer and weight stream: 8 (a buffer covers 2048 elements
// of a row); 4 for the dual form, which streams two rows at once
constexpr int GEMV_TMAX = 4;

struct GemvArgs {
  const __nv_bfloat16* W;
  const __nv_bfloat16* X;
  void* out;
  int M, T, K;
  long long ldw, ldx, ldo;
  int w2_row_off;  // dual: first row of the second matrix
  // push form
  int n_peers, my_rank;
  long long point;
  long long slab_stride;  // 8-byte elements between slabs
  const unsigned long long* epoch;
  unsigned long long* peer_out[8];
};

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void fma8(float (&acc)[GEMV_TMAX], const uint4& w, const __nv_bfloat16* xs, int K, int col, int T) {
  const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
  float2 wf[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) wf[e] = __bfloat1622float2(wp[e]);
#pragma unroll
  for (int t = 0; t < GEMV_TMAX; ++t) {
    if (t < T) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)t * K + col);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 xf = __bfloat1622float2(xp[e]);
        acc[t] = fmaf(wf[e].x, xf.x, acc[t]);
        acc[t] = fmaf(wf[e].y, xf.y, acc[t]);
      }
    }
  }
}

// MODE 0: fp32 out, 1: dual SwiGLU bf16 out, 2: push
template <int MODE>
__global__ void __launch_bounds__(GEMV_WARPS * 32, 1) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t gsm[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gsm);  // [T][K]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * GEMV_WARPS + warp;
  const int nw = gridDim.x * GEMV_WARPS;
  const int K = a.K;
  constexpr int NS = MODE == 1 ? 2 : 1;  // weight streams per unit
  constexpr int GEMV_U = MODE == 1 ? 4 : 8;
  constexpr int GEMV_CHUNK = GEMV_U * 32 * 8;
  pdl_launch_dependents();

  // (row, chunk) walk of this warp, flattened so the two register buffers alternate across
  // chunk and row boundaries
  const int chunks = (K + GEMV_CHUNK - 1) / GEMV_CHUNK;
  const int rows_mine = gw < a.M ? (a.M - gw + nw - 1) / nw : 0;
  const int steps = rows_mine * chunks;
  uint4 buf[2][NS][GEMV_U];
  auto issue = [&](int step, int b) {
    const int m = gw + (step / chunks) * nw;
    const int k0 = (step % chunks) * GEMV_CHUNK;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const __nv_bfloat16* row = a.W + (size_t)(m + s * a.w2_row_off) * a.ldw + k0;
#pragma unroll
      for (int u = 0; u < GEMV_U; ++u) {
        const int col = (u * 32 + lane) * 8;
        buf[b][s][u] = (k0 + col < K) ? ld_stream16(row + col) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  if (steps > 0) issue(0, 0);  // weights never depend on the previous kernel
  pdl_wait();
  for (int i = threadIdx.x; i < a.T * K / 8; i += blockDim.x) {
    const int t = i / (K / 8), c = i % (K / 8);
    *reinterpret_cast<uint4*>(xs + (size_t)t * K + c * 8) = *reinterpret_cast<const uint4*>(a.X + (size_t)t * a.ldx + c * 8);
  }
  __syncthreads();
  unsigned long long seq = 0;
  if (MODE == 2) seq = (((a.epoch ? *a.epoch : 0ull) + (unsigned long long)a.point) & 0xffffffffull) << 32;

  float acc[NS][GEMV_TMAX];
#pragma unroll
  for (int s = 0; s < NS; ++s)
#pragma unroll
    for (int t = 0; t < GEMV_TMAX; ++t) acc[s][t] = 0.0f;
  for (int step = 0; step < steps; ++step) {
    const int b = step & 1;
    if (step + 1 < steps) {
      if (b == 0) issue(step + 1, 1);
      else issue(step + 1, 0);
    }
    const int k0 = (step % chunks) * GEMV_CHUNK;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
#pragma unroll
      for (int u = 0; u < GEMV_U; ++u) {
        const int col = k0 + (u * 32 + lane) * 8;
        if (col < K) {
          if (b == 0) fma8(acc[s], buf[0][s][u], xs, K, col, a.T);
          else fma8(acc[s], buf[1][s][u], xs, K, col, a.T);
        }
      }
    }
    if (step % chunks == chunks - 1) {  // row finished
      const int m = gw + (step / chunks) * nw;
#pragma unroll
      for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int t = 0; t < GEMV_TMAX; ++t) acc[s][t] = warp_sum(acc[s][t]);
      if (lane == 0) {
#pragma unroll
        for (int t = 0; t < GEMV_TMAX; ++t) {
          if (t < a.T) {
            if (MODE == 0) {
              reinterpret_cast<float*>(a.out)[(size_t)t * a.ldo + m] = acc[0][t];
            } else if (MODE == 1) {
              const float g = bf16_round(acc[0][t]), u = bf16_round(acc[NS - 1][t]);
              reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)t * a.ldo + m] = __float2bfloat16_rn(bf16_round(silu(g)) * u);
            } else {
              const unsigned long long word = seq | (unsigned long long)__float_as_uint(acc[0][t]);
              const size_t off = (size_t)a.my_rank * a.slab_stride + (size_t)t * a.ldo + m;
              for (int p = 0; p < a.n_peers; ++p)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.peer_out[p] + off), "l"(word) : "memory");
            }
          }
        }
      }
#pragma unroll
      for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int t = 0; t < GEMV_TMAX; ++t) acc[s][t] = 0.0f;
    }
  }
}

int g_gemv_sms = 0;

template <int MODE>
int launch_gemv(const GemvArgs& a, cudaStream_t stream, bool pdl) {
  const size_t smem = (size_t)a.T * a.K * 2;
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  if (g_gemv_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_gemv_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      g_gemv_sms = 148;
  }
  int grid = (a.M + GEMV_WARPS - 1) / GEMV_WARPS;
  if (grid > g_gemv_sms) grid = g_gemv_sms;
  return (int)prism_launch(gemv_kernel<MODE>, dim3(grid), dim3(GEMV_WARPS * 32), smem, stream, pdl, a);
}

}  // namespace

// out: mode 0 fp32 [T][ldo], mode 1 (dual) bf16 [T][ldo] with the second matrix starting at row
// w2_row_off, mode 2 (push) 8-byte words into slab my_rank of peer_out[p] (row stride ldo, slab
// stride slab_stride, in 8-byte elements).  T <= 4, K a multiple of 8, 16-byte aligned rows.
PRISM_API int prism_gemv(const void* W, const void* X, void* out, int M, int T, int K, long long ldw, long long ldx,
                         long long ldo, int mode, int w2_row_off, const void* const* peer_out, int n_peers, int my_rank,
                         long long point, long long slab_stride, const void* epoch, void* stream, int pdl) {
  if (T < 1 || T > GEMV_TMAX || (K % 8) || (ldw % 8) || (ldx % 8)) return -1;
  if ((reinterpret_cast<unsigned long long>(W) | reinterpret_cast<unsigned long long>(X)) & 15ull) return -2;
  if ((size_t)T * K * 2 > 200 * 1024) return -3;
  GemvArgs a;
  a.W = reinterpret_cast<const __nv_bfloat16*>(W);
  a.X = reinterpret_cast<const __nv_bfloat16*>(X);
  a.out = out;
  a.M = M;
  a.T = T;
  a.K = K;
  a.ldw = ldw;
  a.ldx = ldx;
  a.ldo = ldo;
  a.w2_row_off = w2_row_off;
  a.n_peers = 0;
  a.my_rank = my_rank;
  a.point = point;
  a.slab_stride = slab_stride;
  a.epoch = reinterpret_cast<const unsigned long long*>(epoch);
  for (int p = 0; p < 8; ++p) a.peer_out[p] = nullptr;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (mode) {
    case 0: return launch_gemv<0>(a, s, pdl != 0);
    case 1: return launch_gemv<1>(a, s, pdl != 0);
    case 2:
      if (n_peers < 1 || n_peers > 8 || peer_out == nullptr) return -4;
      a.n_peers = n_peers;
      for (int p = 0; p < n_peers; ++p) a.peer_out[p] = reinterpret_cast<unsigned long long*>(const_cast<void*>(peer_out[p]));
      return launch_gemv<2>(a, s, pdl != 0);
  }
  return -5;
}
