// Symmetric-memory plumbing for the tensor-parallel ranks of one node.
//
// Each rank allocates one device region (flags, step epoch word, CTA counters, two slab
// buffers), exports it with CUDA IPC and maps every peer's region, which gives kernels
// plain peer pointers for st / ld over NVLink.  The fused GEMM -> exchange kernels
// (prism_gemm_wx_push in gemm_tcgen05.cu, prism_add_rmsnorm_wait in norm_rope_kv.cu) use
// those pointers; this file holds the allocation / mapping helpers, the step epoch kernel
// and a distributed arg-max merge.  The reference has no counterpart: its ranks only talk
// through NCCL all-reduce (prism_infer/layers/linear.py:186-190).
//
// Flags are monotonically increasing 64-bit sequence numbers (*epoch + exchange point), so
// nothing is ever reset while a graph replays, and every wait is bounded.
#include <cstring>

#include "common.cuh"

PRISM_DEFINE_TU_STATUS(comm)

namespace {

__global__ void epoch_advance_kernel(unsigned long long* epoch, unsigned long long delta) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) *epoch += delta;
}

// One-shot exchange of per-rank (value, id) winners: every rank writes its pair for each
// row into slot [my_rank] of every peer, raises the flag, waits for all peers, then takes
// the best pair (ties -> lowest id).  vals/ids buffers: [tp][B] per rank.
struct ArgmaxArgs {
  const float* local_val;   // [B]
  const long long* local_id;
  float* peer_val[8];       // base of [tp][Bmax] on every rank
  long long* peer_id[8];
  unsigned long long* peer_flag[8];
  const unsigned long long* wait_flags;  // local [tp]
  const unsigned long long* epoch;
  long long* out;           // [B]
  int n_peers, my_rank, point, B, Bmax;
};

__global__ void __launch_bounds__(256) argmax_exchange_kernel(const ArgmaxArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned long long seq = *a.epoch + (unsigned long long)a.point;
  for (int b = threadIdx.x; b < a.B; b += blockDim.x) {
    const float v = a.local_val[b];
    const long long id = a.local_id[b];
    for (int p = 0; p < a.n_peers; ++p) {
      a.peer_val[p][(size_t)a.my_rank * a.Bmax + b] = v;
      a.peer_id[p][(size_t)a.my_rank * a.Bmax + b] = id;
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < a.n_peers) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.peer_flag[threadIdx.x] + a.my_rank), "l"(seq) : "memory");
    // bounded wait for the same sequence number from that peer
    const long long t0 = clock64();
    bool ok = false;
    for (;;) {
      unsigned long long v;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(a.wait_flags + threadIdx.x) : "memory");
      if (v >= seq) {
        ok = true;
        break;
      }
      if (clock64() - t0 > PRISM_WAIT_CYCLES) break;
    }
    if (!ok) prism_report(PRISM_ERR_PEER_TIMEOUT, 100 + threadIdx.x);
  }
  __syncthreads();
  const float* lv = a.peer_val[a.my_rank];
  const long long* li = a.peer_id[a.my_rank];
  for (int b = threadIdx.x; b < a.B; b += blockDim.x) {
    float best = -INFINITY;
    long long best_i = 0x7fffffffffffffffll;
    for (int r = 0; r < a.n_peers; ++r) {
      const float v = __ldcg(lv + (size_t)r * a.Bmax + b);
      const long long i = __ldcg(li + (size_t)r * a.Bmax + b);
      if (v > best || (v == best && i < best_i)) {
        best = v;
        best_i = i;
      }
    }
    a.out[b] = best_i;
  }
}

// Raise flag[my_rank] = seq on every peer (a rank that had nothing to contribute).
struct SignalArgs {
  unsigned long long* peer_flag[8];
  int n_peers, my_rank;
  unsigned long long seq;
};
__global__ void signal_kernel(const SignalArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)threadIdx.x < a.n_peers) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.peer_flag[threadIdx.x] + a.my_rank), "l"(a.seq) : "memory");
  }
}

// Bounded wait until flags[0..n) >= seq (data other GPUs pushed is then visible to the
// kernels that follow in the stream).
__global__ void wait_flags_kernel(const unsigned long long* flags, int n, unsigned long long seq,
                                  const unsigned long long* epoch) {
  pdl_launch_dependents();
  pdl_wait();
  if (epoch != nullptr) seq += *epoch;  // the step epoch is advanced by a kernel, so graph replays wait for fresh numbers
  if ((int)threadIdx.x < n) {
    const long long t0 = clock64();
    bool ok = false;
    for (;;) {
      unsigned long long v;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + threadIdx.x) : "memory");
      if (v >= seq) {
        ok = true;
        break;
      }
      if (clock64() - t0 > PRISM_WAIT_CYCLES) break;
    }
    if (!ok) prism_report(PRISM_ERR_PEER_TIMEOUT, 200 + threadIdx.x);
  }
}

}  // namespace

PRISM_API int prism_signal_peers(const void* const* peer_flag, int n_peers, int my_rank, long long seq, void* stream) {
  if (n_peers < 1 || n_peers > 8) return -20;
  SignalArgs a;
  for (int p = 0; p < 8; ++p) a.peer_flag[p] = p < n_peers ? (unsigned long long*)peer_flag[p] : nullptr;
  a.n_peers = n_peers;
  a.my_rank = my_rank;
  a.seq = (unsigned long long)seq;
  return (int)prism_launch(signal_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), false, a);
}

PRISM_API int prism_wait_flags(const void* flags, int n, long long seq, const void* epoch, void* stream) {
  if (n < 1 || n > 32) return -20;
  return (int)prism_launch(wait_flags_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), false,
                           (const unsigned long long*)flags, n, (unsigned long long)seq, (const unsigned long long*)epoch);
}

PRISM_API int prism_ipc_alloc(long long bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}

PRISM_API int prism_ipc_free(void* p) { return (int)cudaFree(p); }

PRISM_API int prism_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

PRISM_API int prism_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}

PRISM_API int prism_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }

PRISM_API int prism_epoch_advance(void* epoch, long long delta, void* stream, int pdl) {
  return (int)prism_launch(epoch_advance_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), pdl != 0,
                           (unsigned long long*)epoch, (unsigned long long)delta);
}

PRISM_API int prism_argmax_exchange(const void* local_val, const void* local_id, const void* const* peer_val,
                                    const void* const* peer_id, const void* const* peer_flag, const void* wait_flags,
                                    const void* epoch, void* out, int n_peers, int my_rank, int point, int B, int Bmax,
                                    void* stream, int pdl) {
  if (n_peers < 1 || n_peers > 8) return -20;
  ArgmaxArgs a;
  a.local_val = (const float*)local_val;
  a.local_id = (const long long*)local_id;
  for (int p = 0; p < 8; ++p) {
    a.peer_val[p] = p < n_peers ? (float*)peer_val[p] : nullptr;
    a.peer_id[p] = p < n_peers ? (long long*)peer_id[p] : nullptr;
    a.peer_flag[p] = p < n_peers ? (unsigned long long*)peer_flag[p] : nullptr;
  }
  a.wait_flags = (const unsigned long long*)wait_flags;
  a.epoch = (const unsigned long long*)epoch;
  a.out = (long long*)out;
  a.n_peers = n_peers;
  a.my_rank = my_rank;
  a.point = point;
  a.B = B;
  a.Bmax = Bmax;
  return (int)prism_launch(argmax_exchange_kernel, dim3(1), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), pdl != 0, a);
}
