// Sampler: greedy arg-max with lowest-id tie break and temperature sampling by the
// exponential race (argmax of logits/T + Gumbel noise == sampling from softmax(logits/T)),
// in one launch for mixed batches.  Reference: prism_infer/layers/sampler.py:10-55 (compiled
// softmax / Exp(1) argmax) and the local-max step of
// prism_infer/layers/embed_head.py:103-125.
//
// The kernel reduces fp32 logits given as P split slabs (the LM-head GEMM's fp32 output is
// one slab), and can emit (best value, global id) pairs so tensor-parallel ranks can
// exchange their vocabulary-shard winners.
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(sampler)

namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// temperature[b] == 0 -> greedy.  out_val may be null.  vocab_offset is added to ids.
__global__ void __launch_bounds__(1024) sample_kernel(const float* logits, long long row_stride, long long slab_stride,
                                                      int P, const float* temperature, long long* out_id,
                                                      float* out_val, int V, long long vocab_offset,
                                                      unsigned long long seed, const long long* step,
                                                      float* cand_val, long long* cand_id) {
  const int b = blockIdx.x;
  // blockIdx.y selects a contiguous chunk of the vocabulary; with gridDim.y > 1 the winners
  // go to cand_val / cand_id ([chunk][B]) and merge_candidates_kernel picks the final one.
  pdl_launch_dependents();
  pdl_wait();
  const float temp = temperature ? temperature[b] : 0.0f;
  const unsigned long long stp = step ? (unsigned long long)step[0] : 0ull;
  const float* row = logits + (size_t)b * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int chunk = (V + gridDim.y - 1) / gridDim.y;
  const int i_begin = blockIdx.y * chunk, i_end = min(V, i_begin + chunk);
  for (int i = i_begin + threadIdx.x; i < i_end; i += blockDim.x) {
    float v = 0.0f;
    for (int p = 0; p < P; ++p) v += row[(size_t)p * slab_stride + i];
    if (temp > 0.0f) {
      const uint64_t h = mix64(seed ^ mix64((stp << 20) ^ ((uint64_t)b << 40) ^ (uint64_t)(i + vocab_offset)));
      const float u = ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
      v = v / temp - __logf(-__logf(u));
    }
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    best_i = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (lane == 0) {
      if (gridDim.y > 1) {
        cand_val[(size_t)blockIdx.y * gridDim.x + b] = best;
        cand_id[(size_t)blockIdx.y * gridDim.x + b] = (long long)best_i + vocab_offset;
      } else {
        out_id[b] = (long long)best_i + vocab_offset;
        if (out_val) out_val[b] = best;
      }
    }
  }
}

// Winner over R candidate (value, id) pairs per row: vals [R][B], ids [R][B].
__global__ void merge_candidates_kernel(const float* vals, const long long* ids, long long* out, float* out_val, int R,
                                        int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (b >= B) return;
  float best = -INFINITY;
  long long best_i = 0x7fffffffffffffffll;
  for (int r = 0; r < R; ++r) {
    const float v = vals[(size_t)r * B + b];
    const long long i = ids[(size_t)r * B + b];
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
  out[b] = best_i;
  if (out_val) out_val[b] = best;
}

}  // namespace

// cand_val / cand_id: scratch of chunks * B entries each (chunks > 1 spreads a row over
// several CTAs; required to keep a 150k-entry row from being read by a single CTA).
PRISM_API int prism_sample(const void* logits, long long row_stride, long long slab_stride, int P,
                           const void* temperature, void* out_id, void* out_val, int B, int V, long long vocab_offset,
                           unsigned long long seed, const void* step, void* cand_val, void* cand_id, int chunks,
                           void* stream, int pdl) {
  if (B <= 0) return 0;
  if (chunks < 1 || cand_val == nullptr || cand_id == nullptr) chunks = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc = (int)prism_launch(sample_kernel, dim3(B, chunks), dim3(chunks > 1 ? 256 : 1024), 0, s, pdl != 0,
                             (const float*)logits, row_stride, slab_stride, P < 1 ? 1 : P, (const float*)temperature,
                             (long long*)out_id, (float*)out_val, V, vocab_offset, seed, (const long long*)step,
                             (float*)cand_val, (long long*)cand_id);
  if (rc || chunks == 1) return rc;
  return (int)prism_launch(merge_candidates_kernel, dim3((B + 127) / 128), dim3(128), 0, s, pdl != 0,
                           (const float*)cand_val, (const long long*)cand_id, (long long*)out_id, (float*)out_val, chunks,
                           B);
}

PRISM_API int prism_merge_candidates(const void* vals, const void* ids, void* out, int R, int B, void* stream, int pdl) {
  if (B <= 0) return 0;
  return (int)prism_launch(merge_candidates_kernel, dim3((B + 127) / 128), dim3(128), 0,
                           reinterpret_cast<cudaStream_t>(stream), pdl != 0, (const float*)vals, (const long long*)ids,
                           (long long*)out, (float*)nullptr, R, B);
}
