// Allocation-free entry point of libprism_b200.so.  It has no counterpart in the
// reference project.
//
// Who needs it: code that drives the GPU from a context where device memory cannot be
// allocated, for example a real-time serving loop with a fixed memory plan, a plugin that
// runs inside another framework's memory pool and is forbidden to call cudaMalloc, or
// code that runs while a CUDA graph is being captured, where allocation calls are
// illegal.  Such callers cannot provide the split-KV scratch that prism_paged_decode
// expects, so this variant keeps that scratch inside the library.
//
//   int prism_paged_decode_noalloc(...)
//
// computes exactly what prism_paged_decode computes (one query token per sequence against
// the paged KV cache, all query heads of a KV head in one CTA, context split over nsplit
// CTAs and merged by a combine kernel).  The caller still passes every input and the
// output tensor; only the per-split partial results are placed in a file-scope
//   static __device__ __align__(256) unsigned char [PRISM_NOALLOC_SCRATCH_BYTES]
// array.
//
// Rules of use
//  * Limit: B * Hq * nsplit * (D + 2) floats (rounded up to 256 bytes) must fit in
//    PRISM_NOALLOC_SCRATCH_BYTES (4 MiB).  A larger request returns -10 and
//    prism_noalloc_last_error() explains which sizes were asked for.
//    prism_paged_decode_noalloc_scratch_bytes(B, Hq, D, nsplit) gives the requirement.
//  * Every GPU on which the library is loaded holds the 4 MiB array until the process ends.
//  * The first call on each device resolves the array's device address with
//    cudaGetSymbolAddress (with that device current) and caches it.  Make that first call
//    before starting any stream capture.
//  * The function never calls cudaMalloc, cudaFree or any allocating library routine.
//  * All calls on a device share the one array, and it keeps whatever the previous call
//    left there.  The kernels overwrite every cell they later read, so no clearing is
//    needed, but two calls whose kernels overlap on the GPU (different streams without an
//    ordering between them) race on the array: serialise them.
//  * num_blocks is the number of pages in the cache (0 if unknown).  A page id at or beyond
//    it, or a context longer than max_blocks * page, is skipped and recorded in the
//    library's status word (prism_status_attn) instead of being read.
//  * nsplit is clamped to 1..32 before the scratch requirement is computed.
//  * Returns 0 on success, a positive cudaError_t, or a negative validation code
//    (-10 too large, -13..-16 invalid Hq/Hkv, head dimension, page geometry or kv_mode).
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define PRISM_NOALLOC_SCRATCH_BYTES (4u << 20)

int prism_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const void* k_scale,
                               const void* v_scale, const void* block_tables, const void* context_lens, void* out,
                               int B, int Hq, int Hkv, int D, int page, int max_blocks, int num_blocks, int nsplit,
                               int kv_mode, float scale, void* stream);

long long prism_paged_decode_noalloc_scratch_bytes(int B, int Hq, int D, int nsplit);

const char* prism_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
