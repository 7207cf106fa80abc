// KV-cache maintenance kernels: page copies (copy-on-write, prefix-row copies, swap to and
// from pinned host pages) and physical prefix compaction.  Payload and scales move in the
// same launch.  The cache is one allocation [2 (K,V)][layers][blocks][Hkv][page][D] plus
// scales [2][layers][blocks][Hkv][page]; a "slab" below is one (K|V, layer) slice.
// Reference behaviour: prism_infer/engine/model_runner.py:908-1031 (one copy_ per pair and
// tensor) and prism_infer/ops/kv_compaction.py:32-191 (gather then scatter, twice).
#include "common.cuh"

PRISM_DEFINE_TU_STATUS(kvops)

namespace {

struct Plane {
  const uint8_t* src;
  uint8_t* dst;
  long long src_slab_stride;  // bytes between slabs in the source allocation
  long long dst_slab_stride;
  int row_bytes;              // bytes of one token row for one head (D * elem, or 4 for scales)
};

struct CopyArgs {
  Plane plane[2];
  int n_planes;
  const int* src_blocks;  // [pairs]
  const int* dst_blocks;  // [pairs]
  const int* n_rows;      // [pairs] rows (tokens) to copy from the start of the page; null = whole page
  int Hkv, page, n_slabs;
};

// grid: (pairs, n_slabs * Hkv, n_planes)
__global__ void __launch_bounds__(256) page_copy_kernel(const CopyArgs a) {
  const int pair = blockIdx.x;
  const int slab = blockIdx.y / a.Hkv, h = blockIdx.y % a.Hkv;
  const Plane& p = a.plane[blockIdx.z];
  const int rows = a.n_rows ? a.n_rows[pair] : a.page;
  const size_t bytes = (size_t)rows * p.row_bytes;
  const size_t page_bytes = (size_t)a.page * p.row_bytes;
  const uint8_t* s = p.src + (size_t)slab * p.src_slab_stride + ((size_t)a.src_blocks[pair] * a.Hkv + h) * page_bytes;
  uint8_t* d = p.dst + (size_t)slab * p.dst_slab_stride + ((size_t)a.dst_blocks[pair] * a.Hkv + h) * page_bytes;
  if ((p.row_bytes & 15) == 0) {
    for (size_t i = (size_t)threadIdx.x * 16; i < bytes; i += (size_t)blockDim.x * 16)
      *reinterpret_cast<uint4*>(d + i) = *reinterpret_cast<const uint4*>(s + i);
  } else {
    for (size_t i = (size_t)threadIdx.x * 4; i < bytes; i += (size_t)blockDim.x * 4)
      *reinterpret_cast<uint32_t*>(d + i) = *reinterpret_cast<const uint32_t*>(s + i);
  }
}

struct GatherArgs {
  uint8_t* cache[2];         // payload, scales
  long long slab_stride[2];  // bytes
  int row_bytes[2];
  uint8_t* temp[2];          // [n_slabs][Hkv][R][row_bytes]
  const long long* slots;    // [R] flat slots (block * page + offset)
  int R, Hkv, page, n_slabs, n_planes;
  int scatter;               // 0: cache -> temp, 1: temp -> cache
};

// grid: (ceil(R / rows_per_block), n_slabs * Hkv, n_planes); one warp per row
__global__ void __launch_bounds__(256) slot_move_kernel(const GatherArgs a) {
  const int pl = blockIdx.z;
  const int slab = blockIdx.y / a.Hkv, h = blockIdx.y % a.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + warp;
  if (r >= a.R) return;
  const long long slot = a.slots[r];
  const int rb = a.row_bytes[pl];
  uint8_t* c = a.cache[pl] + (size_t)slab * a.slab_stride[pl] +
               (((size_t)(slot / a.page) * a.Hkv + h) * a.page + (size_t)(slot % a.page)) * rb;
  uint8_t* t = a.temp[pl] + (((size_t)slab * a.Hkv + h) * a.R + r) * rb;
  const uint8_t* s = a.scatter ? t : c;
  uint8_t* d = a.scatter ? c : t;
  for (int i = lane * 4; i < rb; i += 128) *reinterpret_cast<uint32_t*>(d + i) = *reinterpret_cast<const uint32_t*>(s + i);
}

}  // namespace

// Copies page prefixes src_blocks[i] -> dst_blocks[i] for every slab and head.  Plane 0 is
// the payload, plane 1 (optional, scale_src == null to skip) the fp32 scales.  Source and
// destination may be different allocations (device cache <-> pinned host swap pool).
PRISM_API int prism_kv_page_copy(const void* src, void* dst, long long src_slab_stride, long long dst_slab_stride,
                                 int row_bytes, const void* scale_src, void* scale_dst, long long scale_src_slab_stride,
                                 long long scale_dst_slab_stride, const void* src_blocks, const void* dst_blocks,
                                 const void* n_rows, int pairs, int Hkv, int page, int n_slabs, void* stream) {
  if (pairs <= 0) return 0;
  CopyArgs a;
  a.plane[0] = Plane{(const uint8_t*)src, (uint8_t*)dst, src_slab_stride, dst_slab_stride, row_bytes};
  a.n_planes = 1;
  if (scale_src != nullptr) {
    a.plane[1] = Plane{(const uint8_t*)scale_src, (uint8_t*)scale_dst, scale_src_slab_stride, scale_dst_slab_stride, 4};
    a.n_planes = 2;
  } else {
    a.plane[1] = a.plane[0];
  }
  a.src_blocks = (const int*)src_blocks;
  a.dst_blocks = (const int*)dst_blocks;
  a.n_rows = (const int*)n_rows;
  a.Hkv = Hkv;
  a.page = page;
  a.n_slabs = n_slabs;
  dim3 grid(pairs, n_slabs * Hkv, a.n_planes);
  page_copy_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

// Two-phase physical compaction: rows at src_slots are gathered into `temp` (scratch of
// n_slabs*Hkv*R*row_bytes bytes, plus n_slabs*Hkv*R*4 for scales) and then scattered to
// dst_slots, so overlapping source and destination ranges are safe.
PRISM_API int prism_kv_compact(void* cache, long long slab_stride, int row_bytes, void* scales, long long scale_slab_stride,
                               void* temp, void* scale_temp, const void* src_slots, const void* dst_slots, int R, int Hkv,
                               int page, int n_slabs, void* stream) {
  if (R <= 0) return 0;
  GatherArgs a;
  a.cache[0] = (uint8_t*)cache;
  a.cache[1] = (uint8_t*)scales;
  a.slab_stride[0] = slab_stride;
  a.slab_stride[1] = scale_slab_stride;
  a.row_bytes[0] = row_bytes;
  a.row_bytes[1] = 4;
  a.temp[0] = (uint8_t*)temp;
  a.temp[1] = (uint8_t*)scale_temp;
  a.R = R;
  a.Hkv = Hkv;
  a.page = page;
  a.n_slabs = n_slabs;
  a.n_planes = scales != nullptr ? 2 : 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((R + 7) / 8, n_slabs * Hkv, a.n_planes);
  a.slots = (const long long*)src_slots;
  a.scatter = 0;
  slot_move_kernel<<<grid, 256, 0, s>>>(a);
  a.slots = (const long long*)dst_slots;
  a.scatter = 1;
  slot_move_kernel<<<grid, 256, 0, s>>>(a);
  return (int)cudaGetLastError();
}
