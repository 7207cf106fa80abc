// Host-side registration of an L2 prefetch that the next prefetch-capable launch carries.
#include "common.cuh"

namespace {
PrefetchSpec g_pending = {nullptr, 0, 0, 0, 0};
}

PrefetchSpec prism_take_prefetch() {
  PrefetchSpec p = g_pending;
  g_pending = PrefetchSpec{nullptr, 0, 0, 0, 0};
  return p;
}

// Ask the next launch of a prefetch-capable kernel (add+RMSNorm, QK-norm + rotary + KV store,
// paged decode attention) to request `rows` runs of `bytes` bytes, `stride` bytes apart,
// starting at `base`, into L2; kernels with a narrow grid add `helpers` CTAs that only issue requests.  Invalid requests are refused with -1 and nothing is registered.
PRISM_API int prism_set_next_prefetch(const void* base, long long stride, int rows, int bytes, int helpers) {
  if (base == nullptr || rows <= 0 || bytes <= 0) {
    g_pending = PrefetchSpec{nullptr, 0, 0, 0, 0};
    return 0;
  }
  if ((reinterpret_cast<unsigned long long>(base) & 127ull) || (stride & 127) || (bytes & 127) || stride < bytes) return -1;
  if (helpers < 0 || helpers > 1024) return -1;
  g_pending = PrefetchSpec{reinterpret_cast<const char*>(base), stride, rows, bytes, helpers};
  return 0;
}
