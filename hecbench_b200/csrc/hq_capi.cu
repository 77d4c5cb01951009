// Library-wide pieces of the C ABI: version, status strings, per-thread error
// record and the cached SM count.
#include <vector>

#include "hq_common.cuh"

namespace hq {

int& last_cuda_error_ref() {
  static thread_local int err = 0;
  return err;
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return cached;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      cached = n;
    cached_dev = dev;
  }
  return cached;
}

#ifdef HQ_BOUNDS_CHECK
namespace {
std::vector<BoundsAccess>& bounds_accessors() {
  static std::vector<BoundsAccess> v;
  return v;
}
}  // namespace
void register_bounds_access(BoundsAccess fn) { bounds_accessors().push_back(fn); }
#endif

int reserved_smem_per_block() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 1024;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return cached;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrReservedSharedMemoryPerBlock, dev) == cudaSuccess)
      cached = n;
    cached_dev = dev;
  }
  return cached;
}

}  // namespace hq

extern "C" {

int hq_version(void) { return 100; }

int hq_last_cuda_error(void) { return hq::last_cuda_error_ref(); }

int hq_bounds_check_report(unsigned* violations, unsigned* site, unsigned long long* offset,
                           unsigned long long* extent, int reset) {
#ifdef HQ_BOUNDS_CHECK
  unsigned total = 0, first_site = 0;
  unsigned long long first_off = 0, first_ext = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return hq::cuda_status(e);
  for (hq::BoundsAccess fn : hq::bounds_accessors()) {
    hq::BoundsRecord r;
    e = fn(&r, reset != 0);
    if (e != cudaSuccess) return hq::cuda_status(e);
    if (r.violations != 0 && total == 0) {
      first_site = r.site;
      first_off = r.offset;
      first_ext = r.extent;
    }
    total += r.violations;
  }
  if (violations) *violations = total;
  if (site) *site = first_site;
  if (offset) *offset = first_off;
  if (extent) *extent = first_ext;
  return HQ_OK;
#else
  (void)violations; (void)site; (void)offset; (void)extent; (void)reset;
  return HQ_ERR_UNSUPPORTED;  // this library was built without -DHQ_BOUNDS_CHECK
#endif
}

const char* hq_status_string(int status) {
  switch (status) {
    case HQ_OK: return "ok";
    case HQ_ERR_BAD_SHAPE: return "bad shape";
    case HQ_ERR_NULL_POINTER: return "null pointer";
    case HQ_ERR_MISALIGNED: return "misaligned pointer";
    case HQ_ERR_CUDA: return "CUDA runtime error";
    case HQ_ERR_WORKSPACE: return "workspace missing or too small";
    case HQ_ERR_UNSUPPORTED: return "unsupported configuration";
    case HQ_ERR_TOO_LARGE: return "size beyond supported maximum";
    case HQ_ERR_NCCL: return "NCCL call failed";
    default: return "unknown status";
  }
}

}  // extern "C"
