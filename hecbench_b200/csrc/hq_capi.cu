// Library-wide pieces of the C ABI: version, status strings, per-thread error
// record and the cached SM count.
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
