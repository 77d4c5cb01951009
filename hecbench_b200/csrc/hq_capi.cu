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
    default: return "unknown status";
  }
}

}  // extern "C"

// ---- streaming-read probe: what a kernel that only reads `bytes` once achieves ----
namespace hq {
namespace {
__global__ void stream_read_kernel(const uint4* __restrict__ src, size_t nvec, unsigned* sink) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  unsigned acc = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const size_t j = i + u * stride;
      v[u] = j < nvec ? ldg_stream_u4(src + j) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; u++) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  if (acc == 0x9e3779b9u) sink[0] = acc;  // keeps the loads alive; practically never true
}
}  // namespace
}  // namespace hq

extern "C" int hq_probe_stream_read(const void* src, size_t bytes, unsigned* sink,
                                    hq_stream_t stream) {
  using namespace hq;
  if (!src || !sink) return HQ_ERR_NULL_POINTER;
  if (!aligned16(src)) return HQ_ERR_MISALIGNED;
  const size_t nvec = bytes / 16;
  if (nvec == 0) return HQ_OK;
  stream_read_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(src), nvec, sink);
  return launch_status();
}
