// Measurement aid of bench.py, NOT part of the C ABI of libhq.so (it is built
// into hecbench_b200/libhq_probe.so): a kernel that reads `bytes` bytes from
// src exactly once with 128-bit streaming loads and does nothing else.  Timed
// like the real kernels it gives the ceiling a kernel of that footprint can
// reach on this GPU, launch and ramp included.  sink is one device word.
//   int hq_probe_stream_read(const void* src, size_t bytes, unsigned* sink, cudaStream_t stream)
#include "../hq_common.cuh"

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
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = sms * 8;
  stream_read_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(src), nvec, sink);
  return (cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA);
}
