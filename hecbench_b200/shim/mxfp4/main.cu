// Driver with the command line and output of HeCBench's mxfp4 benchmark
// (src/mxfp4-cuda/main.cu:152-245) on top of libhq.so.
//
// In the reference the kernel is defined inside the driver's translation unit,
// so a link-time swap is impossible; this driver keeps its argv (<number of
// elements> <repeat>), its two sections (fp16, then bf16), its inputs
// (srand(123); every group of 32 draws from the driver's list of 31 values and
// gets one +-6 at a random place), its timing printout and its check - the
// reference's own verify.h, taken from the include path at build time - and
// replaces only the kernel launch (reference main.cu:152-166) by hq_mxfp4_qdq.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <type_traits>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "verify.h"
#include "hq.h"

template <typename T>
static void section(int numel, int niters) {
  constexpr bool is_half = std::is_same<T, __half>::value;
  printf(is_half ? "\nSimulate conversion between FP16 and FP4\n"
                 : "\nSimulate conversion between BF16 and FP4\n");
  std::vector<T> src(numel), dst(numel);
  // the functional test values of the reference driver (main.cu:178-182)
  const float v[] = {0.0, 0.5, 1.0, 1.5, 2, 3, 4, -0.0, -0.5, -1.0, -1.5, -2, -3, -4, 0.25, 0.75,
                     1.25, 1.75, 2.5, 3.5, 5, 0.1, 0.3, 0.4, 0.6, 0.9, -0.1, -0.3, -0.4, -0.6, -0.9};
  const int nv = (int)(sizeof(v) / sizeof(v[0]));
  srand(123);
  for (int i = 0; i < numel / 32; i++) {
    for (int j = i * 32; j < (i + 1) * 32; j++) src[j] = v[rand() % nv];
    const int r = rand() % 32;
    src[i * 32 + r] = r < 16 ? 6 : -6;
  }
  const size_t bytes = (size_t)numel * sizeof(T);
  T *d_src, *d_dst;
  cudaMalloc((void**)&d_src, bytes);
  cudaMalloc((void**)&d_dst, bytes);
  cudaMemcpy(d_src, src.data(), bytes, cudaMemcpyHostToDevice);

  int status = 0;
  const auto start = std::chrono::high_resolution_clock::now();
  for (int i = 0; i < niters; i++) {
    const int st = hq_mxfp4_qdq(d_src, d_dst, (size_t)numel, is_half ? HQ_DTYPE_F16 : HQ_DTYPE_BF16,
                                nullptr);
    if (st != 0 && status == 0) status = st;
  }
  cudaDeviceSynchronize();
  const auto end = std::chrono::high_resolution_clock::now();
  const double time =
      std::chrono::duration_cast<std::chrono::microseconds>(end - start).count() / niters / 1.0e6;
  const double size = 2.0 * sizeof(T) * numel / 1.0e9;
  printf("size(GB):%.2f, average time(sec):%f, Bandwidth (GB/sec):%f\n", size, time, size / time);
  if (status != 0) printf("libhq status %d: %s\n", status, hq_status_string(status));

  cudaMemcpy(dst.data(), d_dst, bytes, cudaMemcpyDeviceToHost);
  verify(src.data(), dst.data(), numel);
  cudaFree(d_src);
  cudaFree(d_dst);
}

int main(int argc, char* argv[]) {
  if (argc != 3) {
    printf("Usage: %s <number of elements> <repeat>\n", argv[0]);
    return 1;
  }
  const int numel = atoi(argv[1]);
  const int niters = atoi(argv[2]);
  section<__half>(numel, niters);
  section<__nv_bfloat16>(numel, niters);
  return 0;
}
