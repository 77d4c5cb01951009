// Driver with the command line and output of HeCBench's zeropoint benchmark
// (src/zeropoint-cuda/main.cu:82-181) on top of libhq.so.
//
// In the reference the kernel is defined inside the driver's translation unit,
// so a link-time swap is impossible; this driver keeps its argv (<number of
// min/max values> <repeat>), its inputs (std::default_random_engine g(123),
// uniform in (-1, 1), minimum and maximum drawn alternately), its int8
// symmetric configuration, its timed loop, its comparison with the host
// reference and its output lines, and replaces only the kernel launch
// (reference main.cu:137-147) by hq_zero_point.  The host reference is the
// reference's own reference.h, taken from the include path at build time.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <random>
#include <vector>

#include <cuda_runtime.h>

#include "reference.h"
#include "hq.h"

int main(int argc, char* argv[]) {
  if (argc != 3) {
    printf("Usage: %s <number of min/max values> <repeat>\n", argv[0]);
    return 1;
  }
  const int size = atoi(argv[1]);
  const int repeat = atoi(argv[2]);
  const int32_t qmin = -127, qmax = 127;
  const bool preserve_sparsity = true;

  std::vector<float> lo(size), hi(size), scale(size), scale_ref(size);
  std::vector<int32_t> zp(size), zp_ref(size);
  std::default_random_engine g(123);
  std::uniform_real_distribution<float> distr(-1.f, 1.f);
  for (int i = 0; i < size; i++) {
    lo[i] = distr(g);
    hi[i] = distr(g);
  }
  reference(lo.data(), hi.data(), qmin, qmax, size, preserve_sparsity, scale_ref.data(),
            zp_ref.data());

  const size_t bytes = sizeof(float) * size;
  float *d_lo, *d_hi, *d_scale;
  int32_t* d_zp;
  cudaMalloc((void**)&d_lo, bytes);
  cudaMalloc((void**)&d_hi, bytes);
  cudaMalloc((void**)&d_scale, bytes);
  cudaMalloc((void**)&d_zp, bytes);
  cudaMemcpy(d_lo, lo.data(), bytes, cudaMemcpyHostToDevice);
  cudaMemcpy(d_hi, hi.data(), bytes, cudaMemcpyHostToDevice);

  int status = 0;
  cudaDeviceSynchronize();
  const auto start = std::chrono::steady_clock::now();
  for (int i = 0; i < repeat; i++) {
    const int st = hq_zero_point(d_lo, d_hi, qmin, qmax, size, preserve_sparsity, d_scale, d_zp, nullptr);
    if (st != 0 && status == 0) status = st;
  }
  cudaDeviceSynchronize();
  const auto end = std::chrono::steady_clock::now();
  const auto time = std::chrono::duration_cast<std::chrono::nanoseconds>(end - start).count();
  printf("Average execution time of zero-point kernel: %f (us)\n", (time * 1e-3f) / repeat);
  if (status != 0) printf("libhq status %d: %s\n", status, hq_status_string(status));

  cudaMemcpy(zp.data(), d_zp, bytes, cudaMemcpyDeviceToHost);
  cudaMemcpy(scale.data(), d_scale, bytes, cudaMemcpyDeviceToHost);
  bool ok = status == 0;
  for (int i = 0; i < size && ok; i++)
    if (zp[i] != zp_ref[i] || scale[i] - scale_ref[i] > 1e-3f) ok = false;  // the reference's test
  printf("%s\n", ok ? "PASS" : "FAIL");

  cudaFree(d_zp);
  cudaFree(d_scale);
  cudaFree(d_lo);
  cudaFree(d_hi);
  return 0;
}
