// Driver with the command line and output of HeCBench's quantBnB benchmark
// (src/quantBnB-cuda/main.cu:132-193) on top of libhq.so.
//
// In the reference the kernel is defined inside the driver's translation unit,
// so a link-time swap is impossible; this driver keeps its argv
// (<number of elements> <repeat>), its input stream (mt19937{19937},
// normal_distribution<float>(0,1)), its host check and its two output lines,
// and replaces only the launch `kQuantize<256,256><<<grid,block>>>(...)`
// (reference main.cu:176) by hq_bnb_quantize_u8.  The 256-entry code table is
// the reference's code.h, taken from the include path at build time.  The host
// check below restates dQuantize<0> (reference main.cu:13-66).
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>
#include <cuda_runtime.h>

#include "code.h"
#include "hq.h"

static uint8_t quantize_host(const float* tab, float x) {
  int pivot = 127, upper_pivot = 255, lower_pivot = 0;
  float lower = -1.0f, upper = 1.0f, val = tab[pivot];
  for (int i = 64; i > 0; i >>= 1) {
    if (x > val) { lower_pivot = pivot; lower = val; pivot += i; }
    else { upper_pivot = pivot; upper = val; pivot -= i; }
    val = tab[pivot];
  }
  if (upper_pivot == 255) upper = tab[upper_pivot];
  if (lower_pivot == 0) lower = tab[lower_pivot];
  if (x > val) return (uint8_t)(x > (upper + val) * 0.5f ? upper_pivot : pivot);
  return (uint8_t)(x < (lower + val) * 0.5f ? lower_pivot : pivot);
}

int main(int argc, char* argv[]) {
  if (argc != 3) {
    printf("Usage: %s <number of elements> <repeat>\n", argv[0]);
    return 1;
  }
  const size_t n = atol(argv[1]);
  const int repeat = atoi(argv[2]);

  std::vector<float> A(n);
  std::vector<uint8_t> out(n), ref(n);
  std::mt19937 gen{19937};
  std::normal_distribution<float> d{0.f, 1.f};
  for (size_t i = 0; i < n; i++) {
    A[i] = d(gen);
    ref[i] = quantize_host(code, A[i]);
  }

  float *d_A, *d_code;
  uint8_t* d_out;
  cudaMalloc((void**)&d_A, n * sizeof(float));
  cudaMemcpy(d_A, A.data(), n * sizeof(float), cudaMemcpyHostToDevice);
  cudaMalloc((void**)&d_code, 256 * sizeof(float));
  cudaMemcpy(d_code, code, 256 * sizeof(float), cudaMemcpyHostToDevice);
  cudaMalloc((void**)&d_out, n);

  const int block_size = 256;
  cudaDeviceSynchronize();
  auto start = std::chrono::steady_clock::now();
  int status = HQ_OK;
  for (int i = 0; i < repeat; i++) {
    const int s = hq_bnb_quantize_u8(d_code, d_A, d_out, n, nullptr);
    if (s != HQ_OK) status = s;
  }
  cudaDeviceSynchronize();
  auto end = std::chrono::steady_clock::now();
  auto time = std::chrono::duration_cast<std::chrono::nanoseconds>(end - start).count();
  printf("Average execution time of kQuantize kernel with block size %d: %f (us)\n", block_size,
         (time * 1e-3f) / repeat);
  if (status != HQ_OK) printf("hq_bnb_quantize_u8: %s\n", hq_status_string(status));

  cudaMemcpy(out.data(), d_out, n, cudaMemcpyDeviceToHost);
  printf("%s\n", out == ref ? "PASS" : "FAIL");

  cudaFree(d_A);
  cudaFree(d_code);
  cudaFree(d_out);
  return 0;
}
