// Drop-in replacement for HeCBench's src/gemv-cuda/gemv.cu.
//
// The reference driver (main.cu:85-99) parses the command line and calls
// test_gemv_int8_quantized_with_params / test_gemv_int4_quantized_with_params
// (and, commented out there, test_gemv_with_params), which gemv.cu defines
// together with the launchers and the device-side checks.  This file defines
// the same three functions on top of libhq.so: compile it in place of the
// reference gemv.cu with the reference's kernels.h (for the uint4_2 type) and
// simple_tensor.h on the include path, keep the reference main.cu, link -lhq.
// Same inputs (SimpleTensor::reset), same printed lines; block_dim_x /
// block_dim_y are accepted and ignored (they tune the reference kernels).
//
// The checks restate gemv.cu:83-141: one thread per output row recomputes the
// row in fp32 from the dequantised weights and reports every element that is
// further than 0.125 * n / 512 from the result.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>

#include "hq.h"
#include "kernels.h"
#include "simple_tensor.h"

namespace {

// bits: 16 fp16 matrix, 8 int8, 4 two codes per byte (element 2j in the low nibble)
__global__ void check_rows(const void* mat, const __half* vec, const __half* res, int n, int bits,
                           __half scale_h, __half zero_h, int* bad) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  const float scale = __half2float(scale_h), zp = __half2float(zero_h);
  float sum = 0.f;
  for (int j = 0; j < n; j++) {
    float w;
    if (bits == 16) {
      w = __half2float(reinterpret_cast<const __half*>(mat)[(size_t)row * n + j]);
    } else if (bits == 8) {
      w = ((float)reinterpret_cast<const int8_t*>(mat)[(size_t)row * n + j] - zp) * scale;
    } else {
      const unsigned char b = reinterpret_cast<const unsigned char*>(mat)[(size_t)row * (n / 2) + j / 2];
      w = ((float)((j & 1) ? (b >> 4) : (b & 15)) - zp) * scale;
    }
    sum += w * __half2float(vec[j]);
  }
  const float got = __half2float(res[row]);
  const float diff = sum - got, delta = 0.125f * n / 512;
  if (diff > delta || diff < -delta) {
    printf("!!![idx=%d] %f != %f, diff=%f\n", row, got, sum, diff);
    atomicAdd(bad, 1);
  }
}

template <typename Launch>
void timed(unsigned repeat, Launch launch) {
  cudaDeviceSynchronize();
  const auto start = std::chrono::steady_clock::now();
  for (unsigned i = 0; i < repeat; ++i) {
    const int st = launch();
    if (st != HQ_OK) {
      std::fprintf(stderr, "gemv: %s (status %d)\n", hq_status_string(st), st);
      break;
    }
  }
  cudaDeviceSynchronize();
  const auto end = std::chrono::steady_clock::now();
  const auto ns = std::chrono::duration_cast<std::chrono::nanoseconds>(end - start).count();
  printf("Average kernel execution time: %f (us)\n", (ns * 1e-3f) / repeat);
}

void check(const void* mat, const __half* vec, const __half* res, unsigned size, int bits,
           float scale, float zero_point) {
  printf("Check correctness on the device\n");
  int* bad = nullptr;
  cudaMalloc(&bad, sizeof(int));
  cudaMemset(bad, 0, sizeof(int));
  check_rows<<<(size + 255) / 256, 256>>>(mat, vec, res, (int)size, bits, __float2half(scale),
                                          __float2half(zero_point), bad);
  cudaDeviceSynchronize();
  cudaFree(bad);
}

}  // namespace

void test_gemv_with_params(unsigned int size, unsigned int repeat, unsigned int, unsigned int) {
  SimpleTensor<__half> mat(size, size);
  SimpleTensor<__half> vec(size, 1);
  mat.reset();
  vec.reset();
  printf("GEMV FP16 ..\n");
  SimpleTensor<__half> res(size, 1);
  timed(repeat, [&] {
    return hq_gemv_f16(mat.device_data(), vec.device_data(), res.device_data(), (int)size,
                       (int)size, nullptr);
  });
  check(mat.device_data(), vec.device_data(), res.device_data(), size, 16, 1.f, 0.f);
}

void test_gemv_int8_quantized_with_params(unsigned int size, unsigned int repeat, unsigned int,
                                          unsigned int, float scale, float zero_point) {
  SimpleTensor<int8_t> mat(size, size);
  SimpleTensor<__half> vec(size, 1);
  mat.reset();
  vec.reset();
  printf("GEMV int8 quantized...\n");
  SimpleTensor<__half> res(size, 1);
  timed(repeat, [&] {
    return hq_gemv_int8_f16(mat.device_data(), vec.device_data(), res.device_data(), (int)size,
                            (int)size, scale, zero_point, nullptr);
  });
  check(mat.device_data(), vec.device_data(), res.device_data(), size, 8, scale, zero_point);
}

void test_gemv_int4_quantized_with_params(unsigned int size, unsigned int repeat, unsigned int,
                                          unsigned int, float scale, float zero_point) {
  SimpleTensor<uint4_2> mat(size, size / 2);
  SimpleTensor<__half> vec(size, 1);
  mat.reset();
  vec.reset();
  printf("GEMV int4 quantized...\n");
  SimpleTensor<__half> res(size, 1);
  timed(repeat, [&] {
    return hq_gemv_int4_f16(reinterpret_cast<const uint8_t*>(mat.device_data()), vec.device_data(),
                            res.device_data(), (int)size, (int)size, scale, zero_point, nullptr);
  });
  check(mat.device_data(), vec.device_data(), res.device_data(), size, 4, scale, zero_point);
}
