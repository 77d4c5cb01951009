// Driver with the shapes and output of HeCBench's quantAQLM benchmark
// (src/quantAQLM-cuda/main.cu:143-242) on top of libhq.so.
//
// The reference defines kernel and launcher inside the driver, so this is a
// replacement driver: same problem (4 input vectors of 4096 halves, codes
// 12288 x 512 int16 from srand(123), 3 stacked 65536 x 8 codebooks, the ramp
// initialisers of main.cu:183-191), same launcher name and signature
// (code1x16_matvec, main.cu:113-117, including its per-call timing line), and
// one change of sizing: each of the 4 calls gets its own prob_m output halves
// (the reference allocates b*12288/32 halves in total and offsets the calls by
// 384, main.cu:151,215, while each call stores prob_m halves).
// It adds what the reference lacks: a host check of every output.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "hq.h"

void code1x16_matvec(const void* A, const void* B, void* C, const void* codebook, int prob_m,
                     int prob_k, const int4 codebook_a_sizes, const int codebook_stride) {
  const int sizes[4] = {codebook_a_sizes.x, codebook_a_sizes.y, codebook_a_sizes.z,
                        codebook_a_sizes.w};
  cudaDeviceSynchronize();
  auto start = std::chrono::steady_clock::now();
  const int st = hq_aqlm_1x16_matvec(A, B, C, codebook, prob_m, prob_k, sizes, codebook_stride,
                                     nullptr, nullptr);
  cudaDeviceSynchronize();
  auto end = std::chrono::steady_clock::now();
  auto time = std::chrono::duration_cast<std::chrono::nanoseconds>(end - start).count();
  printf("kernel execution time: %f (us)\n", (time * 1e-3f) / 1);
  if (st != HQ_OK) printf("hq_aqlm_1x16_matvec: %s\n", hq_status_string(st));
}

int main() {
  const int b = 4;
  const int prob_m = 12288, prob_k = 4096;
  const size_t input_size = (size_t)b * prob_k;
  const size_t output_size = (size_t)b * prob_m;
  const size_t code_size = (size_t)prob_m * (prob_k / 8);
  const size_t entries = 65536;
  const size_t codebook_size = 3 * entries * 8;
  const int4 codebook_a_sizes = make_int4(4096, 8192, 12288, 122880);
  const int codebook_stride = entries * 8 * sizeof(__half) / sizeof(int4);

  std::vector<__half> h_input(input_size), h_output(output_size), h_codebook(codebook_size);
  std::vector<short> h_codes(code_size);
  srand(123);
  for (size_t i = 0; i < input_size; i++) h_input[i] = (float)i / input_size;
  for (size_t i = 0; i < code_size; i++) h_codes[i] = rand() % 65536 - 32768;
  for (size_t i = 0; i < codebook_size; i++) h_codebook[i] = (float)i / codebook_size;

  __half *d_input, *d_output, *d_codebook;
  short* d_codes;
  cudaMalloc(&d_input, input_size * sizeof(__half));
  cudaMalloc(&d_output, output_size * sizeof(__half));
  cudaMalloc(&d_codes, code_size * sizeof(short));
  cudaMalloc(&d_codebook, codebook_size * sizeof(__half));
  cudaMemcpy(d_input, h_input.data(), input_size * sizeof(__half), cudaMemcpyHostToDevice);
  cudaMemcpy(d_codes, h_codes.data(), code_size * sizeof(short), cudaMemcpyHostToDevice);
  cudaMemcpy(d_codebook, h_codebook.data(), codebook_size * sizeof(__half),
             cudaMemcpyHostToDevice);

  for (int i = 0; i < b; ++i)
    code1x16_matvec((void*)d_codes, (void*)(d_input + (size_t)prob_k * i),
                    (void*)(d_output + (size_t)prob_m * i), (void*)d_codebook, prob_m, prob_k,
                    codebook_a_sizes, codebook_stride);
  cudaMemcpy(h_output.data(), d_output, output_size * sizeof(__half), cudaMemcpyDeviceToHost);

  // host check: fp64 dot products of the fp16 operands; the kernel accumulates
  // eight-term fp16 partial sums, so allow 1e-2 of the largest output
  double worst = 0.0, scale = 0.0;
  for (int v = 0; v < b; v++)
    for (int m = 0; m < prob_m; m += 97) {
      const __half* cb = h_codebook.data() + (size_t)(m / 4096) * entries * 8;
      double acc = 0.0;
      for (int g = 0; g < prob_k / 8; g++) {
        const unsigned short c = (unsigned short)h_codes[(size_t)m * (prob_k / 8) + g];
        for (int j = 0; j < 8; j++)
          acc += (double)__half2float(cb[(size_t)c * 8 + j]) *
                 (double)__half2float(h_input[(size_t)v * prob_k + 8 * g + j]);
      }
      const double got = (double)__half2float(h_output[(size_t)v * prob_m + m]);
      worst = std::fmax(worst, std::fabs(got - acc));
      scale = std::fmax(scale, std::fabs(acc));
    }
  printf("%s\n", worst <= 1e-2 * scale ? "PASS" : "FAIL");

  cudaFree(d_input);
  cudaFree(d_output);
  cudaFree(d_codes);
  cudaFree(d_codebook);
  return 0;
}
