// Driver with the command line and output of HeCBench's quantVLLM benchmark
// (src/quantVLLM-cuda/main.cu:174-298) on top of libhq.so.
//
// In the reference the four kernels and their two launchers are defined inside
// the driver's translation unit, so a link-time swap is impossible; this
// driver keeps its argv (<number of tokens> <hidden size> <repeat>), its input
// stream (srand(123); rand() % 1000 - 300), its four timed sections, its
// memcmp against the host reference and its output lines, and replaces only
// the launchers static_scaled_int8_quant / dynamic_scaled_int8_quant
// (reference main.cu:137-172) by the C ABI.  The host reference is the
// reference's own reference.h / utils.h, taken from the include path at build
// time.
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "utils.h"
#include "reference.h"
#include "hq.h"

template <typename T> struct DType;
template <> struct DType<__half> { static constexpr int id = HQ_DTYPE_F16; };
template <> struct DType<__nv_bfloat16> { static constexpr int id = HQ_DTYPE_BF16; };
template <> struct DType<float> { static constexpr int id = HQ_DTYPE_F32; };

static int g_status = 0;
static void note(int st) {
  if (st != 0 && g_status == 0) {
    g_status = st;
    printf("libhq status %d: %s\n", st, hq_status_string(st));
  }
}

template <typename scalar_t>
void static_scaled_int8_quant(int8_t* output, const scalar_t* input, int hidden_size,
                              int num_tokens, float scale, int32_t azp) {
  note(hq_vllm_static_scaled_int8_quant(output, input, DType<scalar_t>::id, hidden_size,
                                        num_tokens, scale, azp, nullptr));
}

template <typename scalar_t>
void dynamic_scaled_int8_quant(int8_t* output, const scalar_t* input, int hidden_size,
                               int num_tokens, float* scales, int32_t* azp) {
  note(hq_vllm_dynamic_scaled_int8_quant(output, input, DType<scalar_t>::id, hidden_size,
                                         num_tokens, scales, azp, nullptr));
}

template <typename F>
static void timed(const char* what, int repeat, F&& launch) {
  auto start = std::chrono::steady_clock::now();
  for (int i = 0; i < repeat; i++) launch();
  cudaDeviceSynchronize();
  auto end = std::chrono::steady_clock::now();
  auto time = std::chrono::duration_cast<std::chrono::nanoseconds>(end - start).count();
  printf("Average execution time of %s kernel: %f (us)\n", what, (time * 1e-3f) / repeat);
}

template <typename scalar_t>
void quant(int num_tokens, int hidden_size, int repeat) {
  const size_t n = (size_t)hidden_size * num_tokens;
  std::vector<scalar_t> h_input(n);
  std::vector<float> h_scale(num_tokens);
  std::vector<int32_t> h_azp(num_tokens);
  std::vector<int8_t> h_output(n), h_output_r(n);
  srand(123);
  for (size_t i = 0; i < n; i++) h_input[i] = rand() % 1000 - 300;

  scalar_t* d_input;
  float* d_scale;
  int32_t* d_azp = nullptr;
  int8_t* d_output;
  cudaMalloc(&d_input, n * sizeof(scalar_t));
  cudaMalloc(&d_output, n);
  cudaMalloc(&d_scale, num_tokens * sizeof(float));
  cudaMemcpy(d_input, h_input.data(), n * sizeof(scalar_t), cudaMemcpyHostToDevice);

  const float scale = 0.1;
  int32_t error = 0;
  auto fetch = [&] { cudaMemcpy(h_output.data(), d_output, n, cudaMemcpyDeviceToHost); };

  int32_t azp = 0;
  timed("static_scaled_int8_quant", repeat, [&] {
    static_scaled_int8_quant(d_output, d_input, hidden_size, num_tokens, scale, azp);
  });
  fetch();
  static_scaled_int8_quant_reference(h_input.data(), h_output_r.data(), scale, num_tokens,
                                     hidden_size);
  error = memcmp(h_output.data(), h_output_r.data(), n);

  azp = 54;
  timed("static_scaled_int8_quant_azp", repeat, [&] {
    static_scaled_int8_quant(d_output, d_input, hidden_size, num_tokens, scale, azp);
  });
  fetch();
  static_scaled_int8_azp_quant_reference(h_input.data(), h_output_r.data(), scale, azp, num_tokens,
                                         hidden_size);
  error += memcmp(h_output.data(), h_output_r.data(), n) != 0;

  timed("dynamic_scaled_int8_quant", repeat, [&] {
    dynamic_scaled_int8_quant(d_output, d_input, hidden_size, num_tokens, d_scale, d_azp);
  });
  fetch();
  dynamic_scaled_int8_quant_reference(h_input.data(), h_output_r.data(), h_scale.data(),
                                      num_tokens, hidden_size);
  error += memcmp(h_output.data(), h_output_r.data(), n) != 0;

  cudaMalloc(&d_azp, num_tokens * sizeof(int32_t));
  timed("dynamic_scaled_int8_quant_azp", repeat, [&] {
    dynamic_scaled_int8_quant(d_output, d_input, hidden_size, num_tokens, d_scale, d_azp);
  });
  fetch();
  dynamic_scaled_int8_azp_quant_reference(h_input.data(), h_output_r.data(), h_scale.data(),
                                          h_azp.data(), num_tokens, hidden_size);
  error += memcmp(h_output.data(), h_output_r.data(), n) != 0;

  printf("%s\n", (error || g_status) ? "FAIL" : "PASS");
  cudaFree(d_input);
  cudaFree(d_output);
  cudaFree(d_scale);
  cudaFree(d_azp);
}

int main(int argc, char* argv[]) {
  if (argc != 4) {
    printf("Usage: %s <number of tokens> <hidden size> <repeat>\n", argv[0]);
    return 1;
  }
  const int num_tokens = atoi(argv[1]);
  const int hidden_size = atoi(argv[2]);
  const int repeat = atoi(argv[3]);

  printf("Input type is FP16\n");
  quant<__half>(num_tokens, hidden_size, repeat);

  printf("Input type is BF16\n");
  quant<__nv_bfloat16>(num_tokens, hidden_size, repeat);

  printf("Input type is FP32\n");
  quant<float>(num_tokens, hidden_size, repeat);
  return g_status ? 1 : 0;
}
