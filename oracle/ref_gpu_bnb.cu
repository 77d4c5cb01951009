// Reference kQuantize kernel built from its own source (quantBnB-cuda/main.cu,
// included from the reference tree with main() renamed).  TEST INFRASTRUCTURE ONLY.
#define main hecbench_quantbnb_cuda_main
#include "main.cu"
#undef main

extern "C" void ref_bnb_quantize_gpu(const float* d_code, const float* d_A, uint8_t* d_out, int n) {
  const int block_size = 256;  // launch of quantBnB-cuda/main.cu:168-176
  dim3 grid((n + block_size - 1) / block_size);
  dim3 block(block_size);
  kQuantize<block_size, block_size><<<grid, block>>>(d_code, d_A, d_out, n);
}
