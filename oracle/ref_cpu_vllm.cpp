// Builds the reference's own HOST implementation of the per-token int8
// activation quantization (quantVLLM-cuda/reference.h with the helpers of
// utils.h) into oracle/_ref/libref_cpu.so.  TEST INFRASTRUCTURE ONLY.
//
// Both headers are included from where they lie in the HeCBench tree (the
// build passes -I<reference>/src/quantVLLM-cuda); nothing of them is copied.
// The CUDA headers only provide the __half / __nv_bfloat16 types and the
// __host__ __device__ markers; this file is compiled by g++ as host code.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>

#include "utils.h"
#include "reference.h"

namespace {
template <typename T>
void run_static(const void* in, int8_t* out, float scale, int32_t azp, int64_t tokens, int hidden) {
  // the launcher's choice of form, quantVLLM-cuda/main.cu:147-152
  if (!azp)
    static_scaled_int8_quant_reference(static_cast<const T*>(in), out, scale, tokens, hidden);
  else
    static_scaled_int8_azp_quant_reference(static_cast<const T*>(in), out, scale, azp, tokens,
                                           hidden);
}
template <typename T>
void run_dynamic(const void* in, int8_t* out, float* scale, int32_t* azp, int64_t tokens,
                 int hidden) {
  // quantVLLM-cuda/main.cu:165-171
  if (azp == nullptr)
    dynamic_scaled_int8_quant_reference(static_cast<const T*>(in), out, scale, tokens, hidden);
  else
    dynamic_scaled_int8_azp_quant_reference(static_cast<const T*>(in), out, scale, azp, tokens,
                                            hidden);
}
}  // namespace

extern "C" {
// dtype: 0 = fp16, 1 = bf16, 2 = fp32
void ref_vllm_static_quant(const void* in, int dtype, int8_t* out, float scale, int32_t azp,
                           long long tokens, int hidden) {
  if (dtype == 0) run_static<__half>(in, out, scale, azp, tokens, hidden);
  else if (dtype == 1) run_static<__nv_bfloat16>(in, out, scale, azp, tokens, hidden);
  else run_static<float>(in, out, scale, azp, tokens, hidden);
}
void ref_vllm_dynamic_quant(const void* in, int dtype, int8_t* out, float* scale, int32_t* azp,
                            long long tokens, int hidden) {
  if (dtype == 0) run_dynamic<__half>(in, out, scale, azp, tokens, hidden);
  else if (dtype == 1) run_dynamic<__nv_bfloat16>(in, out, scale, azp, tokens, hidden);
  else run_dynamic<float>(in, out, scale, azp, tokens, hidden);
}
}
