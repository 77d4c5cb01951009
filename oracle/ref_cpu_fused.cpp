// Builds the reference's own HOST checks of the three operators that the fused
// mat-vec entry points wrap around the product - rmsnorm-cuda/reference.h
// (rmsnorm_forward_cpu), geglu-cuda/reference.h (geglu_reference) and
// swish-cuda/reference.h (reference) - into oracle/_ref/libref_cpu.so.
// TEST INFRASTRUCTURE ONLY.
//
// The headers are included from where they lie in the HeCBench tree (the build
// passes -I<reference>/src); nothing of them is copied.  Compiled by g++ as
// host code.
#include <cmath>
#include <cstdint>
#include <vector>

#include "rmsnorm-cuda/reference.h"
#include "geglu-cuda/reference.h"
#include "swish-cuda/reference.h"

extern "C" {

// out[tokens][hidden] = RMSNorm(inp) * gamma, fp32, eps = 1e-5 (fixed by the reference)
void ref_rmsnorm_f32(float* out, const float* inp, const float* gamma, int64_t tokens,
                     int64_t hidden) {
  rmsnorm_forward_cpu(out, inp, gamma, tokens, hidden);
}

// out[n][dim_last] from x_and_gate[n][2][dim_last]: value * gelu(gate), fp32
void ref_geglu_f32(float* out, const float* x_and_gate, int n, int dim_last) {
  geglu_reference<float>(out, x_and_gate, n, dim_last);
}

// y[i] = x[i] / (1 + exp(-x[i])): the forward half of the reference's check
void ref_swish_f32(const float* x, float* y, int n) {
  std::vector<float> dx(n), dy(n, 0.f);
  reference<float>(n, const_cast<float*>(x), y, dx.data(), dy.data());
}

}  // extern "C"
