// Builds the reference's own HOST check of the zero-point computation
// (zeropoint-cuda/reference.h) into oracle/_ref/libref_cpu.so.
// TEST INFRASTRUCTURE ONLY.
//
// The header is included from where it lies in the HeCBench tree (the build
// passes -I<reference>/src/zeropoint-cuda) after the headers the reference
// driver includes before it (main.cu:1-8); nothing of it is copied.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <cstdint>

#include "reference.h"

extern "C" void ref_zero_point(const float* x_min, const float* x_max, int32_t qmin, int32_t qmax,
                               int size, int preserve_sparsity, float* scale,
                               int32_t* zero_point) {
  reference(x_min, x_max, qmin, qmax, size, preserve_sparsity != 0, scale, zero_point);
}
