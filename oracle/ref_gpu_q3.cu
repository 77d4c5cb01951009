// Reference GPU kernels of quant3MatMul built from their own source for the
// on-GPU parity pin (oracle/_ref/libref_gpu.so).  TEST INFRASTRUCTURE ONLY;
// the header is included from the reference tree (-I<reference>/src/quant3MatMul-cuda).
#include "kernels.h"

extern "C" {
void ref_q3_gemv_f32(float* vec, int* mat, float* mul, float* scales, float* zeros, int height,
                     int width) {
  vecquant3matmul<float>(vec, mat, mul, scales, zeros, height, width);
}
void ref_q3_gemv_faster(void* vec_half, int* mat, float* mul, float* scales, float* zeros,
                        int height, int width) {
  vecquant3matmul_faster((half*)vec_half, mat, mul, scales, zeros, height, width);
}
}
