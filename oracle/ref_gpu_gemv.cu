// Reference GPU kernels of gemv built from their own source for the on-GPU
// parity pin (oracle/_ref/libref_gpu.so).  TEST INFRASTRUCTURE ONLY; the header
// is included from the reference tree (-I<reference>/src/gemv-cuda).  The
// launch shapes follow the reference launchers (gemv.cu:15-81): grid
// (1, rows / block_dim_y), block (block_dim_x, block_dim_y), num_per_thread =
// n / block_dim_x; the reference only runs square matrices.
#include "kernels.h"

extern "C" {
void ref_gemv_int8(int8_t* mat, void* vec_half, void* res_half, unsigned size, float scale_f,
                   float zero_point_f, unsigned bx, unsigned by) {
  gemv_quantized_int8<<<dim3(1, size / by), dim3(bx, by)>>>(
      mat, (__half*)vec_half, (__half*)res_half, size, __float2half(scale_f),
      __float2half(zero_point_f), size / bx);
}
void ref_gemv_int4(uint8_t* mat, void* vec_half, void* res_half, unsigned size, float scale_f,
                   float zero_point_f, unsigned bx, unsigned by) {
  gemv_quantized_int4<<<dim3(1, size / by), dim3(bx, by)>>>(
      (uint4_2*)mat, (__half*)vec_half, (__half*)res_half, size, __float2half(scale_f),
      __float2half(zero_point_f), size / bx);
}
void ref_gemv_f16(void* mat_half, void* vec_half, void* res_half, unsigned size, unsigned bx,
                  unsigned by) {
  gemv_fp16<<<dim3(1, size / by), dim3(bx, by)>>>((__half*)mat_half, (__half*)vec_half,
                                                   (__half*)res_half, size, size / bx);
}
}
