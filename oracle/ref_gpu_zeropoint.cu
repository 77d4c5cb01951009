// Reference GPU kernel of zeropoint built from its own source for the on-GPU
// parity pin (oracle/_ref/libref_gpu.so).  TEST INFRASTRUCTURE ONLY.  The kernel
// lives in the reference driver's main.cu, which is included from the reference
// tree (-I<reference>/src/zeropoint-cuda) with its main() renamed; nothing of it
// is copied.  Launch as in the driver (main.cu:131-147): blocks of 256 threads.
#define main hecbench_zeropoint_main
#include "main.cu"
#undef main

extern "C" int ref_zero_point_gpu(const float* x_min, const float* x_max, int32_t qmin,
                                  int32_t qmax, int size, int preserve_sparsity, float* scale,
                                  int32_t* zp) {
  zero_point<<<(size + 255) / 256, 256>>>(x_min, x_max, qmin, qmax, size, preserve_sparsity != 0,
                                          scale, zp);
  return (int)cudaGetLastError();
}
