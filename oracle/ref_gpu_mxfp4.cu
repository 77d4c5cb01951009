// Reference GPU kernel of mxfp4 built from its own source for the on-GPU parity
// pin (oracle/_ref/libref_gpu.so).  TEST INFRASTRUCTURE ONLY.  The kernel lives
// in the reference driver's main.cu, which is included from the reference tree
// (-I<reference>/src/mxfp4-cuda) with its main() renamed; nothing of it is copied.
// The launch is that of the reference's mxfp4() (main.cu:152-166) without its
// timing loop and printout: blocks of 128 threads (64 when the element count is
// no multiple of 128), one element per thread.
#define main hecbench_mxfp4_main
#include "main.cu"
#undef main

extern "C" int ref_mxfp4_qdq(const void* in, void* out, int numel, int bf16) {
  const int block = numel % 128 == 0 ? 128 : 64;
  if (numel % block != 0) return -1;
  if (bf16)
    qdq_mxfp4_kernel<__nv_bfloat16, BFLOAT16_EXP_BITS, BFLOAT16_MANTISSA_BITS, BFLOAT16_EXP_BIAS,
                     BFLOAT16_VAL_TO_ADD, BFLOAT16_SIGN_EXPONENT_MASK>
        <<<numel / block, block>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out);
  else
    qdq_mxfp4_kernel<__half, FLOAT16_EXP_BITS, FLOAT16_MANTISSA_BITS, FLOAT16_EXP_BIAS,
                     FLOAT16_VAL_TO_ADD, FLOAT16_SIGN_EXPONENT_MASK>
        <<<numel / block, block>>>((const __half*)in, (__half*)out);
  return (int)cudaGetLastError();
}
