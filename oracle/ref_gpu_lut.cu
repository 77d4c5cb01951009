// Reference LUT-GEMM kernels built from their own headers (lut-gemm-cuda,
// included from the reference tree).  TEST INFRASTRUCTURE ONLY.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "nQWeight_fp16.h"
#include "mv_fp16.h"

// The class is only declared in the header; its out-of-line members live in the
// reference's nQWeight_fp16.cu, which allocates managed memory.  Here the
// object only borrows caller-owned device pointers, so the destructor must not
// free them.
nQWeight_fp16::~nQWeight_fp16() {}
void nQWeight_fp16::parsing(unsigned int*, float*, int, int, int, bool, int, float*) {}

extern "C" void ref_lutgemm_matmul(void* output, void* input, unsigned int* bW, void* alpha,
                                   void* q_bias, int M, int K, int nb, int num_groups) {
  nQWeight_fp16* w = new nQWeight_fp16();
  w->bWeight = bW;
  w->alpha = alpha;
  w->q_bias = q_bias;
  w->num_groups = num_groups;
  w->group_size = K / num_groups;
  w->mSize = M;
  w->kSize = K;
  w->nb = nb;
  w->is_row_wise_quantize = false;
  // body of matmul(), lut-gemm-cuda/kernels.cu:27-31
  cudaMemset(output, 0, sizeof(__half) * w->mSize);
  if (w->q_bias == nullptr) nqmv((__half*)output, *w, (__half*)input, 0);
  else nqmv_bias((__half*)output, *w, (__half*)input, 0);
  delete w;
}
