// Drop-in replacement for HeCBench's src/lut-gemm-cuda/kernels.cu.
//
// Defines the two matmul overloads declared in the reference's kernels.h:24-25
// on top of libhq.so.  Compile it in place of the reference kernels.cu, with
// the reference's kernels.h / nQWeight_fp16.h on the include path, and link
// with -lhq.  Like the reference (kernels.cu:22-31) the call overwrites
// output[0 .. mSize), is asynchronous on the default stream, and computes one
// input row (the reference ignores its m / n argument as well).
//
// The kernel accumulates K tiles in an fp32 scratch row.  matmul() has no
// workspace argument, so the shim keeps one zero-initialised scratch buffer per
// device, grown on demand (allocation happens only on the first call or when a
// larger mSize appears).
#include <cuda_runtime.h>
#include <cstdio>
#include <mutex>

#include "hq.h"
#include "kernels.h"

namespace {

struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
};
Scratch g_scratch[64];
std::mutex g_mu;

void* scratch_for(int M, size_t* bytes_out) {
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t need = hq_lutgemm_workspace_bytes(M);
  std::lock_guard<std::mutex> lock(g_mu);
  Scratch& s = g_scratch[dev & 63];
  if (s.bytes < need) {
    if (s.ptr) {
      cudaDeviceSynchronize();
      cudaFree(s.ptr);
    }
    s.ptr = nullptr;
    s.bytes = 0;
    if (cudaMalloc(&s.ptr, need) != cudaSuccess) return nullptr;
    cudaMemset(s.ptr, 0, need);
    s.bytes = need;
  }
  *bytes_out = s.bytes;
  return s.ptr;
}

void run(void* output, void* input, nQWeight_fp16& nqW) {
  size_t bytes = 0;
  void* ws = scratch_for(nqW.mSize, &bytes);
  // the reference launcher derives the group size the same way (mv_fp16.h:235)
  const int group_size = nqW.kSize / nqW.num_groups;
  const int st = hq_lutgemm_nqmv(output, input, nqW.bWeight, nqW.alpha, nqW.q_bias, nqW.mSize,
                                 nqW.kSize, nqW.nb, group_size, ws, bytes, nullptr);
  if (st != HQ_OK) std::fprintf(stderr, "matmul: %s (status %d)\n", hq_status_string(st), st);
}

}  // namespace

void matmul(void* output, nQWeight_fp16& nqW, void* input, int n, int algo) {
  (void)n; (void)algo;
  run(output, input, nqW);
}

void matmul(void* output, void* input, nQWeight_fp16& nqW, int m, int algo) {
  (void)m; (void)algo;
  run(output, input, nqW);
}
