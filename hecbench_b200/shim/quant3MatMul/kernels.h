// Drop-in replacement for HeCBench's src/quant3MatMul-cuda/kernels.h.
//
// Presents the launchers the reference driver calls (main.cu:81,96,111,123):
//   template <typename scalar_t> void vecquant3matmul(scalar_t* vec, int* mat,
//       scalar_t* mul, scalar_t* scales, scalar_t* zeros, int height, int width)
//       (reference kernels.h:171-190)
//   void vecquant3matmul_faster(half* vec, int* mat, float* mul, float* scales,
//       float* zeros, int height, int width)        (reference kernels.h:193-217)
// with the same conventions - device pointers, default stream, asynchronous,
// accumulates into mul - and forwards them to libhq.so.  Link with -lhq.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdio>

#include "hq.h"

const int BLOCKWIDTH = 256;
const int BLOCKHEIGHT = 24;

inline void hq_shim_report(const char* what, int status) {
  if (status != HQ_OK)
    std::fprintf(stderr, "%s: %s (status %d)\n", what, hq_status_string(status), status);
}

template <typename scalar_t>
void vecquant3matmul(scalar_t* vec, int* mat, scalar_t* mul, scalar_t* scales, scalar_t* zeros,
                     int height, int width);

// The reference driver instantiates the template with float only
// (main.cu:25 `using scalar_t = float`).
template <>
inline void vecquant3matmul<float>(float* vec, int* mat, float* mul, float* scales, float* zeros,
                                   int height, int width) {
  hq_shim_report("vecquant3matmul",
                 hq_q3_gemv_f32(vec, mat, mul, scales, zeros, height, width, nullptr));
}

inline void vecquant3matmul_faster(half* vec, int* mat, float* mul, float* scales, float* zeros,
                                   int height, int width) {
  hq_shim_report("vecquant3matmul_faster",
                 hq_q3_gemv_f16in(vec, mat, mul, scales, zeros, height, width, nullptr));
}
