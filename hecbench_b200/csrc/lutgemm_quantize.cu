// Greedy binary-coding quantizer for sm_100a: fp16 / bf16 / fp32 weights W[K][M]
// -> the sign planes, scales and offsets that the LUT-GEMM mat-vec
// (hq_lutgemm_nqmv, the layouts of lut-gemm-cuda/main.cu:27-30,118-134) consumes.
// The reference tree holds only the consumer; the rule is the greedy
// binary-coding quantization the format comes from, per output column m and group
// g of group_size consecutive inputs, in fp32 with sums taken in ascending k:
//   q_bias[g][m] = half(mean of the group)                  (when offsets are asked for)
//   r = w - q_bias;  for b = 0 .. nb - 1:
//     alpha[g][b][m] = half(mean |r|);  bit = r >= 0;  r -= +-alpha (the rounded value)
// and bit t of bW[k / 32][b][m] is the bit of input k = 32 (k / 32) + t.
//
// Design: a CTA owns one group of 128 columns; the tile is read once with 128-bit
// loads into shared memory as fp32, then a thread owns a column and walks it
// 1 + 2 nb times (mean; per plane: mean magnitude, then signs and residual
// update in place), writing one 32-bit word of signs per 32 inputs: rows of 128
// consecutive words.
#include <cuda_bf16.h>

#include <algorithm>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kCols = 128;  // columns per CTA = threads per CTA

template <int DTYPE>
__global__ void __launch_bounds__(kCols)
bcq_quantize_kernel(const void* __restrict__ W, int K, int M, int nb, int gs,
                    uint32_t* __restrict__ bW, __half* __restrict__ alpha,
                    __half* __restrict__ q_bias) {
  extern __shared__ __align__(16) float tile[];  // [gs][kCols]
  const int tid = threadIdx.x;
  const int col0 = blockIdx.x * kCols, g = blockIdx.y;
  const size_t total = (size_t)K * M;
  (void)total;
  // ---- the tile: 8 columns per load (M % 8 == 0) ----
  for (int i = tid; i < gs * (kCols / 8); i += kCols) {
    const int k = i / (kCols / 8), c = (i % (kCols / 8)) * 8;
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; j++) w[j] = 0.f;
    if (col0 + c < M) {
      const size_t e = (size_t)(g * gs + k) * M + col0 + c;
      if (DTYPE == HQ_DTYPE_F32) {
        const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(W) + e);
        if (HQ_IN_BOUNDS(p, 32, W, total * 4, 1001)) {
          const uint4 a = ldg_stream_u4(p), b = ldg_stream_u4(p + 1);
          w[0] = __uint_as_float(a.x); w[1] = __uint_as_float(a.y);
          w[2] = __uint_as_float(a.z); w[3] = __uint_as_float(a.w);
          w[4] = __uint_as_float(b.x); w[5] = __uint_as_float(b.y);
          w[6] = __uint_as_float(b.z); w[7] = __uint_as_float(b.w);
        }
      } else {
        const unsigned short* p = reinterpret_cast<const unsigned short*>(W) + e;
        if (HQ_IN_BOUNDS(p, 16, W, total * 2, 1002)) {
          const uint4 a = ldg_stream_u4(p);
          const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            if (DTYPE == HQ_DTYPE_BF16) {
              w[2 * j] = __uint_as_float(u[j] << 16);
              w[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
            } else {
              const float2 f = __half22float2(u32_as_half2(u[j]));
              w[2 * j] = f.x;
              w[2 * j + 1] = f.y;
            }
          }
        }
      }
    }
    float4* dst = reinterpret_cast<float4*>(tile + k * kCols + c);
    dst[0] = make_float4(w[0], w[1], w[2], w[3]);
    dst[1] = make_float4(w[4], w[5], w[6], w[7]);
  }
  __syncthreads();
  const int m = col0 + tid;
  if (m >= M) return;
  float* r = tile + tid;  // this thread's column, stride kCols
  const float fgs = (float)gs;
  float bias = 0.f;
  if (q_bias != nullptr) {
    float s = 0.f;
    for (int k = 0; k < gs; k++) s += r[k * kCols];
    const __half bh = __float2half_rn(s / fgs);
    bias = __half2float(bh);
    if (HQ_IN_BOUNDS(q_bias + (size_t)g * M + m, 2, q_bias, (size_t)(K / gs) * M * 2, 1003))
      q_bias[(size_t)g * M + m] = bh;
  }
  for (int b = 0; b < nb; b++) {
    float s = 0.f;
    for (int k = 0; k < gs; k++) s += fabsf(r[k * kCols] - bias);
    const __half ah = __float2half_rn(s / fgs);
    const float a = __half2float(ah);
    const size_t ai = ((size_t)g * nb + b) * M + m;
    if (HQ_IN_BOUNDS(alpha + ai, 2, alpha, (size_t)(K / gs) * nb * M * 2, 1004)) alpha[ai] = ah;
    for (int k0 = 0; k0 < gs; k0 += 32) {
      uint32_t word = 0;
#pragma unroll 8
      for (int t = 0; t < 32; t++) {
        const float v = r[(k0 + t) * kCols] - bias;
        const bool up = v >= 0.f;
        word |= (up ? 1u : 0u) << t;
        r[(k0 + t) * kCols] = v - (up ? a : -a);
      }
      const size_t wi = ((size_t)((g * gs + k0) >> 5) * nb + b) * M + m;
      if (HQ_IN_BOUNDS(bW + wi, 4, bW, (size_t)(K / 32) * nb * M * 4, 1005)) bW[wi] = word;
    }
    bias = 0.f;  // taken out of the residual during the first plane
  }
}

template <int DTYPE>
int run(const void* W, int K, int M, int nb, int gs, uint32_t* bW, void* alpha, void* q_bias,
        cudaStream_t st) {
  const size_t smem = (size_t)gs * kCols * sizeof(float);
  if (smem > 227 * 1024) return HQ_ERR_UNSUPPORTED;
  constexpr auto kern = bcq_quantize_kernel<DTYPE>;
  const cudaError_t e = ensure_dynamic_smem<kern>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  kern<<<dim3((M + kCols - 1) / kCols, K / gs), kCols, smem, st>>>(
      W, K, M, nb, gs, bW, reinterpret_cast<__half*>(alpha), reinterpret_cast<__half*>(q_bias));
  return launch_status();
}

}  // namespace
}  // namespace hq

extern "C" int hq_lutgemm_quantize(const void* W, int dtype, int K, int M, int nb, int group_size,
                                   uint32_t* bW, void* alpha_half, void* q_bias_half,
                                   hq_stream_t stream) {
  using namespace hq;
  if (K <= 0 || M <= 0 || nb < 1 || nb > 8 || group_size < 32 || group_size % 32 != 0 ||
      K % group_size != 0 || M % 8 != 0)
    return HQ_ERR_BAD_SHAPE;
  if (K / group_size > 65535) return HQ_ERR_TOO_LARGE;
  if (!W || !bW || !alpha_half) return HQ_ERR_NULL_POINTER;
  if (!aligned16(W) || !aligned4(bW)) return HQ_ERR_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HQ_DTYPE_F16: return run<HQ_DTYPE_F16>(W, K, M, nb, group_size, bW, alpha_half, q_bias_half, st);
    case HQ_DTYPE_BF16: return run<HQ_DTYPE_BF16>(W, K, M, nb, group_size, bW, alpha_half, q_bias_half, st);
    case HQ_DTYPE_F32: return run<HQ_DTYPE_F32>(W, K, M, nb, group_size, bW, alpha_half, q_bias_half, st);
    default: return HQ_ERR_UNSUPPORTED;
  }
}
