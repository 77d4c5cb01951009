// Greedy binary-coding quantizer for sm_100a: fp16 / bf16 / fp32 weights W[K][M]
// -> the sign planes, scales and offsets that the LUT-GEMM mat-vec
// (hq_lutgemm_nqmv, the layouts of lut-gemm-cuda/main.cu:27-30,118-134) consumes.
// The reference tree holds only the consumer; the rule is the greedy
// binary-coding quantization the format comes from, per output column m and group
// g of group_size consecutive inputs, in fp32:
//   q_bias[g][m] = half(mean of the group)                  (when offsets are asked for)
//   r = w - q_bias;  for b = 0 .. nb - 1:
//     alpha[g][b][m] = half(mean |r|);  bit = r >= 0;  r -= +-alpha (the rounded value)
// and bit t of bW[k / 32][b][m] is the bit of input k = 32 (k / 32) + t.  A sum
// over a group is formed as one sum per 32 consecutive inputs (ascending k),
// and those partial sums are added in ascending order.
//
// Design: the summation order is the kernel's shape.  A thread holds 32
// consecutive inputs of two adjacent columns in registers - exactly the inputs of
// one output word per column and plane - warp w of a CTA the w-th run of 32 inputs
// of the group, the lanes 64 adjacent columns (one 32-bit load per lane and row,
// 128 contiguous bytes per warp).  Per plane the warps exchange their partial
// sums through shared memory (one barrier), every thread adds them in order,
// takes the signs of its residuals, updates them in registers and stores its two
// words.  The weights are read once; nothing else touches memory.
#include <cuda_bf16.h>

#include <algorithm>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kColsPerCta = 64;   // two per lane
constexpr int kMaxRuns = 16;      // runs of 32 inputs per group = warps per CTA (group_size <= 512)

template <int DTYPE>
__global__ void __launch_bounds__(kMaxRuns * 32)
bcq_quantize_kernel(const void* __restrict__ W, int K, int M, int nb, int gs,
                    uint32_t* __restrict__ bW, __half* __restrict__ alpha,
                    __half* __restrict__ q_bias) {
  __shared__ float s_part[2][kMaxRuns][kColsPerCta];  // [parity][run][column]
  const int lane = threadIdx.x & 31, run = threadIdx.x >> 5, runs = gs >> 5;
  const int g = blockIdx.y;
  const int m = blockIdx.x * kColsPerCta + 2 * lane;  // this thread's first column
  const bool live = m < M;                            // M is even: both columns or none
  const int k0 = g * gs + run * 32;                   // this thread's first input
  const size_t total = (size_t)K * M;
  (void)total;
  float r[32][2];
#pragma unroll
  for (int t = 0; t < 32; t++) {
    r[t][0] = r[t][1] = 0.f;
    if (!live) continue;
    const size_t e = (size_t)(k0 + t) * M + m;
    if (DTYPE == HQ_DTYPE_F32) {
      const uint2* p = reinterpret_cast<const uint2*>(reinterpret_cast<const float*>(W) + e);
      if (HQ_IN_BOUNDS(p, 8, W, total * 4, 1001)) {
        const uint2 a = ldg_stream_u2(p);
        r[t][0] = __uint_as_float(a.x);
        r[t][1] = __uint_as_float(a.y);
      }
    } else {
      const unsigned short* p = reinterpret_cast<const unsigned short*>(W) + e;
      if (HQ_IN_BOUNDS(p, 4, W, total * 2, 1002)) {
        const uint32_t u = ldg_stream_u32(p);
        if (DTYPE == HQ_DTYPE_BF16) {
          r[t][0] = __uint_as_float(u << 16);
          r[t][1] = __uint_as_float(u & 0xffff0000u);
        } else {
          const float2 f = __half22float2(u32_as_half2(u));
          r[t][0] = f.x;
          r[t][1] = f.y;
        }
      }
    }
  }
  const float fgs = (float)gs;
  int parity = 0;
  // sum over the group of what every thread holds as its run's partial sum
  auto group_sum = [&](float p0, float p1, float& s0, float& s1) {
    s_part[parity][run][2 * lane] = p0;
    s_part[parity][run][2 * lane + 1] = p1;
    __syncthreads();
    s0 = s1 = 0.f;
    for (int w = 0; w < runs; w++) {
      s0 += s_part[parity][w][2 * lane];
      s1 += s_part[parity][w][2 * lane + 1];
    }
    parity ^= 1;  // the next exchange uses the other half: no second barrier
  };
  if (q_bias != nullptr) {
    float p0 = 0.f, p1 = 0.f, s0, s1;
#pragma unroll
    for (int t = 0; t < 32; t++) {
      p0 += r[t][0];
      p1 += r[t][1];
    }
    group_sum(p0, p1, s0, s1);
    const __half2 bh = __floats2half2_rn(s0 / fgs, s1 / fgs);
    const float2 bias = __half22float2(bh);
#pragma unroll
    for (int t = 0; t < 32; t++) {
      r[t][0] -= bias.x;
      r[t][1] -= bias.y;
    }
    if (live && run == 0 &&
        HQ_IN_BOUNDS(q_bias + (size_t)g * M + m, 4, q_bias, (size_t)(K / gs) * M * 2, 1003))
      *reinterpret_cast<__half2*>(q_bias + (size_t)g * M + m) = bh;
  }
  for (int b = 0; b < nb; b++) {
    float p0 = 0.f, p1 = 0.f, s0, s1;
#pragma unroll
    for (int t = 0; t < 32; t++) {
      p0 += fabsf(r[t][0]);
      p1 += fabsf(r[t][1]);
    }
    group_sum(p0, p1, s0, s1);
    const __half2 ah = __floats2half2_rn(s0 / fgs, s1 / fgs);
    const float2 a = __half22float2(ah);
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int t = 0; t < 32; t++) {
      const bool up0 = r[t][0] >= 0.f, up1 = r[t][1] >= 0.f;
      w0 |= (up0 ? 1u : 0u) << t;
      w1 |= (up1 ? 1u : 0u) << t;
      r[t][0] -= up0 ? a.x : -a.x;
      r[t][1] -= up1 ? a.y : -a.y;
    }
    if (!live) continue;
    const size_t ai = ((size_t)g * nb + b) * M + m;
    if (run == 0 && HQ_IN_BOUNDS(alpha + ai, 4, alpha, (size_t)(K / gs) * nb * M * 2, 1004))
      *reinterpret_cast<__half2*>(alpha + ai) = ah;
    const size_t wi = ((size_t)(k0 >> 5) * nb + b) * M + m;
    if (HQ_IN_BOUNDS(bW + wi, 8, bW, (size_t)(K / 32) * nb * M * 4, 1005))
      *reinterpret_cast<uint2*>(bW + wi) = make_uint2(w0, w1);
  }
}

template <int DTYPE>
int run(const void* W, int K, int M, int nb, int gs, uint32_t* bW, void* alpha, void* q_bias,
        cudaStream_t st) {
  if (gs / 32 > kMaxRuns) return HQ_ERR_UNSUPPORTED;
  bcq_quantize_kernel<DTYPE><<<dim3((M + kColsPerCta - 1) / kColsPerCta, K / gs), gs, 0, st>>>(
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
  if (!aligned16(W) || !aligned16(bW) || !aligned4(alpha_half) ||
      (q_bias_half && !aligned4(q_bias_half)))
    return HQ_ERR_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HQ_DTYPE_F16: return run<HQ_DTYPE_F16>(W, K, M, nb, group_size, bW, alpha_half, q_bias_half, st);
    case HQ_DTYPE_BF16: return run<HQ_DTYPE_BF16>(W, K, M, nb, group_size, bW, alpha_half, q_bias_half, st);
    case HQ_DTYPE_F32: return run<HQ_DTYPE_F32>(W, K, M, nb, group_size, bW, alpha_half, q_bias_half, st);
    default: return HQ_ERR_UNSUPPORTED;
  }
}
