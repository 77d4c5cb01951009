// Decode-time MLP entry fused around the weight-only mat-vec, for sm_100a:
//   RMSNorm of the input vector  ->  mat-vec  ->  gated activation of row pairs
// in ONE kernel, for fp16 and uniform int8 / int4 weights (the NF4 form is a
// variant of the NF4 mat-vec kernel itself, nf4.cu).  At batch 1 the
// normalised vector (K halves) and the two projections (2 x N halves) otherwise
// make two round trips through memory and cost two more launches, each as long
// as the mat-vec of a small layer.
//
// Semantics (the host references of the stand-alone benchmarks):
//  * RMSNorm (rmsnorm-cuda/reference.h:4-25): xn[k] = x[k] * rsqrt(mean(x^2) +
//    eps) * gamma[k]; skipped when gamma is null.  Computed in fp32, rounded to
//    fp16 once (the products of the mat-vec are fp16 pairs).
//  * mat-vec: as hq_gemv_f16 / hq_gemv_int8_f16 / hq_gemv_int4_f16 (same
//    layouts, same scale / zero point rules), fp32 accumulation over 32- or
//    64-weight partial sums.
//  * gated activation: with act != 0 the matrix has 2 * rows_out rows, row 2m the
//    value row and row 2m + 1 the gate row of output m (the x / gate order of
//    geglu-cuda/reference.h:8-16, per output feature), and
//      out[m] = v * g / (1 + exp(-g))                (HQ_ACT_SWIGLU; swish-cuda/reference.h:4)
//      out[m] = v * 0.5 * g * (1 + erf(g / sqrt 2))  (HQ_ACT_GEGLU;  geglu-cuda/reference.h:1-5)
//    in fp32, rounded to fp16 once.  With act == 0 the kernel is the plain
//    mat-vec (plus the RMSNorm) and writes rows_out results.
//
// Design: the row-streaming form of gemv_uniform.cu (two 512-thread CTAs per SM,
// a warp owns a PAIR of adjacent rows - here exactly a value / gate pair -, the
// input vector piece-major in shared memory, eight 128-bit streaming loads per
// lane in flight).  The prologue reads the input vector twice from L1/L2 (sum of
// squares, then scale and stage).
#include <algorithm>

#include "gemv_rows.cuh"

namespace hq {
namespace {

using namespace rows;

struct FusedParams {
  const unsigned char* mat;
  const __half* x;
  const __half* gamma;   // null: no RMSNorm
  __half* out;
  float eps, scale, zero_point;
  int rows_out, n, act;
};

// sum over the CTA (all threads get the result); buf holds kWarps floats
__device__ __forceinline__ float block_sum(float v, float* buf, int lane, int warp) {
  v = warp_sum(v);
  __syncthreads();  // buf may still be read from an earlier use
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; w++) t += buf[w];
  return t;
}

template <int BITS>
__global__ void __launch_bounds__(kThreads, 2)
gemv_fused_kernel(const FusedParams p) {
  extern __shared__ __align__(16) unsigned char dsm_raw[];  // the inputs
  __shared__ float s_part[kWarps];
  __half* xs = reinterpret_cast<__half*>(dsm_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kPieces = BITS == 16 ? 1 : 16 / BITS;  // 16-byte pieces of inputs per chunk
  const int n = p.n;
  const size_t row_bytes = (size_t)n * BITS / 8;
  const int chunks = (int)(row_bytes / 16);
  const int rows_mat = p.act ? 2 * p.rows_out : p.rows_out;

  // Programmatic dependent launch: nothing that earlier work of the stream may
  // have produced is read, and nothing is written, before the wait.
  pdl_launch_dependents();
  pdl_wait();

  // ---- RMSNorm: sum of squares over the whole vector ----
  const uint4* xg = reinterpret_cast<const uint4*>(p.x);
  const uint4* gg = reinterpret_cast<const uint4*>(p.gamma);
  float norm = 1.f;
  if (p.gamma != nullptr) {
    float sq = 0.f;
    for (int i = tid; i < n / 8; i += kThreads) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (HQ_IN_BOUNDS(xg + i, 16, p.x, (size_t)n * 2, 501)) v = ld_dependent_u4(xg + i);
      const uint32_t h[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float2 f = __half22float2(u32_as_half2(h[k]));
        sq = fmaf(f.x, f.x, fmaf(f.y, f.y, sq));
      }
    }
    sq = block_sum(sq, s_part, lane, warp);
    norm = rsqrtf(sq / (float)n + p.eps);
  }
  // ---- scale, round to fp16, stage piece-major; sum of the staged inputs ----
  float part = 0.f;
  for (int i = tid; i < n / 8; i += kThreads) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (HQ_IN_BOUNDS(xg + i, 16, p.x, (size_t)n * 2, 502)) v = ld_dependent_u4(xg + i);
    if (p.gamma != nullptr) {
      uint4 g = make_uint4(0, 0, 0, 0);
      if (HQ_IN_BOUNDS(gg + i, 16, p.gamma, (size_t)n * 2, 503)) g = __ldg(gg + i);
      uint32_t h[4] = {v.x, v.y, v.z, v.w};
      const uint32_t gh[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float2 f = __half22float2(u32_as_half2(h[k]));
        const float2 w = __half22float2(u32_as_half2(gh[k]));
        h[k] = half2_as_u32(__floats2half2_rn(f.x * norm * w.x, f.y * norm * w.y));
      }
      v = make_uint4(h[0], h[1], h[2], h[3]);
    }
    // 16-byte piece q of chunk c goes to [q][c] (int4: in the order of its conversion)
    reinterpret_cast<uint4*>(xs)[(i % kPieces) * chunks + i / kPieces] = BITS == 4 ? pair_inputs(v) : v;
    const float2 f0 = __half22float2(u32_as_half2(v.x)), f1 = __half22float2(u32_as_half2(v.y)),
                 f2 = __half22float2(u32_as_half2(v.z)), f3 = __half22float2(u32_as_half2(v.w));
    part += ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
  }
  const float sumx = block_sum(part, s_part, lane, warp);  // also: table and inputs complete

  // ---- row pairs of this warp ----
  const int warps_total = gridDim.x * kWarps;
  constexpr int kPerRow = kInFlight / kRows;
  const size_t mat_bytes = (size_t)rows_mat * row_bytes;
  (void)mat_bytes;
  for (long long row0 = ((long long)blockIdx.x * kWarps + warp) * kRows; row0 < rows_mat;
       row0 += (long long)warps_total * kRows) {
    const unsigned char* src = p.mat + (size_t)row0 * row_bytes;
    float acc[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) acc[r] = 0.f;
    for (int c0 = lane; c0 < chunks; c0 += 32 * kPerRow) {
      uint4 w[kPerRow][kRows];
#pragma unroll
      for (int u = 0; u < kPerRow; u++) {
        const int c = c0 + 32 * u;
#pragma unroll
        for (int r = 0; r < kRows; r++) {
          const unsigned char* at = src + (size_t)r * row_bytes + (size_t)c * 16;
          w[u][r] = make_uint4(0, 0, 0, 0);  // a row past the end contributes zeros
          if (c < chunks && row0 + r < rows_mat && HQ_IN_BOUNDS(at, 16, p.mat, mat_bytes, 504))
            w[u][r] = ldg_stream_u4(at);
        }
      }
#pragma unroll
      for (int u = 0; u < kPerRow; u++) {
        const int c = c0 + 32 * u;
        if (c < chunks) {
          float part2[kRows];
          chunk_dot<BITS, kRows>(w[u], reinterpret_cast<const uint4*>(xs) + c, chunks, part2);
#pragma unroll
          for (int r = 0; r < kRows; r++)
            acc[r] += part2[r];
        }
      }
    }
    float val[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) {
      const float total = warp_sum(acc[r]);
      val[r] = BITS == 16 ? total : p.scale * (total - p.zero_point * sumx);
    }
    if (lane == 0) {
      if (p.act) {
        const long long m = row0 >> 1;  // row0 is even: the value row; row0 + 1 the gate row
        if (HQ_IN_BOUNDS(p.out + m, 2, p.out, (size_t)p.rows_out * 2, 506))
          p.out[m] = __float2half_rn(val[0] * gate_act(val[1], p.act));
      } else {
#pragma unroll
        for (int r = 0; r < kRows; r++)
          if (row0 + r < rows_mat && HQ_IN_BOUNDS(p.out + row0 + r, 2, p.out, (size_t)p.rows_out * 2, 507))
            p.out[row0 + r] = __float2half_rn(val[r]);
      }
    }
  }
}

template <int BITS>
int launch(FusedParams prm, hq_stream_t stream) {
  if (!prm.mat || !prm.x || !prm.out) return HQ_ERR_NULL_POINTER;
  if (prm.rows_out <= 0 || prm.n <= 0 || prm.n % (128 / BITS) != 0) return HQ_ERR_BAD_SHAPE;
  if (prm.act != HQ_ACT_NONE && prm.act != HQ_ACT_SWIGLU && prm.act != HQ_ACT_GEGLU)
    return HQ_ERR_BAD_SHAPE;
  if (!aligned16(prm.mat) || !aligned16(prm.x) || (prm.gamma && !aligned16(prm.gamma)))
    return HQ_ERR_MISALIGNED;
  const size_t smem = (size_t)prm.n * 2;
  if (smem > 226 * 1024) return HQ_ERR_TOO_LARGE;  // beyond 113 KiB only one CTA fits an SM
  constexpr auto kern = gemv_fused_kernel<BITS>;
  const cudaError_t e = ensure_dynamic_smem<kern>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  const int rows_mat = prm.act ? 2 * prm.rows_out : prm.rows_out;
  const int grid = std::min(2 * sm_count(), (rows_mat + kWarps * kRows - 1) / (kWarps * kRows));
  return cuda_status(
      launch_pdl(kern, dim3(grid), dim3(kThreads), smem, (cudaStream_t)stream, prm));
}

FusedParams base_params(const void* mat, const void* x_half, const void* gamma_half, float eps,
                        void* out_half, int rows_out, int n, int act) {
  FusedParams prm = {};
  prm.mat = reinterpret_cast<const unsigned char*>(mat);
  prm.x = reinterpret_cast<const __half*>(x_half);
  prm.gamma = reinterpret_cast<const __half*>(gamma_half);
  prm.out = reinterpret_cast<__half*>(out_half);
  prm.eps = eps;
  prm.scale = 1.f;
  prm.rows_out = rows_out;
  prm.n = n;
  prm.act = act;
  return prm;
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_gemv_fused_f16(const void* x_half, const void* gamma_half, float eps, const void* mat_half,
                      void* out_half, int rows_out, int n, int act, hq_stream_t stream) {
  using namespace hq;
  return launch<16>(base_params(mat_half, x_half, gamma_half, eps, out_half, rows_out, n, act),
                      stream);
}

int hq_gemv_fused_int8_f16(const void* x_half, const void* gamma_half, float eps, const int8_t* mat,
                           void* out_half, int rows_out, int n, float scale, float zero_point,
                           int act, hq_stream_t stream) {
  using namespace hq;
  FusedParams prm = base_params(mat, x_half, gamma_half, eps, out_half, rows_out, n, act);
  prm.scale = __half2float(__float2half_rn(scale));  // as the reference launchers (gemv.cu:21-22)
  prm.zero_point = __half2float(__float2half_rn(zero_point));
  return launch<8>(prm, stream);
}

int hq_gemv_fused_int4_f16(const void* x_half, const void* gamma_half, float eps,
                           const uint8_t* mat, void* out_half, int rows_out, int n, float scale,
                           float zero_point, int act, hq_stream_t stream) {
  using namespace hq;
  FusedParams prm = base_params(mat, x_half, gamma_half, eps, out_half, rows_out, n, act);
  prm.scale = __half2float(__float2half_rn(scale));
  prm.zero_point = __half2float(__float2half_rn(zero_point));
  return launch<4>(prm, stream);
}

}  // extern "C"
