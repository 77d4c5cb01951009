// Round-to-nearest 3-bit quantizer and packer for sm_100a: fp16 / bf16 / fp32
// weights W[K][N] -> the packed matrix, scales and zeros that the 3-bit mat-vec
// kernels (hq_q3_gemv_f32 / _f16in, the layout of quant3MatMul-cuda) consume.
// The reference tree only holds the consumer (quant3MatMul-cuda/kernels.h); the
// rule is the per-column min / max quantizer of GPTQ without its error search:
//   lo = min(min_k W[k][c], 0), hi = max(max_k W[k][c], 0); lo = -1, hi = 1 if both are 0
//   scale = (hi - lo) / 7                        (fp32)
//   z     = rint(-lo / scale)                    (the integer zero point, ties to even)
//   q     = clamp(rint(W[k][c] / scale) + z, 0, 7)
//   scales[c] = scale, zeros[c] = scale * z      (the kernels compute scale * q - zeros[c])
// and the codes of rows 32 r .. 32 r + 31 of a column fill the 96-bit
// little-endian integer formed by rows 3 r, 3 r + 1, 3 r + 2 of mat at bits 3 j
// (the order quant3MatMul-cuda/kernels.h:41-87 extracts them in).
//
// Design.  Two passes over W (2 x 2 bytes per fp16 weight read, 0.375 written):
//  1. column minima and maxima: a warp reads 8 columns per lane (128-bit loads,
//     4 rows in flight), the CTAs of a column tile split K, partial results meet in
//     one atomicMin / atomicMax per column and CTA on order-preserving integer
//     keys of the floats;
//  2. quantize and pack: a warp owns 32 rows x 128 columns, a lane 4 columns; the
//     quotient by the column's scale is a product with the correctly rounded
//     reciprocal and one fused residual correction (the correctly rounded
//     quotient), its rounding to an integer one addition of 1.5 * 2^23; 8 rows at
//     a time become 24 bits that are merged into the three words of the group;
//     one 128-bit store per word row.
#include <cuda_bf16.h>

#include <algorithm>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// float <-> unsigned key with the same order
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// C consecutive weights of row-major W starting at element index e, as fp32
template <int DTYPE, int C>
__device__ __forceinline__ void load_cols(const void* W, size_t e, size_t total, float (&w)[C]) {
  static_assert(C == 4 || C == 8, "4 or 8 columns per lane");
  if (DTYPE == HQ_DTYPE_F32) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(W) + e);
#pragma unroll
    for (int h = 0; h < C / 4; h++) {
      uint4 a = make_uint4(0, 0, 0, 0);
      if (HQ_IN_BOUNDS(p + h, 16, W, total * 4, 901)) a = ldg_stream_u4(p + h);
      w[4 * h] = __uint_as_float(a.x);
      w[4 * h + 1] = __uint_as_float(a.y);
      w[4 * h + 2] = __uint_as_float(a.z);
      w[4 * h + 3] = __uint_as_float(a.w);
    }
  } else {
    uint32_t u[C / 2];
    const unsigned short* p = reinterpret_cast<const unsigned short*>(W) + e;
    if (C == 8) {
      uint4 a = make_uint4(0, 0, 0, 0);
      if (HQ_IN_BOUNDS(p, 16, W, total * 2, 902)) a = ldg_stream_u4(p);
      u[0] = a.x; u[1] = a.y; u[C / 2 - 2] = a.z; u[C / 2 - 1] = a.w;
    } else {
      uint2 a = make_uint2(0, 0);
      if (HQ_IN_BOUNDS(p, 8, W, total * 2, 903)) a = ldg_stream_u2(p);
      u[0] = a.x; u[1] = a.y;
    }
#pragma unroll
    for (int j = 0; j < C / 2; j++) {
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

// pass 1: keys[c] = min, keys[N + c] = max over the rows of this CTA's K slice
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
q3_minmax_kernel(const void* __restrict__ W, int K, int N, int rows_per_cta,
                 uint32_t* __restrict__ keys) {
  __shared__ float s_lo[kWarps][256], s_hi[kWarps][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const int k0 = blockIdx.y * rows_per_cta, k1 = min(K, k0 + rows_per_cta);
  const size_t total = (size_t)K * N;
  float lo[8], hi[8];
#pragma unroll
  for (int j = 0; j < 8; j++) {
    lo[j] = __int_as_float(0x7f800000);
    hi[j] = __int_as_float(0xff800000);
  }
  if (col < N) {
    for (int k = k0 + warp; k < k1; k += kWarps * 4) {
      float w[4][8];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int kk = k + u * kWarps;
        if (kk < k1) load_cols<DTYPE, 8>(W, (size_t)kk * N + col, total, w[u]);
        else {
#pragma unroll
          for (int j = 0; j < 8; j++) w[u][j] = __int_as_float(0x7fc00000);  // NaN: ignored by fmin / fmax
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
          lo[j] = fminf(lo[j], w[u][j]);
          hi[j] = fmaxf(hi[j], w[u][j]);
        }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; j++) {
    s_lo[warp][lane * 8 + j] = lo[j];
    s_hi[warp][lane * 8 + j] = hi[j];
  }
  __syncthreads();
  const int c = threadIdx.x;  // one column of the tile per thread
  if (blockIdx.x * 256 + c < N) {
    float l = s_lo[0][c], h = s_hi[0][c];
#pragma unroll
    for (int w = 1; w < kWarps; w++) {
      l = fminf(l, s_lo[w][c]);
      h = fmaxf(h, s_hi[w][c]);
    }
    const int gc = blockIdx.x * 256 + c;
    if (HQ_IN_BOUNDS(keys + gc, 4, keys, (size_t)N * 8, 904)) atomicMin(keys + gc, order_key(l));
    if (HQ_IN_BOUNDS(keys + N + gc, 4, keys, (size_t)N * 8, 905))
      atomicMax(keys + N + gc, order_key(h));
  }
}

struct ColumnParams {
  float scale, rcp, zero;  // zero: the integer zero point as rint left it (a zero keeps its sign)
  int zero_int;
  bool plain;  // the scale is too small or too large for the corrected product: divide
};
__device__ __forceinline__ ColumnParams column_params(float lo, float hi) {
  lo = fminf(lo, 0.f);
  hi = fmaxf(hi, 0.f);
  if (lo == 0.f && hi == 0.f) {
    lo = -1.f;
    hi = 1.f;
  }
  ColumnParams p;
  p.scale = (hi - lo) / 7.f;
  p.rcp = 1.f / p.scale;
  p.zero = rintf(-lo / p.scale);
  p.zero_int = (int)p.zero;
  p.plain = !(p.scale >= 0x1p-60f && p.scale <= 0x1p60f);
  return p;
}
// clamp(rint(w / scale) + z, 0, 7).  The quotient is the corrected product q' = q +
// (w - q * scale) * RN(1 / scale), i.e. the correctly rounded w / scale: every
// weight of the column lies within 7 scales of zero, so nothing overflows, and
// where the residual would underflow (|w| below 2^-87 with a scale of at least
// 2^-60) the quotient is below 2^-27 and rounds to 0 whatever its last bit.  The
// rounding to an integer is the addition of 1.5 * 2^23, which leaves rint(q) in
// the low mantissa bits.
template <bool PLAIN>
__device__ __forceinline__ uint32_t code_of(float w, const ColumnParams& p) {
  float q;
  if (PLAIN) {
    q = w / p.scale;
  } else {
    q = w * p.rcp;
    q = fmaf(fmaf(-q, p.scale, w), p.rcp, q);
  }
  const int r = __float_as_int(q + 12582912.f) - 0x4b400000 + p.zero_int;
  return (uint32_t)min(max(r, 0), 7);
}

// four adjacent weights as they lie in memory, and as fp32
template <int DTYPE>
struct Raw4 {
  uint4 v;  // fp32: all of it; 16-bit types: x and y
};
template <int DTYPE>
__device__ __forceinline__ Raw4<DTYPE> load_raw4(const void* W, size_t e, size_t total) {
  Raw4<DTYPE> r;
  r.v = make_uint4(0, 0, 0, 0);
  if (DTYPE == HQ_DTYPE_F32) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(W) + e);
    if (HQ_IN_BOUNDS(p, 16, W, total * 4, 901)) r.v = ldg_stream_u4(p);
  } else {
    const unsigned short* p = reinterpret_cast<const unsigned short*>(W) + e;
    if (HQ_IN_BOUNDS(p, 8, W, total * 2, 903)) {
      const uint2 a = ldg_stream_u2(p);
      r.v.x = a.x;
      r.v.y = a.y;
    }
  }
  return r;
}
template <int DTYPE>
__device__ __forceinline__ void widen4(const Raw4<DTYPE>& r, float (&w)[4]) {
  if (DTYPE == HQ_DTYPE_F32) {
    w[0] = __uint_as_float(r.v.x); w[1] = __uint_as_float(r.v.y);
    w[2] = __uint_as_float(r.v.z); w[3] = __uint_as_float(r.v.w);
  } else if (DTYPE == HQ_DTYPE_BF16) {
    w[0] = __uint_as_float(r.v.x << 16); w[1] = __uint_as_float(r.v.x & 0xffff0000u);
    w[2] = __uint_as_float(r.v.y << 16); w[3] = __uint_as_float(r.v.y & 0xffff0000u);
  } else {
    const float2 a = __half22float2(u32_as_half2(r.v.x)), b = __half22float2(u32_as_half2(r.v.y));
    w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
  }
}

// the codes of RB rows x 4 columns (rows b0 .. b0 + RB - 1 of the group) merged
// into the columns' 96 bits
template <int DTYPE, int RB, bool PLAIN>
__device__ __forceinline__ void pack_rows(const Raw4<DTYPE> (&raw)[RB], int b0, const ColumnParams (&cp)[4],
                                          unsigned long long (&low)[4], uint32_t (&high)[4]) {
#pragma unroll
  for (int sb = 0; sb < RB / 8; sb++) {  // 8 rows = 24 bits at bit 24 b
    uint32_t v[4] = {0, 0, 0, 0};
#pragma unroll
    for (int r = 0; r < 8; r++) {
      float w[4];
      widen4<DTYPE>(raw[sb * 8 + r], w);
#pragma unroll
      for (int c = 0; c < 4; c++) v[c] |= code_of<PLAIN>(w[c], cp[c]) << (3 * r);
    }
    const int b = b0 / 8 + sb;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      if (b < 2) low[c] |= (unsigned long long)v[c] << (24 * b);
      if (b == 2) {
        low[c] |= (unsigned long long)v[c] << 48;
        high[c] |= v[c] >> 16;
      }
      if (b == 3) high[c] |= v[c] << 8;
    }
  }
}

// pass 2: a warp packs rows 32 g .. 32 g + 31 of 128 columns.  16-bit inputs: all
// 32 rows of the lane's four columns are requested before the first is used
// (256 bytes per lane in flight); fp32 inputs: 8 rows at a time.
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
q3_pack_kernel(const void* __restrict__ W, int K, int N, const uint32_t* __restrict__ keys,
               int32_t* __restrict__ mat, float* __restrict__ scales, float* __restrict__ zeros) {
  constexpr int RB = DTYPE == HQ_DTYPE_F32 ? 8 : 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 128 + lane * 4;
  const int g = blockIdx.y * kWarps + warp;  // K group of this warp
  if (col >= N || g * 32 >= K) return;
  const size_t total = (size_t)K * N;
  Raw4<DTYPE> raw[RB];
#pragma unroll
  for (int r = 0; r < RB; r++) raw[r] = load_raw4<DTYPE>(W, (size_t)(g * 32 + r) * N + col, total);
  ColumnParams cp[4];
#pragma unroll
  for (int c = 0; c < 4; c++)
    cp[c] = column_params(key_value(__ldg(keys + col + c)), key_value(__ldg(keys + N + col + c)));
  if (g == 0) {
    if (HQ_IN_BOUNDS(scales + col, 16, scales, (size_t)N * 4, 906))
      *reinterpret_cast<float4*>(scales + col) =
          make_float4(cp[0].scale, cp[1].scale, cp[2].scale, cp[3].scale);
    if (HQ_IN_BOUNDS(zeros + col, 16, zeros, (size_t)N * 4, 907))
      *reinterpret_cast<float4*>(zeros + col) =
          make_float4(cp[0].scale * cp[0].zero, cp[1].scale * cp[1].zero, cp[2].scale * cp[2].zero,
                      cp[3].scale * cp[3].zero);
  }
  const bool plain = cp[0].plain || cp[1].plain || cp[2].plain || cp[3].plain;
  unsigned long long low[4] = {0, 0, 0, 0};  // bits 0 .. 63 of each column's 96
  uint32_t high[4] = {0, 0, 0, 0};           // bits 64 .. 95
#pragma unroll
  for (int b0 = 0; b0 < 32; b0 += RB) {
    if (b0 > 0) {
#pragma unroll
      for (int r = 0; r < RB; r++)
        raw[r] = load_raw4<DTYPE>(W, (size_t)(g * 32 + b0 + r) * N + col, total);
    }
    if (plain) pack_rows<DTYPE, RB, true>(raw, b0, cp, low, high);
    else pack_rows<DTYPE, RB, false>(raw, b0, cp, low, high);
  }
  int32_t* out = mat + (size_t)(3 * g) * N + col;
  const size_t mat_bytes = (size_t)(K / 32) * 3 * N * 4;
  (void)mat_bytes;
  if (HQ_IN_BOUNDS(out, 16, mat, mat_bytes, 908))
    *reinterpret_cast<uint4*>(out) =
        make_uint4((uint32_t)low[0], (uint32_t)low[1], (uint32_t)low[2], (uint32_t)low[3]);
  if (HQ_IN_BOUNDS(out + N, 16, mat, mat_bytes, 909))
    *reinterpret_cast<uint4*>(out + N) = make_uint4((uint32_t)(low[0] >> 32), (uint32_t)(low[1] >> 32),
                                                    (uint32_t)(low[2] >> 32), (uint32_t)(low[3] >> 32));
  if (HQ_IN_BOUNDS(out + 2 * (size_t)N, 16, mat, mat_bytes, 910))
    *reinterpret_cast<uint4*>(out + 2 * (size_t)N) = make_uint4(high[0], high[1], high[2], high[3]);
}

template <int DTYPE>
int run(const void* W, int K, int N, int32_t* mat, float* scales, float* zeros, uint32_t* keys,
        cudaStream_t st) {
  // keys: minima start at the largest key, maxima at the smallest
  cudaError_t e = cudaMemsetAsync(keys, 0xff, (size_t)N * 4, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(keys + N, 0, (size_t)N * 4, st);
  if (e != cudaSuccess) return cuda_status(e);
  const int tiles = (N + 255) / 256;
  // enough K slices to fill the GPU a few times over, at least 256 rows each
  int splits = std::max(1, std::min((K + 255) / 256, (4 * sm_count() + tiles - 1) / tiles));
  const int rows_per_cta = ((K + splits - 1) / splits + 31) / 32 * 32;
  splits = (K + rows_per_cta - 1) / rows_per_cta;
  q3_minmax_kernel<DTYPE><<<dim3(tiles, splits), kThreads, 0, st>>>(W, K, N, rows_per_cta, keys);
  int rc = launch_status();
  if (rc != HQ_OK) return rc;
  const dim3 grid((N + 127) / 128, (K / 32 + kWarps - 1) / kWarps);
  q3_pack_kernel<DTYPE><<<grid, kThreads, 0, st>>>(W, K, N, keys, mat, scales, zeros);
  return launch_status();
}

}  // namespace
}  // namespace hq

extern "C" {

size_t hq_q3_quantize_workspace_bytes(int N) { return N > 0 ? (size_t)N * 8 : 0; }

int hq_q3_quantize(const void* W, int dtype, int K, int N, int32_t* mat, float* scales,
                   float* zeros, void* workspace, size_t workspace_bytes, hq_stream_t stream) {
  using namespace hq;
  if (K <= 0 || N <= 0 || K % 32 != 0 || N % 8 != 0) return HQ_ERR_BAD_SHAPE;
  if (!W || !mat || !scales || !zeros) return HQ_ERR_NULL_POINTER;
  if (!workspace || workspace_bytes < hq_q3_quantize_workspace_bytes(N)) return HQ_ERR_WORKSPACE;
  if (!aligned16(W) || !aligned16(mat) || !aligned16(scales) || !aligned16(zeros) ||
      !aligned4(workspace))
    return HQ_ERR_MISALIGNED;
  if ((size_t)K * (size_t)N > (size_t)1 << 40) return HQ_ERR_TOO_LARGE;
  auto* keys = reinterpret_cast<uint32_t*>(workspace);
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HQ_DTYPE_F16: return run<HQ_DTYPE_F16>(W, K, N, mat, scales, zeros, keys, st);
    case HQ_DTYPE_BF16: return run<HQ_DTYPE_BF16>(W, K, N, mat, scales, zeros, keys, st);
    case HQ_DTYPE_F32: return run<HQ_DTYPE_F32>(W, K, N, mat, scales, zeros, keys, st);
    default: return HQ_ERR_UNSUPPORTED;
  }
}

}  // extern "C"
