// Affine quantization parameters from per-channel minima and maxima
// (zeropoint-cuda) for sm_100a: the step before any of the integer packers.
//
// Reference semantics (zeropoint-cuda/main.cu:10-80, host check
// reference.h:1-71), per channel i, bit for bit:
//  * preserve_sparsity and min < 0 < max: the range is made symmetric around zero
//    first - m = max(|min / -(span/2 + 1)|, |max / (span/2)|) with span = qmax -
//    qmin and the two quotients formed in fp32, then min = m * -(span/2 + 1),
//    max = m * (span/2), products in fp64 rounded to fp32;
//  * the range is widened to contain 0; scale = fp32((double(max) - min) / span);
//    a scale of 0, or one whose fp32 reciprocal overflows, becomes 0.1;
//  * the zero point is taken from the end of the range with the smaller
//    |q| + |x / scale| (fp64), or is (qmin + qmax) / 2 in the symmetric case,
//    then clamped to [qmin, qmax] and rounded to the nearest integer, ties to even.
// The arithmetic types are part of the result and are kept: fp32 quotients where
// the reference divides a float by an int, fp64 elsewhere.
//
// Design: four channels per thread (128-bit loads and stores), grid-stride.  16
// bytes per channel move; what the reference spends its time on is five
// divisions per channel (two fp32, three fp64).  Here
//  * a division by a kernel-wide constant (the two symmetric bounds in fp32, the
//    span in fp64) is a product with the correctly rounded reciprocal and one
//    fused residual correction, q' = q + (a - q b) * RN(1/b), which is the
//    correctly rounded quotient when q is within an ulp and nothing underflows
//    (tiny fp32 numerators take the division);
//  * "the fp32 reciprocal of the scale overflows" is |scale| <= 2^-128;
//  * the symmetric case needs no further quotient.  Otherwise, unless both ends
//    of the range lie away from zero (possible only without preserve_sparsity),
//    one of min / scale and max / scale is zero and the other is only needed
//    exactly where an fp32 estimate of it cannot settle the outcome: see below.
#include <algorithm>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;

// clamp to [qmin, qmax], then to the nearest integer, ties to even
__device__ __forceinline__ int nudge(double z, int qmin, int qmax) {
  if (z < (double)qmin) return qmin;
  if (z > (double)qmax) return qmax;
  return (int)rint(z);
}
// the end of the range with the smaller |q| + |x / scale| gives the zero point
__device__ __forceinline__ int choose_and_nudge(double q_lo, double q_hi, int qmin, int qmax) {
  const double err_lo = (double)abs(qmin) + fabs(q_lo), err_hi = (double)abs(qmax) + fabs(q_hi);
  return nudge(err_lo < err_hi ? (double)qmin - q_lo : (double)qmax - q_hi, qmin, qmax);
}

// what does not depend on the channel
struct Consts {
  int qmin, qmax, preserve;
  float sym_lo, sym_hi, rcp_sym_lo, rcp_sym_hi;  // the symmetric bounds and RN(1 / bound)
  bool sym_exact;                                // |bounds| < 2^24: exact in fp32
  double span, rcp_span;
  int mid_nudged;                                // the zero point of the symmetric case
  float fqmin, fqmax, tol_base;
};

// a / b in fp32, correctly rounded, b a constant with rcp = RN(1 / b)
__device__ __forceinline__ float div_const(float a, float b, float rcp) {
  if (!(fabsf(a) >= 0x1p-87f)) return a / b;  // the residual below could underflow (or a is NaN)
  const float q = a * rcp;
  return fmaf(fmaf(-q, b, a), rcp, q);
}
__device__ __forceinline__ float rcp_estimate(float x) {
  float r;  // within an ulp; a denormal result is flushed to zero
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void one_channel(float lo, float hi, const Consts& k, float& scale,
                                            int& zero_point) {
  if (k.preserve && lo < 0.f && hi > 0.f) {
    // float / int: fp32 quotients
    const float m = fmaxf(fabsf(k.sym_exact ? div_const(lo, k.sym_lo, k.rcp_sym_lo) : lo / k.sym_lo),
                          fabsf(k.sym_exact ? div_const(hi, k.sym_hi, k.rcp_sym_hi) : hi / k.sym_hi));
    if (k.sym_exact) {  // the fp64 product of a float and a 24-bit integer, rounded to fp32,
      lo = m * k.sym_lo;  // is the fp32 product
      hi = m * k.sym_hi;
    } else {
      lo = (float)((double)m * (double)k.sym_lo);
      hi = (float)((double)m * (double)k.sym_hi);
    }
  }
  lo = fminf(lo, 0.f);
  hi = fmaxf(hi, 0.f);
  // RN((hi - lo) / span): product with RN(1 / span), exact residual, correction
  const double d = (double)hi - (double)lo;
  double q = d * k.rcp_span;
  q = fma(fma(-q, k.span, d), k.rcp_span, q);
  if (isinf(d)) q = d;  // an adjusted range that overflowed fp32: the residual is not a number
  float sc = (float)q;
  // zero, or 1.0f / sc overflows: the largest such magnitude is 2^-128
  if (fabsf(sc) <= 0x1p-128f) sc = 0.1f;
  int nudged;
  if (k.preserve && lo < 0.f && hi > 0.f) {  // asked again of the adjusted range
    nudged = k.mid_nudged;
  } else if (lo != 0.f && hi != 0.f) {  // both ends away from zero: preserve_sparsity off
    const double s = (double)sc;
    nudged = choose_and_nudge((double)lo / s, (double)hi / s, k.qmin, k.qmax);
  } else {
    // One end is zero and so is its quotient; the other quotient is first
    // estimated in fp32 from an approximate reciprocal of the scale.  Which end
    // wins and where the zero point rounds to are read off the estimate whenever
    // it is further than its error bound from every point of decision - it
    // always is when the zero end wins, as in the reference driver's own
    // configuration; the fp64 division runs only for the channels where it is not.
    const bool lo_side = lo != 0.f;  // the end with the non-zero numerator
    const float num = lo_side ? lo : hi;
    const float rs = rcp_estimate(sc);
    const float est = num * rs;      // relative error below 2^-21, absolute 2^-126 when tiny
    const float mag = fabsf(est);
    const float f_num = lo_side ? k.fqmin : k.fqmax, f_zero = lo_side ? k.fqmax : k.fqmin;
    const float e_num = fabsf(f_num) + mag, e_zero = fabsf(f_zero);
    const bool lo_wins = lo_side ? e_num < e_zero : e_zero < e_num;  // err_lo < err_hi
    const bool num_wins = lo_side == lo_wins;
    const float tol = (mag + k.tol_base) * 0x1p-19f;  // covers est, int -> float and the sums
    bool sure = num == 0.f || (fabsf(rs) >= 1.17549435e-38f && fabsf(rs) < 3.0e38f &&
                               fabsf(e_num - e_zero) > tol);
    nudged = lo_wins ? k.qmin : k.qmax;  // the zero end: its candidate is qmin or qmax itself
    if (sure && num_wins && num != 0.f) {
      const float z = f_num - est;
      if (z < k.fqmin - tol) nudged = k.qmin;
      else if (z > k.fqmax + tol) nudged = k.qmax;
      else if (z > k.fqmin + tol && z < k.fqmax - tol && fabsf(z - floorf(z) - 0.5f) > tol)
        nudged = (int)rintf(z);
      else sure = false;
    }
    if (!sure) {
      const double one = (double)num / (double)sc;
      nudged = choose_and_nudge(lo_side ? one : 0.0, lo_side ? 0.0 : one, k.qmin, k.qmax);
    }
  }
  scale = sc;
  zero_point = nudged;
}

__global__ void __launch_bounds__(kThreads)
zero_point_kernel(const float* __restrict__ x_min, const float* __restrict__ x_max, int qmin,
                  int qmax, int size, int preserve_sparsity, float* __restrict__ scale,
                  int* __restrict__ zero_point, int vectors) {
  Consts k;
  const int span = qmax - qmin;
  const int sym_lo = -(span / 2 + 1), sym_hi = span / 2;
  k.qmin = qmin;
  k.qmax = qmax;
  k.preserve = preserve_sparsity;
  k.sym_lo = (float)sym_lo;
  k.sym_hi = (float)sym_hi;
  k.sym_exact = -sym_lo < (1 << 24) && sym_hi > 0;
  k.rcp_sym_lo = 1.f / k.sym_lo;
  k.rcp_sym_hi = sym_hi > 0 ? 1.f / k.sym_hi : 0.f;
  k.span = (double)span;
  k.rcp_span = 1.0 / k.span;
  k.mid_nudged = nudge((double)(qmin + qmax) / 2.0, qmin, qmax);
  k.fqmin = (float)qmin;
  k.fqmax = (float)qmax;
  k.tol_base = fabsf(k.fqmin) + fabsf(k.fqmax) + 1.f;
  const int stride = gridDim.x * kThreads;
  // whole groups of four channels (vectors != 0: all four pointers are 16-byte aligned)
  const int nvec = vectors ? size / 4 : 0;
  for (int v = blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
    if (!HQ_IN_BOUNDS(x_min + 4 * v, 16, x_min, (size_t)size * 4, 701) ||
        !HQ_IN_BOUNDS(x_max + 4 * v, 16, x_max, (size_t)size * 4, 702))
      continue;
    const uint4 l4 = ldg_stream_u4(reinterpret_cast<const uint4*>(x_min) + v);
    const uint4 h4 = ldg_stream_u4(reinterpret_cast<const uint4*>(x_max) + v);
    const float lo[4] = {__uint_as_float(l4.x), __uint_as_float(l4.y), __uint_as_float(l4.z),
                         __uint_as_float(l4.w)};
    const float hi[4] = {__uint_as_float(h4.x), __uint_as_float(h4.y), __uint_as_float(h4.z),
                         __uint_as_float(h4.w)};
    float sc[4];
    int zp[4];
#pragma unroll
    for (int j = 0; j < 4; j++) one_channel(lo[j], hi[j], k, sc[j], zp[j]);
    if (HQ_IN_BOUNDS(scale + 4 * v, 16, scale, (size_t)size * 4, 703))
      reinterpret_cast<float4*>(scale)[v] = make_float4(sc[0], sc[1], sc[2], sc[3]);
    if (HQ_IN_BOUNDS(zero_point + 4 * v, 16, zero_point, (size_t)size * 4, 704))
      reinterpret_cast<int4*>(zero_point)[v] = make_int4(zp[0], zp[1], zp[2], zp[3]);
  }
  // the channels left over, or all of them
  for (int i = 4 * nvec + blockIdx.x * kThreads + threadIdx.x; i < size; i += stride) {
    if (!HQ_IN_BOUNDS(x_min + i, 4, x_min, (size_t)size * 4, 705) ||
        !HQ_IN_BOUNDS(x_max + i, 4, x_max, (size_t)size * 4, 706))
      continue;
    float sc;
    int zp;
    one_channel(__ldg(x_min + i), __ldg(x_max + i), k, sc, zp);
    if (HQ_IN_BOUNDS(scale + i, 4, scale, (size_t)size * 4, 707)) scale[i] = sc;
    if (HQ_IN_BOUNDS(zero_point + i, 4, zero_point, (size_t)size * 4, 708)) zero_point[i] = zp;
  }
}

}  // namespace
}  // namespace hq

extern "C" int hq_zero_point(const float* x_min, const float* x_max, int32_t qmin, int32_t qmax,
                             int size, int preserve_sparsity, float* scale, int32_t* zero_point,
                             hq_stream_t stream) {
  using namespace hq;
  if (size < 0 || qmax <= qmin) return HQ_ERR_BAD_SHAPE;
  if (size == 0) return HQ_OK;
  if (!x_min || !x_max || !scale || !zero_point) return HQ_ERR_NULL_POINTER;
  const int vectors = aligned16(x_min) && aligned16(x_max) && aligned16(scale) && aligned16(zero_point);
  const int items = vectors ? (size + 3) / 4 : size;
  const int grid = std::min((items + kThreads - 1) / kThreads, sm_count() * 8);
  zero_point_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
      x_min, x_max, qmin, qmax, size, preserve_sparsity, scale, zero_point, vectors);
  return launch_status();
}
