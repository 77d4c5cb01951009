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
// Design: one channel per thread, grid-stride.  16 bytes per channel move, but
// the kernel waits for its fp64 divisions (the reference has three per channel).
// Here: (max - min) / span divides by a kernel-wide constant, so it is a product
// with the correctly rounded reciprocal and one fused residual correction, which
// gives the correctly rounded quotient (q' = q + (a - q b) * RN(1/b), q faithful).
// The symmetric case needs no further quotient.  Otherwise, unless both ends of
// the range lie away from zero (possible only without preserve_sparsity), one of
// min / scale and max / scale is zero and the other is only needed exactly where
// an fp32 estimate of it cannot settle the outcome: see the kernel.
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

__global__ void __launch_bounds__(kThreads)
zero_point_kernel(const float* __restrict__ x_min, const float* __restrict__ x_max, int qmin,
                  int qmax, int size, int preserve_sparsity, float* __restrict__ scale,
                  int* __restrict__ zero_point) {
  const int span = qmax - qmin;
  const int sym_lo = -(span / 2 + 1), sym_hi = span / 2;
  const double dspan = (double)span, rcp_span = 1.0 / dspan;
  const bool sym_exact = -sym_lo < (1 << 24);
  const int mid_nudged = nudge((double)(qmin + qmax) / 2.0, qmin, qmax);  // the symmetric case
  const float fqmin = (float)qmin, fqmax = (float)qmax;
  const float tol_base = fabsf(fqmin) + fabsf(fqmax) + 1.f;
  for (int i = blockIdx.x * kThreads + threadIdx.x; i < size; i += gridDim.x * kThreads) {
    if (!HQ_IN_BOUNDS(x_min + i, 4, x_min, (size_t)size * 4, 701) ||
        !HQ_IN_BOUNDS(x_max + i, 4, x_max, (size_t)size * 4, 702))
      continue;
    float lo = __ldg(x_min + i), hi = __ldg(x_max + i);
    if (preserve_sparsity && lo < 0.f && hi > 0.f) {
      // float / int: an fp32 division
      const float m = fmaxf(fabsf(lo / (float)sym_lo), fabsf(hi / (float)sym_hi));
      if (sym_exact) {  // the fp64 product of a float and a 24-bit integer, rounded to fp32,
        lo = m * (float)sym_lo;  // is the fp32 product
        hi = m * (float)sym_hi;
      } else {
        lo = (float)((double)m * (double)sym_lo);
        hi = (float)((double)m * (double)sym_hi);
      }
    }
    lo = fminf(lo, 0.f);
    hi = fmaxf(hi, 0.f);
    // RN((hi - lo) / span): product with RN(1 / span), exact residual, correction
    const double d = (double)hi - (double)lo;
    double q = d * rcp_span;
    q = fma(fma(-q, dspan, d), rcp_span, q);
    if (isinf(d)) q = d;  // an adjusted range that overflowed fp32: the residual is not a number
    float sc = (float)q;
    if (sc == 0.f || isinf(1.f / sc)) sc = 0.1f;
    int nudged;
    if (preserve_sparsity && lo < 0.f && hi > 0.f) {  // asked again of the adjusted range
      nudged = mid_nudged;
    } else if (lo != 0.f && hi != 0.f) {  // both ends away from zero: preserve_sparsity off
      const double s = (double)sc;
      nudged = choose_and_nudge((double)lo / s, (double)hi / s, qmin, qmax);
    } else {
      // One end is zero and so is its quotient; the other quotient is first
      // estimated in fp32 from the reciprocal of the scale.  Which end wins and
      // where the zero point rounds to are read off the estimate whenever it is
      // further than its error bound from every point of decision - it always is
      // when the zero end wins, as in the reference driver's own configuration;
      // the fp64 division runs only for the channels where it is not.
      const bool lo_side = lo != 0.f;  // the end with the non-zero numerator
      const float num = lo_side ? lo : hi;
      const float rs = 1.f / sc;
      const float est = num * rs;      // relative error below 2^-22, absolute 2^-149 when tiny
      const float mag = fabsf(est);
      const float f_num = lo_side ? fqmin : fqmax, f_zero = lo_side ? fqmax : fqmin;
      const float e_num = fabsf(f_num) + mag, e_zero = fabsf(f_zero);
      const bool lo_wins = lo_side ? e_num < e_zero : e_zero < e_num;  // err_lo < err_hi
      const bool num_wins = lo_side == lo_wins;
      const float tol = (mag + tol_base) * 0x1p-20f;  // covers est, int -> float and the sums
      bool sure = num == 0.f || (fabsf(rs) >= 1.17549435e-38f && fabsf(e_num - e_zero) > tol);
      nudged = lo_wins ? qmin : qmax;  // the zero end: its candidate is qmin or qmax itself
      if (sure && num_wins && num != 0.f) {
        const float z = f_num - est;
        if (z < fqmin - tol) nudged = qmin;
        else if (z > fqmax + tol) nudged = qmax;
        else if (z > fqmin + tol && z < fqmax - tol && fabsf(z - floorf(z) - 0.5f) > tol)
          nudged = (int)rintf(z);
        else sure = false;
      }
      if (!sure) {
        const double one = (double)num / (double)sc;
        nudged = choose_and_nudge(lo_side ? one : 0.0, lo_side ? 0.0 : one, qmin, qmax);
      }
    }
    if (HQ_IN_BOUNDS(scale + i, 4, scale, (size_t)size * 4, 703)) scale[i] = sc;
    if (HQ_IN_BOUNDS(zero_point + i, 4, zero_point, (size_t)size * 4, 704)) zero_point[i] = nudged;
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
  const int grid = std::min((size + kThreads - 1) / kThreads, sm_count() * 8);
  zero_point_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
      x_min, x_max, qmin, qmax, size, preserve_sparsity, scale, zero_point);
  return launch_status();
}
