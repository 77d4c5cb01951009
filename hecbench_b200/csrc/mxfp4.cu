// MXFP4 (OCP microscaling: 32 elements share one power-of-two scale, each
// element is a 4-bit e2m1 float) for sm_100a: quantize-dequantize in place of
// the reference kernel, plus the packer and the unpacker that the simulation
// stands for.
//
// Reference semantics (mxfp4-cuda/main.cu:112-150, qdq_mxfp4_kernel; constants
// common.h:12-34), per group of 32 consecutive elements of an fp16 or bf16 tensor:
//   m  = max |x|, its mantissa rounded to a power of two: bits + (quarter of the
//        mantissa range), mantissa cleared - so 1.75 * 2^e and above become 2^(e+1)
//   k  = clamp(floor(log2 m) - 2, -127, 127)      (e2m1's largest binade is 2^2)
//   q  = x / 2^k rounded to the e2m1 grid {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the
//        even mantissa (main.cu:21-109: .25 -> 0, .75 -> 1, 1.25 -> 1, 1.75 -> 2,
//        2.5 -> 2, 3.5 -> 4, 5 -> 4), magnitudes above 6 saturate, sign kept
//   y  = q * 2^k
// The reference computes in the input type.  Every step is a scaling by a power
// of two or a rounding to a grid coarser than the input's, so the same values
// come out of fp32 arithmetic, which is what the kernels below use; fp32 also
// makes the extension to what the reference leaves undefined harmless: a group
// whose maximum rounds to a zero exponent field (zero, small denormals: the
// reference takes log2 of 0 and overflows an int) here gets the smallest scale
// the reference's expression can produce, and a zero group gives zeros.
// NaN and infinity are not treated specially in either.
//
// Packed form (hq_mxfp4_quantize / hq_mxfp4_dequantize): one byte per two
// elements, element 2j in the LOW nibble, nibble = sign << 3 | index into the
// grid above; one E8M0 byte (k + 127) per group.
//
// Design.  HBM-bound streaming kernels (4 bytes per element for the
// quantize-dequantize, 2.53 for the packer).  A thread owns 8 consecutive elements
// (one 128-bit load), four adjacent lanes own a group: the group maximum is a
// per-halfword unsigned integer maximum of the magnitudes (three SIMD
// instructions per thread) and two quad shuffles; rounding to the grid is one
// add and one subtract of a magic constant chosen by the magnitude's binade.
// The fp16 packer does this in half2 arithmetic and reads the 3-bit grid index
// straight out of the sum's mantissa (pack8_half).
#include <cuda_bf16.h>

#include <algorithm>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;  // 128-bit loads per thread in flight

template <bool BF16>
__device__ __forceinline__ float2 to_float2(uint32_t w) {
  if (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  return __half22float2(u32_as_half2(w));
}
template <bool BF16>
__device__ __forceinline__ uint32_t from_float2(float a, float b) {
  if (BF16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  return half2_as_u32(__floats2half2_rn(a, b));
}

// exponent k of the group's scale from the largest magnitude (16 bits of T, sign
// clear): a quarter of the mantissa range added, the exponent field kept; a field
// of 0 (zero or small denormal maximum: undefined in the reference) counts as 1
template <bool BF16>
__device__ __forceinline__ int scale_exponent(uint32_t max_bits) {
  constexpr int M = BF16 ? 7 : 10, B = BF16 ? 127 : 15;
  const int field = max((int)((max_bits + (1u << (M - 2))) >> M), 1);
  return max(-127, min(field - B - 2, 127));
}
// 2^k for k in [-127, 127] (2^-127 is an fp32 denormal)
__device__ __forceinline__ float pow2i(int k) {
  return k > -127 ? __uint_as_float((uint32_t)(k + 127) << 23) : __uint_as_float(0x00200000u);
}

// |v| scaled into the e2m1 range -> the grid value, ties to even, saturating at 6
__device__ __forceinline__ float to_grid(float a) {
  // grid step .5 below 2, 1 below 4, 2 above: adding 1.5 * 2^(23 + log2 step) and
  // taking it away again rounds to that step, ties to even
  const float c = a < 2.f ? 6291456.f : (a < 4.f ? 12582912.f : 25165824.f);
  return fminf((a + c) - c, 6.f);
}
// grid value -> index 0..7 into {0, .5, 1, 1.5, 2, 3, 4, 6}: from 1 on the index
// is (exponent - 126) * 2 + mantissa bit = the fp32 pattern >> 22, less 252; .5 is
// e2m1's one denormal (index 1) and 0 is 0
__device__ __forceinline__ uint32_t grid_index(float q) {
  const uint32_t b = __float_as_uint(q);
  return (uint32_t)max((int)(b >> 22) - 252, (int)min(b, 1u));
}

// The packer for fp16 inputs, two elements per instruction in half2 arithmetic.
// |x| / 2^k is two exact multiplications (2^-k alone can leave fp16's range);
// adding 768, 1538 or 3080 - by the binade of the scaled magnitude - rounds to the
// grid's step there (.5, 1, 2), ties to even, and the offsets 0, 2 and 8 folded
// into those constants make the low three mantissa bits of the sum the grid
// index itself: 768 + r has mantissa 512 + 2r, 1538 + r has 514 + r, 3080 + r has
// 516 + r / 2.  Returns the four bytes of 8 elements.
__device__ __forceinline__ uint32_t pack8_half(const uint4& v, int k) {
  const int k1 = k >> 1, k2 = k - k1;  // both in [-8, 7]
  const uint32_t b1 = (uint32_t)(15 - k1) << 10, b2 = (uint32_t)(15 - k2) << 10;
  const __half2 s1 = u32_as_half2(b1 | (b1 << 16)), s2 = u32_as_half2(b2 | (b2 << 16));
  const __half2 six = __float2half2_rn(6.f), k1024 = __float2half2_rn(1024.f),
                k512 = __float2half2_rn(512.f), m2047 = __float2half2_rn(-2047.f),
                c0 = __float2half2_rn(768.f),
                d1 = __float2half2_rn(770.f), d2 = __float2half2_rn(1542.f);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t m[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    __half2 a = __hmul2(__hmul2(u32_as_half2(w[j] & 0x7fff7fffu), s1), s2);
    a = __hmin2(a, six);
    // 1 from 2 (from 4) on, else 0: a saturating fused multiply-add on the
    // fp16 pipe, exact at the boundary (fp16 neighbours of 2 and 4 are 2^-10 and
    // 2^-9 below them)
    const __half2 ge2 = __hfma2_sat(a, k1024, m2047), ge4 = __hfma2_sat(a, k512, m2047);
    __half2 c = __hfma2(ge2, d1, c0);   // 768, or 1538 from 2 on
    c = __hfma2(ge4, d2, c);            // 3080 from 4 on
    const uint32_t n = (half2_as_u32(__hadd2(a, c)) & 0x00070007u) | ((w[j] >> 12) & 0x00080008u);
    m[j] = n | (n >> 12);  // byte 0: element 2j in the low nibble, 2j + 1 in the high one
  }
  return __byte_perm(__byte_perm(m[0], m[1], 0x0040), __byte_perm(m[2], m[3], 0x0040), 0x5410);
}

// the group maximum of the magnitudes as 16 bits of T: this thread's 8 elements,
// then the quad
__device__ __forceinline__ uint32_t quad_max(const uint4& v) {
  const uint32_t m01 = __vmaxu2(v.x & 0x7fff7fffu, v.y & 0x7fff7fffu);
  const uint32_t m23 = __vmaxu2(v.z & 0x7fff7fffu, v.w & 0x7fff7fffu);
  const uint32_t m = __vmaxu2(m01, m23);
  uint32_t mx = max(m & 0xffffu, m >> 16);
  mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  return mx;
}

// MODE 0: out = quantize-dequantize of in (type T); MODE 1: codes + scales
template <bool BF16, int MODE>
__global__ void __launch_bounds__(kThreads)
mxfp4_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, uint32_t* __restrict__ codes,
             uint8_t* __restrict__ scales, size_t nvec) {
  // nvec (8-element vectors) is a multiple of 4 and so is every thread's index
  // distance to its quad's first lane: a quad is inside or outside as a whole
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
  const size_t rounds = (nvec + stride * kUnroll - 1) / (stride * kUnroll);
  for (size_t r = 0; r < rounds; r++) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {  // all loads of the round before any arithmetic
      const size_t i = first + (r * kUnroll + u) * stride;
      v[u] = make_uint4(0, 0, 0, 0);
      if (i < nvec && HQ_IN_BOUNDS(in + i, 16, in, nvec * 16, 601)) v[u] = ldg_stream_u4(in + i);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const size_t i = first + (r * kUnroll + u) * stride;
      const int k = scale_exponent<BF16>(quad_max(v[u]));  // shuffles: every lane takes part
      const float inv = pow2i(-k), scale = pow2i(k);
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
      uint32_t o[4];
      uint32_t packed = 0;
      if (MODE == 1 && !BF16) packed = pack8_half(v[u], k);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (MODE == 1 && !BF16) break;
        const float2 f = to_float2<BF16>(w[j]);
        const float q0 = to_grid(fabsf(f.x) * inv), q1 = to_grid(fabsf(f.y) * inv);
        if (MODE == 0) {
          o[j] = from_float2<BF16>(copysignf(q0 * scale, f.x), copysignf(q1 * scale, f.y));
        } else {
          const uint32_t s0 = (w[j] >> 12) & 8u, s1 = (w[j] >> 28) & 8u;  // the sign bits
          packed |= ((grid_index(q0) | s0) | ((grid_index(q1) | s1) << 4)) << (8 * j);
        }
      }
      if (i >= nvec) continue;
      if (MODE == 0) {
        if (HQ_IN_BOUNDS(out + i, 16, out, nvec * 16, 602))
          out[i] = make_uint4(o[0], o[1], o[2], o[3]);
      } else {
        if (HQ_IN_BOUNDS(codes + i, 4, codes, nvec * 4, 603)) codes[i] = packed;
        if ((i & 3) == 0 && HQ_IN_BOUNDS(scales + (i >> 2), 1, scales, nvec / 4, 604))
          scales[i >> 2] = (uint8_t)(k + 127);
      }
    }
  }
}

// codes + scales -> T
template <bool BF16>
__global__ void __launch_bounds__(kThreads)
mxfp4_dequant_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                     uint4* __restrict__ out, size_t nvec) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride) {
    if (!HQ_IN_BOUNDS(codes + i, 4, codes, nvec * 4, 605) ||
        !HQ_IN_BOUNDS(scales + (i >> 2), 1, scales, nvec / 4, 606))
      continue;
    const uint32_t c = ldg_stream_u32(codes + i);
    const float scale = pow2i((int)__ldg(scales + (i >> 2)) - 127);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float q[2];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const uint32_t n = (c >> (8 * j + 4 * h)) & 15u, idx = n & 7u;
        // {0, .5, 1, 1.5} then 2^(idx/2 - 1) * (1 + idx % 2 / 2): 2, 3, 4, 6
        const float mag = idx < 4u ? 0.5f * (float)idx
                                   : (float)(1u << ((idx >> 1) - 1)) * (1.f + 0.5f * (float)(idx & 1u));
        q[h] = (n & 8u) ? -mag * scale : mag * scale;
      }
      o[j] = from_float2<BF16>(q[0], q[1]);
    }
    if (HQ_IN_BOUNDS(out + i, 16, out, nvec * 16, 607)) out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

int grid_for(size_t nvec) {
  const size_t want = (nvec + kThreads - 1) / kThreads;
  return (int)std::min<size_t>(want, (size_t)sm_count() * 8);
}

int check_args(const void* a, const void* b, size_t numel, int dtype) {
  if (dtype != HQ_DTYPE_F16 && dtype != HQ_DTYPE_BF16) return HQ_ERR_UNSUPPORTED;
  if (numel % 32 != 0) return HQ_ERR_BAD_SHAPE;
  if (numel && (!a || !b)) return HQ_ERR_NULL_POINTER;
  return HQ_OK;
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_mxfp4_qdq(const void* in, void* out, size_t numel, int dtype, hq_stream_t stream) {
  using namespace hq;
  const int rc = check_args(in, out, numel, dtype);
  if (rc != HQ_OK || numel == 0) return rc;
  if (!aligned16(in) || !aligned16(out)) return HQ_ERR_MISALIGNED;
  const size_t nvec = numel / 8;
  auto* i4 = reinterpret_cast<const uint4*>(in);
  auto* o4 = reinterpret_cast<uint4*>(out);
  if (dtype == HQ_DTYPE_BF16)
    mxfp4_kernel<true, 0><<<grid_for(nvec), kThreads, 0, (cudaStream_t)stream>>>(i4, o4, nullptr,
                                                                                 nullptr, nvec);
  else
    mxfp4_kernel<false, 0><<<grid_for(nvec), kThreads, 0, (cudaStream_t)stream>>>(i4, o4, nullptr,
                                                                                  nullptr, nvec);
  return launch_status();
}

int hq_mxfp4_quantize(const void* in, uint8_t* codes, uint8_t* scales_e8m0, size_t numel, int dtype,
                      hq_stream_t stream) {
  using namespace hq;
  const int rc = check_args(in, codes, numel, dtype);
  if (rc != HQ_OK || numel == 0) return rc;
  if (!scales_e8m0) return HQ_ERR_NULL_POINTER;
  if (!aligned16(in) || !aligned4(codes)) return HQ_ERR_MISALIGNED;
  const size_t nvec = numel / 8;
  auto* i4 = reinterpret_cast<const uint4*>(in);
  auto* c4 = reinterpret_cast<uint32_t*>(codes);
  if (dtype == HQ_DTYPE_BF16)
    mxfp4_kernel<true, 1><<<grid_for(nvec), kThreads, 0, (cudaStream_t)stream>>>(i4, nullptr, c4,
                                                                                 scales_e8m0, nvec);
  else
    mxfp4_kernel<false, 1><<<grid_for(nvec), kThreads, 0, (cudaStream_t)stream>>>(i4, nullptr, c4,
                                                                                  scales_e8m0, nvec);
  return launch_status();
}

int hq_mxfp4_dequantize(const uint8_t* codes, const uint8_t* scales_e8m0, void* out, size_t numel,
                        int dtype, hq_stream_t stream) {
  using namespace hq;
  const int rc = check_args(codes, out, numel, dtype);
  if (rc != HQ_OK || numel == 0) return rc;
  if (!scales_e8m0) return HQ_ERR_NULL_POINTER;
  if (!aligned4(codes) || !aligned16(out)) return HQ_ERR_MISALIGNED;
  const size_t nvec = numel / 8;
  auto* c4 = reinterpret_cast<const uint32_t*>(codes);
  auto* o4 = reinterpret_cast<uint4*>(out);
  if (dtype == HQ_DTYPE_BF16)
    mxfp4_dequant_kernel<true><<<grid_for(nvec), kThreads, 0, (cudaStream_t)stream>>>(
        c4, scales_e8m0, o4, nvec);
  else
    mxfp4_dequant_kernel<false><<<grid_for(nvec), kThreads, 0, (cudaStream_t)stream>>>(
        c4, scales_e8m0, o4, nvec);
  return launch_status();
}

}  // extern "C"
