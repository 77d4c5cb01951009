// Shared pieces of the row-streaming mat-vec kernels (gemv_uniform.cu,
// gemv_fused.cu): a warp owns whole rows, the input vector sits piece-major in
// shared memory, 16 bytes of weights per lane and load.
#ifndef HQ_GEMV_ROWS_CUH_
#define HQ_GEMV_ROWS_CUH_
#include "hq_common.cuh"

namespace hq {
namespace rows {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kInFlight = 8;            // 16-byte loads per lane in flight
constexpr int kRows = 2;                // adjacent rows a warp works on at a time
__device__ __forceinline__ float sum4(__half2 a0, __half2 a1, __half2 a2, __half2 a3) {
  const float2 f = __half22float2(__hadd2(__hadd2(a0, a1), __hadd2(a2, a3)));
  return f.x + f.y;
}

// 16 bytes of weights of each of R rows against the matching inputs -> one fp32
// partial sum per row; the inputs are read once for the R rows.
// BITS = 16: 8 halves x 8 inputs; 8: 16 int8 x 16 inputs; 4: 32 nibbles x 32 inputs.
// xs points at the chunk's first 16-byte piece of inputs; its further pieces
// follow at a distance of `pitch` pieces (the inputs are stored piece-major so
// that the 32 lanes of a warp, which hold consecutive chunks, read consecutive
// 16-byte words: chunk-major, a chunk's 32 or 64 bytes apart, they would meet in
// the same banks two or four at a time).
template <int BITS, int R>
__device__ __forceinline__ void chunk_dot(const uint4 (&w)[R], const uint4* xs, int pitch,
                                          float (&part)[R]) {
  if (BITS == 16) {
    const uint4 x = xs[0];
#pragma unroll
    for (int r = 0; r < R; r++) {
      // one product per accumulator: summed in fp32 right away
      const float2 f0 = __half22float2(__hmul2(u32_as_half2(w[r].x), u32_as_half2(x.x))),
                   f1 = __half22float2(__hmul2(u32_as_half2(w[r].y), u32_as_half2(x.y))),
                   f2 = __half22float2(__hmul2(u32_as_half2(w[r].z), u32_as_half2(x.z))),
                   f3 = __half22float2(__hmul2(u32_as_half2(w[r].w), u32_as_half2(x.w)));
      part[r] = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
    }
  } else if (BITS == 8) {
    const uint4 xa = xs[0], xb = xs[pitch];
    const uint32_t x2[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
    const __half2 off = __float2half2_rn(1152.f);  // 1024 (exponent byte) + 128 (sign flip)
#pragma unroll
    for (int r = 0; r < R; r++) {
      const uint32_t ww[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
      __half2 a0 = __float2half2_rn(0.f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint32_t t = ww[i] ^ 0x80808080u;
        const __half2 lo = __hsub2(u32_as_half2(__byte_perm(t, 0x64646464u, 0x4140)), off);
        const __half2 hi = __hsub2(u32_as_half2(__byte_perm(t, 0x64646464u, 0x4342)), off);
        if (i & 1) {
          a2 = __hfma2(lo, u32_as_half2(x2[2 * i]), a2);
          a3 = __hfma2(hi, u32_as_half2(x2[2 * i + 1]), a3);
        } else {
          a0 = __hfma2(lo, u32_as_half2(x2[2 * i]), a0);
          a1 = __hfma2(hi, u32_as_half2(x2[2 * i + 1]), a1);
        }
      }
      part[r] = sum4(a0, a1, a2, a3);
    }
  } else {
    // A word holds 8 nibbles = elements 0 .. 7.  (w & 0x000f000f) | 0x64006400 is
    // half2(1024 + e0, 1024 + e4), (w & 0x00f000f0) | 0x64006400 is half2(1024 +
    // 16 e1, 1024 + 16 e5); w >> 8 brings e2, e6 and e3, e7 to the same places.
    // One subtraction of 1024, or one fused x / 16 - 64, leaves the integers,
    // exactly: two logic operations and one fp16 instruction per two weights, no
    // table.  The inputs are staged in the matching order (pair_inputs).
    const __half2 k1024 = __float2half2_rn(1024.f), k16th = __float2half2_rn(0.0625f),
                  km64 = __float2half2_rn(-64.f);
    __half2 a[R][4];
#pragma unroll
    for (int r = 0; r < R; r++) a[r][0] = a[r][1] = a[r][2] = a[r][3] = __float2half2_rn(0.f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 x = xs[i * pitch];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const uint32_t wi = i == 0 ? w[r].x : i == 1 ? w[r].y : i == 2 ? w[r].z : w[r].w;
        const uint32_t hi = wi >> 8;
        const __half2 e04 = __hsub2(u32_as_half2((wi & 0x000f000fu) | 0x64006400u), k1024);
        const __half2 e15 = __hfma2(u32_as_half2((wi & 0x00f000f0u) | 0x64006400u), k16th, km64);
        const __half2 e26 = __hsub2(u32_as_half2((hi & 0x000f000fu) | 0x64006400u), k1024);
        const __half2 e37 = __hfma2(u32_as_half2((hi & 0x00f000f0u) | 0x64006400u), k16th, km64);
        a[r][0] = __hfma2(e04, u32_as_half2(x.x), a[r][0]);
        a[r][1] = __hfma2(e15, u32_as_half2(x.y), a[r][1]);
        a[r][2] = __hfma2(e26, u32_as_half2(x.z), a[r][2]);
        a[r][3] = __hfma2(e37, u32_as_half2(x.w), a[r][3]);
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) part[r] = sum4(a[r][0], a[r][1], a[r][2], a[r][3]);
  }
}

// 8 consecutive inputs (x0,x1)(x2,x3)(x4,x5)(x6,x7) in the order the 4-bit
// conversion above produces its weights: (x0,x4)(x1,x5)(x2,x6)(x3,x7)
__device__ __forceinline__ uint4 pair_inputs(const uint4& v) {
  return make_uint4(__byte_perm(v.x, v.z, 0x5410), __byte_perm(v.x, v.z, 0x7632),
                    __byte_perm(v.y, v.w, 0x5410), __byte_perm(v.y, v.w, 0x7632));
}

}  // namespace rows
}  // namespace hq
#endif  // HQ_GEMV_ROWS_CUH_
