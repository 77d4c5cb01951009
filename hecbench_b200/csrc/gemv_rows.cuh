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
constexpr int kLutImm = 2048;           // shared-window address of the int4 table
constexpr int kLutBytes = 256 * 256;    // 256 rows of 256 bytes (first 128: one copy per bank)

template <int IMM>
__device__ __forceinline__ uint32_t lds_u32_imm(uint32_t addr) {
  uint32_t v;  // not volatile: the table is constant after the prologue barrier
  asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
  return v;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
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
                                          uint32_t lane4, float (&part)[R]) {
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
    __half2 a[R][4];
#pragma unroll
    for (int r = 0; r < R; r++) a[r][0] = a[r][1] = a[r][2] = a[r][3] = __float2half2_rn(0.f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 x = xs[i * pitch];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const uint32_t wi = i == 0 ? w[r].x : i == 1 ? w[r].y : i == 2 ? w[r].z : w[r].w;
        // byte k of the word -> (byte << 8) | lane*4: bytes {lane4.0, w.k, 0, 0}
        const uint32_t l0 = lds_u32_imm<kLutImm>(__byte_perm(wi, lane4, 0x7604));
        const uint32_t l1 = lds_u32_imm<kLutImm>(__byte_perm(wi, lane4, 0x7614));
        const uint32_t l2 = lds_u32_imm<kLutImm>(__byte_perm(wi, lane4, 0x7624));
        const uint32_t l3 = lds_u32_imm<kLutImm>(__byte_perm(wi, lane4, 0x7634));
        a[r][0] = __hfma2(u32_as_half2(l0), u32_as_half2(x.x), a[r][0]);
        a[r][1] = __hfma2(u32_as_half2(l1), u32_as_half2(x.y), a[r][1]);
        a[r][2] = __hfma2(u32_as_half2(l2), u32_as_half2(x.z), a[r][2]);
        a[r][3] = __hfma2(u32_as_half2(l3), u32_as_half2(x.w), a[r][3]);
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) part[r] = sum4(a[r][0], a[r][1], a[r][2], a[r][3]);
  }
}


// The 256-row byte table of the 4-bit formats: row b (256 bytes apart, 32 copies
// of one word in its first 128 bytes, one per bank) holds half2(first element,
// second element) of byte b.  level_of(k) = the value code k stands for;
// low_first: element 2j is the low nibble of byte j (else the high nibble).
template <class LevelOf>
__device__ __forceinline__ void build_nibble_table(unsigned char* lut, LevelOf level_of,
                                                    bool low_first, int tid, int nthreads) {
  for (int e4 = tid; e4 < 256 * 4; e4 += nthreads) {
    const int entry = e4 >> 2, quarter = e4 & 3;  // four threads per 128-byte table row
    const int lo = entry & 15, hi = entry >> 4;
    const float first = level_of(low_first ? lo : hi), second = level_of(low_first ? hi : lo);
    const uint32_t u = half2_as_u32(__floats2half2_rn(first, second));
    const uint4 u4 = make_uint4(u, u, u, u);
    uint4* row = reinterpret_cast<uint4*>(lut + (size_t)entry * 256 + quarter * 32);
    row[0] = u4;
    row[1] = u4;
  }
}

}  // namespace rows
}  // namespace hq
#endif  // HQ_GEMV_ROWS_CUH_
