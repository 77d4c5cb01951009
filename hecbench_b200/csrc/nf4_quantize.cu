// Blockwise 4-bit quantizer for sm_100a: fp16 / bf16 / fp32 weights -> the packed
// codes and per-block absmax that hq_nf4_dequant_f16, hq_nf4_gemv_f16 and
// hq_qgemm_nf4_f16 consume.  The inverse of those kernels' dequantisation; the
// reference tree has no blockwise 4-bit quantizer (its quantBnB benchmark is the
// 8-bit, whole-tensor kQuantize), so the rule is stated here:
//   absmax[b] = max |w| over block b (fp32)
//   x         = fp32(w) * (1 / absmax[b])          (0 where absmax is 0, denormal or infinite)
//   code      = number of the 15 midpoints m_j = (lut16[j] + lut16[j+1]) / 2 (fp32)
//               that are < x: the nearest level, a tie going to the lower one
// with lut16 the 16 ascending levels, and two codes per byte in the nibble order
// of the flags (default: even element in the high nibble).
//
// Design.  HBM-bound stream (2.56 bytes per fp16 weight with blocks of 64).  A
// thread owns 8 consecutive weights (one or two 128-bit loads, one 32-bit
// store); blocks of up to 256 weights live in the lanes of one warp and their
// absmax is a shuffle tree, larger blocks are walked twice by one warp (the
// second pass reads L1/L2).  The nearest level is NOT searched: the interval
// [-1 - 1/32, 1 + 1/32) is cut into 66 cells of width 1/32, and a table built per
// CTA (one copy per bank, as the byte tables of the mat-vec kernels) holds for
// each cell the number of midpoints below it and the one midpoint inside it, so
// code = count + (x > midpoint): one multiply, one floor, one 64-bit
// shared-memory read, one compare.  A level table with two midpoints in one cell
// (levels closer than 1/32) makes the CTA count midpoints one by one instead.
#include <cuda_bf16.h>

#include <algorithm>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;           // 8-weight vectors per thread in flight
constexpr int kCells = 66;          // cell c covers [(c - 33) / 32, (c - 32) / 32)
constexpr int kCellStride = 256;    // bytes between cells: 32 lanes x 8 bytes

// loads 8 consecutive weights as fp32
template <int DTYPE>
__device__ __forceinline__ void load8(const void* base, size_t vec, size_t nvec, float (&w)[8]) {
  if (DTYPE == HQ_DTYPE_F32) {
    const uint4* p = reinterpret_cast<const uint4*>(base) + 2 * vec;
    uint4 a = make_uint4(0, 0, 0, 0), b = a;
    if (HQ_IN_BOUNDS(p, 32, base, nvec * 32, 801)) {
      a = ldg_stream_u4(p);
      b = ldg_stream_u4(p + 1);
    }
    w[0] = __uint_as_float(a.x); w[1] = __uint_as_float(a.y);
    w[2] = __uint_as_float(a.z); w[3] = __uint_as_float(a.w);
    w[4] = __uint_as_float(b.x); w[5] = __uint_as_float(b.y);
    w[6] = __uint_as_float(b.z); w[7] = __uint_as_float(b.w);
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(base) + vec;
    uint4 a = make_uint4(0, 0, 0, 0);
    if (HQ_IN_BOUNDS(p, 16, base, nvec * 16, 802)) a = ldg_stream_u4(p);
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

__device__ __forceinline__ float max_abs8(const float (&w)[8]) {
  float m = fabsf(w[0]);
#pragma unroll
  for (int j = 1; j < 8; j++) m = fmaxf(m, fabsf(w[j]));
  return m;
}

// 1 / absmax, or 0 where that is not a finite number (absmax zero, denormal,
// infinite): such a block quantizes to the code of 0
__device__ __forceinline__ float block_inverse(float m) {
  return (m >= 1.17549435e-38f && m <= 3.40282347e38f) ? 1.f / m : 0.f;
}

// codes of 8 weights scaled by inv, packed into one word (byte j = elements 2j, 2j + 1)
template <bool DENSE>
__device__ __forceinline__ uint32_t encode8(const float (&w)[8], float inv, const unsigned char* cells,
                                            const float* mids, int lane, bool low_first) {
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float x = w[j] * inv;
    uint32_t code;
    if (DENSE) {
      code = 0;
#pragma unroll
      for (int k = 0; k < 15; k++) code += x > mids[k] ? 1u : 0u;
    } else {
      // x * 32 is exact, so is the cell.  |x| <= 1 + 2^-23 or x is not a number
      // (which converts to 0): floor(x * 32) lies in -33 .. 32 without a clamp
      const int cell = __float2int_rd(x * 32.f);
      const float2 e = *reinterpret_cast<const float2*>(cells + (cell + 33) * kCellStride + lane * 8);
      code = __float_as_uint(e.x) + (x > e.y ? 1u : 0u);
    }
    const bool high = ((j & 1) == 0) != low_first;  // even element: high nibble by default
    word |= code << (8 * (j >> 1) + (high ? 4 : 0));
  }
  return word;
}

// LPB: lanes per block (blocksize / 8) for blocks inside a warp, 0: a warp walks
// a whole block of `blocksize` weights twice
template <int DTYPE, int LPB>
__global__ void __launch_bounds__(kThreads)
nf4_quantize_kernel(const void* __restrict__ W, size_t nvec, int blocksize,
                    const float* __restrict__ lut16, int low_first, uint32_t* __restrict__ B,
                    float* __restrict__ absmax) {
  __shared__ __align__(16) unsigned char s_cells[kCells * kCellStride];
  __shared__ float s_mid[16];
  __shared__ float2 s_cell[kCells];
  __shared__ int s_dense;
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid < 15) s_mid[tid] = 0.5f * (__ldg(lut16 + tid) + __ldg(lut16 + tid + 1));
  if (tid == 0) s_dense = 0;
  __syncthreads();
  for (int c = tid; c < kCells; c += kThreads) {
    const float lo = (float)(c - 33) * 0.03125f, hi = (float)(c - 32) * 0.03125f;
    uint32_t below = 0, inside = 0;
    float mid = __int_as_float(0x7f800000);  // no midpoint inside: x > +inf never holds
    for (int k = 0; k < 15; k++) {
      const float m = s_mid[k];
      if (m < lo) below++;
      else if (m < hi) { inside++; mid = m; }
    }
    if (inside > 1) s_dense = 1;
    s_cell[c] = make_float2(__uint_as_float(below), mid);
  }
  __syncthreads();
  // one copy per bank, written by all threads
  for (int i = tid; i < kCells * 32; i += kThreads)
    *reinterpret_cast<float2*>(s_cells + (i >> 5) * kCellStride + (i & 31) * 8) = s_cell[i >> 5];
  __syncthreads();
  const bool dense = s_dense != 0;
  const bool lf = low_first != 0;

  if (LPB > 0) {
    // nvec is a multiple of LPB and so is the distance of a thread to the first
    // lane of its block: the lanes of a block are inside or outside together
    const size_t stride = (size_t)gridDim.x * kThreads;
    const size_t first = (size_t)blockIdx.x * kThreads + tid;
    const size_t rounds = (nvec + stride * kUnroll - 1) / (stride * kUnroll);
    for (size_t r = 0; r < rounds; r++) {
      float w[kUnroll][8];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {  // all loads of the round before any arithmetic
        const size_t v = first + (r * kUnroll + u) * stride;
        if (v < nvec) load8<DTYPE>(W, v, nvec, w[u]);
        else {
#pragma unroll
          for (int j = 0; j < 8; j++) w[u][j] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const size_t v = first + (r * kUnroll + u) * stride;
        float m = max_abs8(w[u]);
#pragma unroll
        for (int d = 1; d < LPB; d <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        const float inv = block_inverse(m);
        const uint32_t word = dense ? encode8<true>(w[u], inv, s_cells, s_mid, lane, lf)
                                    : encode8<false>(w[u], inv, s_cells, s_mid, lane, lf);
        if (v >= nvec) continue;
        if (HQ_IN_BOUNDS(B + v, 4, B, nvec * 4, 803)) B[v] = word;
        if ((v % LPB) == 0 && HQ_IN_BOUNDS(absmax + v / LPB, 4, absmax, nvec / LPB * 4, 804))
          absmax[v / LPB] = m;
      }
    }
  } else {
    const int vpb = blocksize / 8;  // vectors per block, a multiple of 32
    const size_t nblocks = nvec / vpb;
    const size_t warps = (size_t)gridDim.x * (kThreads / 32);
    for (size_t b = (size_t)blockIdx.x * (kThreads / 32) + (tid >> 5); b < nblocks; b += warps) {
      float m = 0.f;
      for (int i = lane; i < vpb; i += 32) {
        float w[8];
        load8<DTYPE>(W, b * vpb + i, nvec, w);
        m = fmaxf(m, max_abs8(w));
      }
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
      const float inv = block_inverse(m);
      for (int i = lane; i < vpb; i += 32) {
        float w[8];
        const size_t v = b * vpb + i;
        load8<DTYPE>(W, v, nvec, w);
        const uint32_t word = dense ? encode8<true>(w, inv, s_cells, s_mid, lane, lf)
                                    : encode8<false>(w, inv, s_cells, s_mid, lane, lf);
        if (HQ_IN_BOUNDS(B + v, 4, B, nvec * 4, 805)) B[v] = word;
      }
      if (lane == 0 && HQ_IN_BOUNDS(absmax + b, 4, absmax, nblocks * 4, 806)) absmax[b] = m;
    }
  }
}

template <int DTYPE>
int launch(const void* W, size_t n, int blocksize, const float* lut16, int flags, uint8_t* B,
           float* absmax, cudaStream_t st) {
  const size_t nvec = n / 8;
  const int low = (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0;
  auto* b32 = reinterpret_cast<uint32_t*>(B);
  const size_t want = (nvec + kThreads - 1) / kThreads;
  // every CTA builds the table once: no more CTAs than are resident together
  const int grid = (int)std::min<size_t>(want, (size_t)sm_count() * 4);
#define HQ_GO(LPB_)                                                                          \
  nf4_quantize_kernel<DTYPE, LPB_><<<grid, kThreads, 0, st>>>(W, nvec, blocksize, lut16, low, b32, \
                                                              absmax)
  switch (blocksize) {
    case 32: HQ_GO(4); break;
    case 64: HQ_GO(8); break;
    case 128: HQ_GO(16); break;
    case 256: HQ_GO(32); break;
    default: HQ_GO(0); break;
  }
#undef HQ_GO
  return launch_status();
}

}  // namespace
}  // namespace hq

extern "C" int hq_nf4_quantize(const void* W, int dtype, size_t n, int blocksize,
                               const float* lut16, int flags, uint8_t* B, float* absmax,
                               hq_stream_t stream) {
  using namespace hq;
  if (blocksize < 32 || blocksize > 4096 || (blocksize & (blocksize - 1)) != 0)
    return HQ_ERR_BAD_SHAPE;
  if (n % (size_t)blocksize != 0) return HQ_ERR_BAD_SHAPE;
  if (!lut16) return HQ_ERR_NULL_POINTER;
  if (n == 0) return HQ_OK;
  if (!W || !B || !absmax) return HQ_ERR_NULL_POINTER;
  if (!aligned16(W) || !aligned4(B)) return HQ_ERR_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HQ_DTYPE_F16: return launch<HQ_DTYPE_F16>(W, n, blocksize, lut16, flags, B, absmax, st);
    case HQ_DTYPE_BF16: return launch<HQ_DTYPE_BF16>(W, n, blocksize, lut16, flags, B, absmax, st);
    case HQ_DTYPE_F32: return launch<HQ_DTYPE_F32>(W, n, blocksize, lut16, flags, B, absmax, st);
    default: return HQ_ERR_UNSUPPORTED;
  }
}
