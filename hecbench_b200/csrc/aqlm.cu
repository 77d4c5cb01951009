// AQLM additive-codebook mat-vec for sm_100a: 1x16 (one 65536-entry codebook,
// uint16 codes) and 2x8 (two 256-entry codebooks, uint8 codes).
//
// 1x16 follows the arithmetic of Code1x16MatVec (quantAQLM-cuda/main.cu:31-111)
// exactly - lane l of a row's warp takes the 16-byte code vectors l, l+32, ...;
// each code gathers a 16-byte codebook row, four hfma2 against the matching
// 8 inputs, the two halves are added to the lane's fp32 sum, lanes are combined
// with the shfl_down tree - so results are bit-identical to the reference
// kernel.  What changes is the memory behaviour: all code vectors of a row and
// all their 16-byte gathers are issued before any arithmetic (up to 16 gathers
// in flight per lane instead of 1), a warp walks several rows, and the 1 MiB
// codebook is read through the read-only path so that it stays L2-resident
// while the codes stream past it without allocating in L1.
//
// 2x8: both codebooks (8 KiB) live in shared memory, replicated 8 times with
// entry e of replica r at 16-byte slot 8*e + r, so the 8 lanes that a 128-bit
// shared load serves per cycle (r = lane % 8) always hit distinct bank groups.
#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kWarps1x16 = 8;
// Rows per warp: 4 when that still gives every SM two CTAs, else 2 (a 4096-row
// layer is latency-bound: more resident warps pay more than the per-CTA staging
// of the inputs costs: 12.5 -> 11.0 us for 1x16, 11.5 -> 8.0 us for 2x8).
inline int rows_per_warp_for(int prob_m, int warps) {
  return prob_m / (warps * 4) >= 2 * sm_count() ? 4 : 2;
}
constexpr int kPad = 9;  // input slots per 8 groups (one pad slot: conflict-free 128-bit reads)

__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float dot8_ref_order(const uint4& a, const uint4& b) {
  // res2 = hfma2(a[j], b[j], res2), j = 0..3, from zero; float(res2.x) + float(res2.y)
  __half2 r = __float2half2_rn(0.f);
  r = __hfma2(u32_as_half2(a.x), u32_as_half2(b.x), r);
  r = __hfma2(u32_as_half2(a.y), u32_as_half2(b.y), r);
  r = __hfma2(u32_as_half2(a.z), u32_as_half2(b.z), r);
  r = __hfma2(u32_as_half2(a.w), u32_as_half2(b.w), r);
  return __half2float(__low2half(r)) + __half2float(__high2half(r));
}

// VPL = 16-byte code vectors per lane per row (prob_k / 64 / 32 rounded up),
// RPW = rows per warp.  The dependent chain code -> codebook row -> FMA is what
// bounds this kernel, so everything that does not depend on the input vector
// is issued first: the code vectors of ALL rows of the warp, then the gathers
// of the first vector, and only then the CTA stages the inputs in shared
// memory; afterwards the gathers of vector u + 1 are in flight while vector u
// is multiplied.  The arithmetic (and its order) is the reference's.
template <int VPL, int RPW>
__global__ void __launch_bounds__(kWarps1x16 * 32)
aqlm_1x16_kernel(const uint4* __restrict__ codes, const uint4* __restrict__ x,
                 __half* __restrict__ out, const uint4* __restrict__ codebook, int prob_m,
                 int prob_k, int4 cb_sizes, int cb_stride, const __half* __restrict__ scales) {
  extern __shared__ __align__(16) uint4 sh_x[];  // padded inputs: slot 9*(g/8) + g%8
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int groups = prob_k >> 3;    // 16-byte input groups
  const int vec_per_row = prob_k >> 6;
  const int row_begin = (blockIdx.x * kWarps1x16 + warp) * RPW;
  constexpr int kUnits = RPW * VPL;  // unit u = (row u / VPL, vector u % VPL)

  uint4 cv[kUnits];
#pragma unroll
  for (int u = 0; u < kUnits; u++) {
    const int m = row_begin + u / VPL, idx = lane + 32 * (u % VPL);
    cv[u] = (m < prob_m && idx < vec_per_row)
                ? ldg_stream_u4(codes + (size_t)m * vec_per_row + idx)
                : make_uint4(0, 0, 0, 0);
  }
  auto book = [&](int m) {
    const uint4* cb = codebook;
    if (m >= cb_sizes.x) cb += cb_stride;
    if (m >= cb_sizes.y) cb += cb_stride;
    if (m >= cb_sizes.z) cb += cb_stride;
    return cb;
  };
  auto gather = [&](int u, uint4 (&rows)[8]) {
    const int m = row_begin + u / VPL, idx = lane + 32 * (u % VPL);
    if (m < prob_m && idx < vec_per_row) {
      const uint4* cb = book(m);
      const uint32_t cw[4] = {cv[u].x, cv[u].y, cv[u].z, cv[u].w};
#pragma unroll
      for (int i = 0; i < 8; i++)
        rows[i] = ldg_nc_u4(cb + ((cw[i >> 1] >> (16 * (i & 1))) & 0xffffu));
    }
  };
  uint4 rows[2][8];
  gather(0, rows[0]);

  for (int g = tid; g < groups; g += blockDim.x) sh_x[kPad * (g >> 3) + (g & 7)] = x[g];
  __syncthreads();

  float res = 0.f;
#pragma unroll
  for (int u = 0; u < kUnits; u++) {
    if (u + 1 < kUnits) gather(u + 1, rows[(u + 1) & 1]);
    const int m = row_begin + u / VPL, idx = lane + 32 * (u % VPL);
    if (m < prob_m && idx < vec_per_row) {
#pragma unroll
      for (int i = 0; i < 8; i++) res += dot8_ref_order(rows[u & 1][i], sh_x[kPad * idx + i]);
    }
    if (u % VPL == VPL - 1) {  // the row is complete
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) res += __shfl_down_sync(0xffffffffu, res, o);
      if (lane == 0 && m < prob_m) {
        if (scales != nullptr) res *= __half2float(scales[m]);
        out[m] = __float2half(res);
      }
      res = 0.f;
    }
  }
}

constexpr int kWarps2x8 = 8;

__global__ void __launch_bounds__(kWarps2x8 * 32)
aqlm_2x8_kernel(const uint4* __restrict__ codes, const uint4* __restrict__ x,
                __half* __restrict__ out, const uint4* __restrict__ codebooks, int prob_m,
                int prob_k, const __half* __restrict__ scales, int rows_per_warp) {
  extern __shared__ __align__(16) uint4 smem4[];
  uint4* cbs = smem4;                  // [2][256][8 replicas]
  uint4* sh_x = smem4 + 2 * 256 * 8;   // padded inputs
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int groups = prob_k >> 3;
  const int vec_per_row = prob_k >> 6;  // 16 bytes = 8 groups x 2 codes
  for (int i = tid; i < 2 * 256 * 8; i += blockDim.x) cbs[i] = codebooks[i >> 3];
  for (int g = tid; g < groups; g += blockDim.x) sh_x[kPad * (g >> 3) + (g & 7)] = x[g];
  __syncthreads();

  const uint4* cb0 = cbs + (lane & 7);
  const uint4* cb1 = cbs + 256 * 8 + (lane & 7);
  const int row_begin = (blockIdx.x * kWarps2x8 + warp) * rows_per_warp;
  for (int rr = 0; rr < rows_per_warp; rr++) {
    const int m = row_begin + rr;
    if (m >= prob_m) break;
    const uint4* crow = codes + (size_t)m * vec_per_row;
    float res = 0.f;
    for (int idx = lane; idx < vec_per_row; idx += 32) {
      const uint4 cv = ldg_stream_u4(crow + idx);
      const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const uint32_t pair = (cw[i >> 1] >> (16 * (i & 1))) & 0xffffu;
        const uint4 a0 = cb0[(pair & 0xffu) * 8];
        const uint4 a1 = cb1[(pair >> 8) * 8];
        const uint4 b = sh_x[kPad * idx + i];
        __half2 r = __float2half2_rn(0.f);
        r = __hfma2(u32_as_half2(a0.x), u32_as_half2(b.x), r);
        r = __hfma2(u32_as_half2(a0.y), u32_as_half2(b.y), r);
        r = __hfma2(u32_as_half2(a0.z), u32_as_half2(b.z), r);
        r = __hfma2(u32_as_half2(a0.w), u32_as_half2(b.w), r);
        r = __hfma2(u32_as_half2(a1.x), u32_as_half2(b.x), r);
        r = __hfma2(u32_as_half2(a1.y), u32_as_half2(b.y), r);
        r = __hfma2(u32_as_half2(a1.z), u32_as_half2(b.z), r);
        r = __hfma2(u32_as_half2(a1.w), u32_as_half2(b.w), r);
        res += __half2float(__low2half(r)) + __half2float(__high2half(r));
      }
    }
    res = warp_sum(res);
    if (lane == 0) {
      if (scales != nullptr) res *= __half2float(scales[m]);
      out[m] = __float2half_rn(res);
    }
  }
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_aqlm_1x16_matvec(const void* codes, const void* x_half, void* out_half, const void* codebook,
                        int prob_m, int prob_k, const int cb_sizes[4], int cb_stride_int4,
                        const void* scales_half, hq_stream_t stream) {
  using namespace hq;
  if (!codes || !x_half || !out_half || !codebook || !cb_sizes) return HQ_ERR_NULL_POINTER;
  if (prob_m <= 0 || prob_k <= 0 || prob_k % 64 != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(codes) || !aligned16(x_half) || !aligned16(codebook)) return HQ_ERR_MISALIGNED;
  const int vec_per_row = prob_k / 64;
  const int vpl = (vec_per_row + 31) / 32;
  if (vpl > 4) return HQ_ERR_TOO_LARGE;  // prob_k <= 8192
  const int groups = prob_k / 8;
  const size_t smem = (size_t)kPad * ((groups + 7) / 8) * 16;
  const int rows_per_warp = rows_per_warp_for(prob_m, kWarps1x16);
  const int rows_per_cta = kWarps1x16 * rows_per_warp;
  const int grid = (prob_m + rows_per_cta - 1) / rows_per_cta;
  const int4 sizes = make_int4(cb_sizes[0], cb_sizes[1], cb_sizes[2], cb_sizes[3]);
  cudaStream_t st = (cudaStream_t)stream;
#define HQ_AQLM_LAUNCH(VPL, RPW)                                                             \
  {                                                                                          \
    constexpr auto kern = aqlm_1x16_kernel<VPL, RPW>;                                        \
    if (smem > 48 * 1024) {                                                                  \
      cudaError_t e = ensure_dynamic_smem<kern>(smem);                                       \
      if (e != cudaSuccess) return cuda_status(e);                                           \
    }                                                                                        \
    kern<<<grid, kWarps1x16 * 32, smem, st>>>(                                               \
        reinterpret_cast<const uint4*>(codes), reinterpret_cast<const uint4*>(x_half),       \
        reinterpret_cast<__half*>(out_half), reinterpret_cast<const uint4*>(codebook),       \
        prob_m, prob_k, sizes, cb_stride_int4, reinterpret_cast<const __half*>(scales_half)); \
  }
#define HQ_AQLM_ROWS(VPL)                                \
  if (rows_per_warp == 4) HQ_AQLM_LAUNCH(VPL, 4)         \
  else HQ_AQLM_LAUNCH(VPL, 2)
  switch (vpl) {
    case 1: HQ_AQLM_ROWS(1) break;
    case 2: HQ_AQLM_ROWS(2) break;
    case 3: HQ_AQLM_ROWS(3) break;
    default: HQ_AQLM_ROWS(4) break;
  }
#undef HQ_AQLM_ROWS
#undef HQ_AQLM_LAUNCH
  return launch_status();
}

int hq_aqlm_2x8_matvec(const void* codes, const void* x_half, void* out_half, const void* codebooks,
                       int prob_m, int prob_k, const void* scales_half, hq_stream_t stream) {
  using namespace hq;
  if (!codes || !x_half || !out_half || !codebooks) return HQ_ERR_NULL_POINTER;
  if (prob_m <= 0 || prob_k <= 0 || prob_k % 64 != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(codes) || !aligned16(x_half) || !aligned16(codebooks)) return HQ_ERR_MISALIGNED;
  const int groups = prob_k / 8;
  const size_t smem = (size_t)2 * 256 * 8 * 16 + (size_t)kPad * ((groups + 7) / 8) * 16;
  if (smem > 220 * 1024) return HQ_ERR_TOO_LARGE;
  constexpr auto kern2x8 = aqlm_2x8_kernel;
  cudaError_t e = ensure_dynamic_smem<kern2x8>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  const int rows_per_warp = rows_per_warp_for(prob_m, kWarps2x8);
  const int rows_per_cta = kWarps2x8 * rows_per_warp;
  const int grid = (prob_m + rows_per_cta - 1) / rows_per_cta;
  aqlm_2x8_kernel<<<grid, kWarps2x8 * 32, smem, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(codes), reinterpret_cast<const uint4*>(x_half),
      reinterpret_cast<__half*>(out_half), reinterpret_cast<const uint4*>(codebooks), prob_m,
      prob_k, reinterpret_cast<const __half*>(scales_half), rows_per_warp);
  return launch_status();
}

}  // extern "C"
