// NF4 blockwise 4-bit dequantize and batch-1 GEMV for sm_100a.
//
// Format: element e of the flattened [N][K] matrix has its 4-bit code in byte
// e/2 (even element = high nibble by default, low nibble with
// HQ_NF4_LOW_NIBBLE_FIRST); one fp32 absmax per `blocksize` consecutive
// elements; the 16 levels are a runtime fp32 table.
//   dequant : out[e] = half_rn(lut16[code] * absmax[e/blocksize])   (bit exact)
//   gemv    : out[n] = half_rn(sum_k A[k] * lut16[code[n][k]] * absmax[...])
//
// GEMV design (HBM-bound, 0.5 B of codes + 1/16 B of absmax per weight):
//  * a warp owns two rows at a time; a lane reads 16 bytes (32 codes) per row
//    per step, so the warp streams 512 contiguous bytes of each row;
//  * one byte = two codes = one shared-memory lookup into a 256-entry half2
//    table (lut[first code], lut[second code]); the table is stored once per
//    bank (lut2[byte][lane], 32 KiB) so the 32 random lookups of a warp never
//    conflict; the byte is turned into a shared-memory offset with one shift
//    and one logic op;
//  * products are summed in half2 over the 32 weights of a chunk (two
//    accumulators of 8 fused multiply-adds), then scaled by the chunk's fp32
//    absmax and accumulated in fp32; the input chunk is read from shared
//    memory once for both rows;
//  * a warp-shuffle tree combines the lanes, lane 0 stores the fp16 result.
#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRows = 2;  // rows per warp step

// sum of the 32 products of one 16-byte chunk against 16 half2 inputs
__device__ __forceinline__ float chunk_dot(const uint4& codes, const uint32_t (&x2)[16],
                                           const unsigned char* lut_lane) {
  const uint32_t w[4] = {codes.x, codes.y, codes.z, codes.w};
  __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    // byte b of the word -> offset (byte << 7) into lut2[byte][lane] (4-byte entries)
    const uint32_t o0 = (w[i] << 7) & 0x7f80u;
    const uint32_t o1 = (w[i] >> 1) & 0x7f80u;
    const uint32_t o2 = (w[i] >> 9) & 0x7f80u;
    const uint32_t o3 = (w[i] >> 17) & 0x7f80u;
    const uint32_t l0 = *reinterpret_cast<const uint32_t*>(lut_lane + o0);
    const uint32_t l1 = *reinterpret_cast<const uint32_t*>(lut_lane + o1);
    const uint32_t l2 = *reinterpret_cast<const uint32_t*>(lut_lane + o2);
    const uint32_t l3 = *reinterpret_cast<const uint32_t*>(lut_lane + o3);
    a0 = __hfma2(u32_as_half2(l0), u32_as_half2(x2[4 * i + 0]), a0);
    a1 = __hfma2(u32_as_half2(l1), u32_as_half2(x2[4 * i + 1]), a1);
    a0 = __hfma2(u32_as_half2(l2), u32_as_half2(x2[4 * i + 2]), a0);
    a1 = __hfma2(u32_as_half2(l3), u32_as_half2(x2[4 * i + 3]), a1);
  }
  const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
  return (f0.x + f0.y) + (f1.x + f1.y);
}

__global__ void __launch_bounds__(kThreads)
nf4_gemv_kernel(const __half* __restrict__ A, const uint8_t* __restrict__ B,
                const float* __restrict__ absmax, const float* __restrict__ lut16,
                __half* __restrict__ out, int N, int K, int chunks_per_block, int low_first) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* lut2 = reinterpret_cast<uint32_t*>(smem);             // [256][32]
  uint4* xs = reinterpret_cast<uint4*>(smem + 256 * 32 * 4);       // K halves
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  {
    // thread t builds entry t (byte value t) and writes its 32 copies
    const int hi = tid >> 4, lo = tid & 15;
    const int first = low_first ? lo : hi, second = low_first ? hi : lo;
    const __half2 v = __floats2half2_rn(lut16[first], lut16[second]);
    const uint32_t u = half2_as_u32(v);
    uint4 u4 = make_uint4(u, u, u, u);
    uint4* row = reinterpret_cast<uint4*>(lut2 + tid * 32);
#pragma unroll
    for (int q = 0; q < 8; q++) row[(q + tid) & 7] = u4;
  }
  const int nchunks = K >> 5;  // 32-code chunks per row
  for (int i = tid; i < (K >> 3); i += kThreads) xs[i] = reinterpret_cast<const uint4*>(A)[i];
  __syncthreads();

  const unsigned char* lut_lane = smem + lane * 4;
  const int warps_total = gridDim.x * kWarps;
  const int gwarp = blockIdx.x * kWarps + warp;

  for (int n0 = gwarp * kRows; n0 < N; n0 += warps_total * kRows) {
    const bool has1 = (n0 + 1) < N;
    const int n1 = has1 ? n0 + 1 : n0;
    const uint4* b0 = reinterpret_cast<const uint4*>(B + (size_t)n0 * (K >> 1));
    const uint4* b1 = reinterpret_cast<const uint4*>(B + (size_t)n1 * (K >> 1));
    const uint32_t cbase0 = (uint32_t)n0 * (uint32_t)nchunks;  // chunk index of row start
    const uint32_t cbase1 = (uint32_t)n1 * (uint32_t)nchunks;
    float acc0 = 0.f, acc1 = 0.f;
    for (int c = lane; c < nchunks; c += 64) {
      const int c2 = c + 32;
      const bool two = c2 < nchunks;
      const int cc2 = two ? c2 : c;
      // issue all loads of the step first
      const uint4 q00 = ldg_stream_u4(b0 + c), q10 = ldg_stream_u4(b1 + c);
      const uint4 q01 = ldg_stream_u4(b0 + cc2), q11 = ldg_stream_u4(b1 + cc2);
      const float s00 = __ldg(absmax + (cbase0 + c) / chunks_per_block);
      const float s10 = __ldg(absmax + (cbase1 + c) / chunks_per_block);
      const float s01 = __ldg(absmax + (cbase0 + cc2) / chunks_per_block);
      const float s11 = __ldg(absmax + (cbase1 + cc2) / chunks_per_block);
      uint32_t x2[16];
      {
        const uint4* xp = xs + 4 * c;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const uint4 t = xp[q];
          x2[4 * q] = t.x; x2[4 * q + 1] = t.y; x2[4 * q + 2] = t.z; x2[4 * q + 3] = t.w;
        }
      }
      acc0 = fmaf(chunk_dot(q00, x2, lut_lane), s00, acc0);
      acc1 = fmaf(chunk_dot(q10, x2, lut_lane), s10, acc1);
      if (two) {
        const uint4* xp = xs + 4 * c2;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const uint4 t = xp[q];
          x2[4 * q] = t.x; x2[4 * q + 1] = t.y; x2[4 * q + 2] = t.z; x2[4 * q + 3] = t.w;
        }
        acc0 = fmaf(chunk_dot(q01, x2, lut_lane), s01, acc0);
        acc1 = fmaf(chunk_dot(q11, x2, lut_lane), s11, acc1);
      }
    }
    acc0 = warp_sum(acc0);
    acc1 = warp_sum(acc1);
    if (lane == 0) {
      out[n0] = __float2half_rn(acc0);
      if (has1) out[n1] = __float2half_rn(acc1);
    }
  }
}

// One thread: 4 bytes of codes (8 elements) -> 16 bytes of fp16.
__global__ void __launch_bounds__(kThreads)
nf4_dequant_kernel(const uint8_t* __restrict__ B, const float* __restrict__ absmax,
                   const float* __restrict__ lut16, __half* __restrict__ out, size_t nwords,
                   int words_per_block, int low_first) {
  __shared__ float lut[16 * 32];  // [code][lane]
  const int tid = threadIdx.x, lane = tid & 31;
  for (int i = tid; i < 16 * 32; i += kThreads) lut[i] = lut16[i >> 5];
  __syncthreads();
  const float* lut_lane = lut + lane;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t w = (size_t)blockIdx.x * kThreads + tid; w < nwords; w += stride) {
    const uint32_t codes = ldg_stream_u32(reinterpret_cast<const uint32_t*>(B) + w);
    const float s = __ldg(absmax + w / (size_t)words_per_block);
    uint32_t o[4];
#pragma unroll
    for (int b = 0; b < 4; b++) {
      const uint32_t byte = (codes >> (8 * b)) & 0xffu;
      const uint32_t hi = byte >> 4, lo = byte & 15u;
      const uint32_t first = low_first ? lo : hi, second = low_first ? hi : lo;
      const float v0 = __fmul_rn(lut_lane[first * 32], s);
      const float v1 = __fmul_rn(lut_lane[second * 32], s);
      o[b] = half2_as_u32(__floats2half2_rn(v0, v1));
    }
    reinterpret_cast<uint4*>(out)[w] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_nf4_dequant_f16(const uint8_t* B, const float* absmax, const float* lut16, void* out_half,
                       size_t n, int blocksize, int flags, hq_stream_t stream) {
  using namespace hq;
  if (!lut16 || (n && (!B || !absmax || !out_half))) return HQ_ERR_NULL_POINTER;
  if (blocksize <= 0 || blocksize % 32 != 0 || n % 32 != 0) return HQ_ERR_BAD_SHAPE;
  if (n == 0) return HQ_OK;
  if (!aligned4(B) || !aligned16(out_half)) return HQ_ERR_MISALIGNED;
  const size_t nwords = n / 8;
  const size_t want = (nwords + kThreads - 1) / kThreads;
  const size_t cap = (size_t)sm_count() * 16;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  nf4_dequant_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
      B, absmax, lut16, reinterpret_cast<__half*>(out_half), nwords, blocksize / 8,
      (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0);
  return launch_status();
}

int hq_nf4_gemv_f16(const void* A_half, const uint8_t* B, const float* absmax, const float* lut16,
                    void* out_half, int N, int K, int blocksize, int flags, hq_stream_t stream) {
  using namespace hq;
  if (!A_half || !B || !absmax || !lut16 || !out_half) return HQ_ERR_NULL_POINTER;
  if (N <= 0 || K <= 0 || K % 32 != 0 || blocksize <= 0 || blocksize % 32 != 0 ||
      K % blocksize != 0)
    return HQ_ERR_BAD_SHAPE;
  if (!aligned16(B) || !aligned16(A_half)) return HQ_ERR_MISALIGNED;
  if ((uint64_t)N * (uint64_t)(K / 32) > 0xffffffffull) return HQ_ERR_TOO_LARGE;
  const size_t smem = 256 * 32 * 4 + (size_t)K * 2;
  if (smem > 200 * 1024) return HQ_ERR_TOO_LARGE;
  cudaError_t e = cudaFuncSetAttribute(nf4_gemv_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_status(e);
  const int sms = sm_count();
  int ctas_per_sm = (int)((220 * 1024) / (smem + 1024));
  if (ctas_per_sm > 6) ctas_per_sm = 6;
  if (ctas_per_sm < 1) ctas_per_sm = 1;
  const int need = (N + kWarps * kRows - 1) / (kWarps * kRows);
  int grid = sms * ctas_per_sm;
  if (grid > need) grid = need;
  nf4_gemv_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(
      reinterpret_cast<const __half*>(A_half), B, absmax, lut16,
      reinterpret_cast<__half*>(out_half), N, K, blocksize / 32,
      (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0);
  return launch_status();
}

}  // extern "C"
