// Uniformly quantized weight-only mat-vec (gemv-cuda) for sm_100a: fp16, int8
// and packed int4 weights with ONE scale and zero point per tensor.
//
// Reference semantics (gemv-cuda/kernels.h:64-123 fp16, :127-200 int8, :205-307
// int4; launchers gemv.cu:15-81): mat is row-major [rows][n] (int4: n/2 bytes
// per row, element 2j in the LOW nibble of byte j, 2j+1 in the high nibble);
// scale and zero point are rounded to fp16 by the launcher and used as fp32;
//   res[row] = half( scale * sum_j float(vec[j]) * (float(w[row][j]) - zero_point) )
// with fp32 accumulation.  Here the affine part is factored,
//   scale * ( sum_j w*x  -  zero_point * sum_j x ),
// the products are formed in fp16 pairs (an integer weight is exact in fp16)
// and summed in fp32 every 32 (int8, fp16) or 64 (int4) weights per lane.
//
// Design.  HBM-bound (2, 1 or 0.5 bytes per weight).  Two 512-thread CTAs per
// SM; the input vector is staged once per CTA in shared memory (fp16) and its
// sum reduced there; a warp owns whole rows, two adjacent ones at a time (a
// piece of the input vector read from shared memory then serves both), and
// streams them with 128-bit loads that bypass L1, eight loads (128 bytes per
// lane) in flight.
//  * int8 -> fp16: one XOR flips the sign bits of four bytes (b + 128), a byte
//    permute places two of them under the exponent byte 0x64 (1024 + b + 128,
//    exact), one half2 subtract of 1152 leaves the integers, one half2 fma
//    multiplies with the inputs: 7 instructions per 4 weights.
//  * int4: a 32-bit word holds 8 weights; (w & 0x000f000f) | 0x64006400 is
//    half2(1024 + e0, 1024 + e4) and (w & 0x00f000f0) | 0x64006400 is half2(1024 +
//    16 e1, 1024 + 16 e5) (w >> 8 for the other four); one half2 subtraction, or
//    one fused x / 16 - 64, leaves the integers exactly: 13 instructions per 8
//    weights, no table, no shared-memory lookups.  The inputs are staged in the
//    matching order (x0, x4)(x1, x5)(x2, x6)(x3, x7).
#include <algorithm>

#include "gemv_rows.cuh"

namespace hq {
namespace {

using namespace rows;

// n: inputs per row; row_bytes = n * BITS / 8 (a multiple of 16).
template <int BITS>
__global__ void __launch_bounds__(kThreads, 2)
gemv_uniform_kernel(const unsigned char* __restrict__ mat, const __half* __restrict__ vec,
                    __half* __restrict__ res, int rows, int n, float scale, float zero_point) {
  extern __shared__ __align__(16) unsigned char dsm_raw[];  // the inputs
  __shared__ float s_part[kWarps];
  __half* xs = reinterpret_cast<__half*>(dsm_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kPieces = 16 / BITS == 0 ? 1 : 16 / BITS;  // 16-byte pieces of inputs per chunk
  const size_t row_bytes = (size_t)n * BITS / 8;
  const int chunks = (int)(row_bytes / 16);   // 16-byte chunks per row

  // Programmatic dependent launch: the next kernel of the stream may become
  // resident while this grid drains; everything that earlier work may have
  // produced - the input vector - is read after the wait, and nothing is written
  // before it.
  pdl_launch_dependents();
  pdl_wait();
  // ---- prologue: inputs to shared memory (piece-major) and their sum ----
  float part = 0.f;
  for (int i = tid; i < n / 8; i += kThreads) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (HQ_IN_BOUNDS(reinterpret_cast<const uint4*>(vec) + i, 16, vec, (size_t)n * 2, 401))
      v = ld_dependent_u4(reinterpret_cast<const uint4*>(vec) + i);
    // 16-byte piece p of chunk c goes to [p][c] (int4: in the order of its conversion)
    reinterpret_cast<uint4*>(xs)[(i % kPieces) * chunks + i / kPieces] = BITS == 4 ? pair_inputs(v) : v;
    const float2 f0 = __half22float2(u32_as_half2(v.x)), f1 = __half22float2(u32_as_half2(v.y)),
                 f2 = __half22float2(u32_as_half2(v.z)), f3 = __half22float2(u32_as_half2(v.w));
    part += ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
  }
  part = warp_sum(part);
  if (lane == 0) s_part[warp] = part;
  __syncthreads();
  float sumx = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; w++) sumx += s_part[w];

  // ---- rows of this warp: kRows adjacent rows at a time, so that a piece of the
  // input vector read from shared memory serves kRows rows ----
  const int warps_total = gridDim.x * kWarps;
  constexpr int kPerRow = kInFlight / kRows;  // loads per row and batch
  const size_t mat_bytes = (size_t)rows * row_bytes;
  (void)mat_bytes;
  for (long long row0 = ((long long)blockIdx.x * kWarps + warp) * kRows; row0 < rows;
       row0 += (long long)warps_total * kRows) {
    const unsigned char* src = mat + (size_t)row0 * row_bytes;
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
          if (c < chunks && row0 + r < rows && HQ_IN_BOUNDS(at, 16, mat, mat_bytes, 402))
            w[u][r] = ldg_stream_u4(at);
        }
      }
#pragma unroll
      for (int u = 0; u < kPerRow; u++) {
        const int c = c0 + 32 * u;
        if (c < chunks) {
          float part[kRows];
          chunk_dot<BITS, kRows>(w[u], reinterpret_cast<const uint4*>(xs) + c, chunks, part);
#pragma unroll
          for (int r = 0; r < kRows; r++) acc[r] += part[r];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRows; r++) {
      const float total = warp_sum(acc[r]);
      if (lane == 0 && row0 + r < rows && HQ_IN_BOUNDS(res + row0 + r, 2, res, (size_t)rows * 2, 403))
        res[row0 + r] = __float2half_rn(BITS == 16 ? total : scale * (total - zero_point * sumx));
    }
  }
}

template <int BITS>
int launch(const void* mat, const void* vec_half, void* res_half, int rows, int n, float scale,
           float zero_point, hq_stream_t stream) {
  if (!mat || !vec_half || !res_half) return HQ_ERR_NULL_POINTER;
  // a row is a whole number of 16-byte chunks and the inputs a whole number of
  // 16-byte groups: n a multiple of 8 (fp16), 16 (int8), 32 (int4)
  if (rows <= 0 || n <= 0 || n % (128 / BITS) != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(mat) || !aligned16(vec_half)) return HQ_ERR_MISALIGNED;
  const size_t smem = (size_t)n * 2;
  if (smem > 226 * 1024) return HQ_ERR_TOO_LARGE;  // beyond 113 KiB only one CTA fits an SM
  constexpr auto kern = gemv_uniform_kernel<BITS>;
  const cudaError_t e = ensure_dynamic_smem<kern>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  // the launcher of the reference rounds both parameters to fp16 (gemv.cu:21-22)
  const float s = __half2float(__float2half_rn(scale));
  const float z = __half2float(__float2half_rn(zero_point));
  const int grid = std::min(2 * sm_count(), (rows + kWarps * kRows - 1) / (kWarps * kRows));
  return cuda_status(launch_pdl(kern, dim3(grid), dim3(kThreads), smem, (cudaStream_t)stream,
                                reinterpret_cast<const unsigned char*>(mat),
                                reinterpret_cast<const __half*>(vec_half),
                                reinterpret_cast<__half*>(res_half), rows, n, s, z));
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_gemv_f16(const void* mat_half, const void* vec_half, void* res_half, int rows, int n,
                hq_stream_t stream) {
  return hq::launch<16>(mat_half, vec_half, res_half, rows, n, 1.f, 0.f, stream);
}

int hq_gemv_int8_f16(const int8_t* mat, const void* vec_half, void* res_half, int rows, int n,
                     float scale, float zero_point, hq_stream_t stream) {
  return hq::launch<8>(mat, vec_half, res_half, rows, n, scale, zero_point, stream);
}

int hq_gemv_int4_f16(const uint8_t* mat, const void* vec_half, void* res_half, int rows, int n,
                     float scale, float zero_point, hq_stream_t stream) {
  return hq::launch<4>(mat, vec_half, res_half, rows, n, scale, zero_point, stream);
}

}  // extern "C"
