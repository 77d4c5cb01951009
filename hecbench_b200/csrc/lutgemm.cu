// LUT-GEMM binary-coding mat-vec (nqmv / nqmv_bias) for sm_100a.
//
// Layouts (lut-gemm-cuda/nQWeight_fp16.h:24-26, main.cu:118-134):
//   bW     uint32[K/32][nb][M]   bit t of a word <-> input k = 32*row + t, 1 => +1
//   alpha  half[K/group][nb][M]
//   q_bias half[K/group][M]      (nullable)
//   out[m] = sum_g [ q_bias[g][m]*sum_{k in g} x_k
//                    + sum_b alpha[g][b][m] * sum_{k in g} (2*bit_b[k][m]-1)*x_k ]
//
// Like the reference (mv_fp16.h:133-227) the +-sums over 8 inputs are looked up
// by bit-plane byte in a table built from x, but:
//  * a CTA owns a K tile of 128 inputs (4 packed rows) and a range of columns;
//    the 16 tables of a tile are laid out lut[row][byte][replica c][byte-lane j]
//    so that lane (c,j) of a warp - which handles byte j of the words of
//    columns 4c..4c+3 - always reads bank 4c+j: no lookup ever conflicts;
//  * table entries and all sums are fp32 (the reference uses fp16 throughout
//    and half2 atomics on the output);
//  * the four lanes of a column quad are combined with two shuffles, each CTA
//    adds its tile's partial sums to an fp32 scratch row with one coalesced
//    reduction per 32 columns, and the last CTA to finish converts the scratch
//    to fp16, stores the output and re-zeroes the scratch.
#include <mutex>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kTileRows = 4;                       // packed rows (32 inputs each) per tile
constexpr int kLutWords = kTileRows * 256 * 32;    // replicated tables, 128 KiB
constexpr int kCompactWords = kTileRows * 256 * 4; // [row][byte value][j], 16 KiB
constexpr size_t kSmemBytes = (size_t)(kLutWords + kCompactWords + 128) * 4;

__device__ __forceinline__ void red_add_f32(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

// RPG: packed rows that share one alpha group inside a tile (4, 2 or 1).
template <int NB, int RPG>
__global__ void __launch_bounds__(kThreads, 1)
lutgemm_kernel(const uint32_t* __restrict__ bW, const __half* __restrict__ alpha,
               const __half* __restrict__ q_bias, const __half* __restrict__ x,
               __half* __restrict__ out, float* __restrict__ ws, unsigned* __restrict__ counter,
               int M, int K, int rows_per_group, int cols_per_cta) {
  extern __shared__ __align__(16) float smem[];
  float* lut = smem;                          // [row][byte][32]
  float* compact = smem + kLutWords;          // [row][byte][4]
  float* xs = compact + kCompactWords;        // 128 inputs of the tile
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.y;
  const int row0 = tile * kTileRows;               // first packed row of the tile
  const int total_rows = K >> 5;
  const int nrows = min(kTileRows, total_rows - row0);

  // ---- stage the tile's inputs (zero beyond K) ----
  if (tid < kTileRows * 32) {
    const int k = row0 * 32 + tid;
    xs[tid] = (k < K) ? __half2float(x[k]) : 0.f;
  }
  __syncthreads();

  // ---- phase A: thread = byte value; signed sums of 8 inputs for 16 byte groups ----
  {
    uint32_t sgn[8];
#pragma unroll
    for (int t = 0; t < 8; t++) sgn[t] = ((tid >> t) & 1) ? 0u : 0x80000000u;
#pragma unroll
    for (int r = 0; r < kTileRows; r++) {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float4 xa = *reinterpret_cast<const float4*>(xs + r * 32 + j * 8);
        const float4 xb = *reinterpret_cast<const float4*>(xs + r * 32 + j * 8 + 4);
        float s = __uint_as_float(__float_as_uint(xa.x) ^ sgn[0]);
        s += __uint_as_float(__float_as_uint(xa.y) ^ sgn[1]);
        s += __uint_as_float(__float_as_uint(xa.z) ^ sgn[2]);
        s += __uint_as_float(__float_as_uint(xa.w) ^ sgn[3]);
        s += __uint_as_float(__float_as_uint(xb.x) ^ sgn[4]);
        s += __uint_as_float(__float_as_uint(xb.y) ^ sgn[5]);
        s += __uint_as_float(__float_as_uint(xb.z) ^ sgn[6]);
        s += __uint_as_float(__float_as_uint(xb.w) ^ sgn[7]);
        v[j] = s;
      }
      *reinterpret_cast<float4*>(compact + (r * 256 + tid) * 4) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
  __syncthreads();
  // ---- phase B: replicate each (row, byte) entry 8 times: lane = (byte&3, replica) ----
  {
    const int c = lane & 7, bl = lane >> 3;
#pragma unroll 4
    for (int it = 0; it < kTileRows * 256 / (kWarps * 4); it++) {
      const int e = (it * kWarps + warp) * 4 + bl;  // (row*256 + byte)
      const float4 v = *reinterpret_cast<const float4*>(compact + e * 4);
      *reinterpret_cast<float4*>(lut + e * 32 + c * 4) = v;
    }
  }
  __syncthreads();

  // ---- lookup phase ----
  const int j = lane & 3;            // byte of the word this lane looks up
  const int cq = lane >> 2;          // column quad inside the 32-column step
  const unsigned char* lut_lane = reinterpret_cast<const unsigned char*>(lut) + lane * 4;
  const int shift = 8 * j;
  const int m_begin = blockIdx.x * cols_per_cta;
  const int m_end = min(M, m_begin + cols_per_cta);
  const int g0 = row0 / rows_per_group;  // alpha group of the tile's first row

  // bias uses the all-ones entry (byte 255): sum of this lane's 8 inputs per row
  float ones[kTileRows];
#pragma unroll
  for (int r = 0; r < kTileRows; r++)
    ones[r] = *reinterpret_cast<const float*>(lut_lane + (size_t)(r * 256 + 255) * 128);

  for (int ms = m_begin + warp * 32; ms < m_end; ms += kWarps * 32) {
    const int m = ms + cq * 4;
    const bool active = m < m_end;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (active) {
      uint4 wv[kTileRows][NB];
#pragma unroll
      for (int r = 0; r < kTileRows; r++)
#pragma unroll
        for (int b = 0; b < NB; b++)
          wv[r][b] = (r < nrows)
                         ? ldg_stream_u4(bW + ((size_t)(row0 + r) * NB + b) * M + m)
                         : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int r0 = 0; r0 < kTileRows; r0 += RPG) {
        if (r0 < nrows) {
          const int g = g0 + (RPG == kTileRows ? 0 : r0 / RPG);
          float t[NB][4];
#pragma unroll
          for (int b = 0; b < NB; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) t[b][c] = 0.f;
          float ones_g = 0.f;
#pragma unroll
          for (int r = r0; r < r0 + RPG; r++) {
            if (r < nrows) {
              ones_g += ones[r];
              const unsigned char* lr = lut_lane + (size_t)r * 256 * 128;
#pragma unroll
              for (int b = 0; b < NB; b++) {
                const uint32_t w4[4] = {wv[r][b].x, wv[r][b].y, wv[r][b].z, wv[r][b].w};
#pragma unroll
                for (int c = 0; c < 4; c++) {
                  const uint32_t off = ((w4[c] >> shift) & 0xffu) << 7;
                  t[b][c] += *reinterpret_cast<const float*>(lr + off);
                }
              }
            }
          }
#pragma unroll
          for (int b = 0; b < NB; b++) {
            const uint2 av = *reinterpret_cast<const uint2*>(alpha + ((size_t)g * NB + b) * M + m);
            const float2 a01 = __half22float2(u32_as_half2(av.x));
            const float2 a23 = __half22float2(u32_as_half2(av.y));
            acc[0] = fmaf(a01.x, t[b][0], acc[0]);
            acc[1] = fmaf(a01.y, t[b][1], acc[1]);
            acc[2] = fmaf(a23.x, t[b][2], acc[2]);
            acc[3] = fmaf(a23.y, t[b][3], acc[3]);
          }
          if (q_bias != nullptr) {
            const uint2 bv = *reinterpret_cast<const uint2*>(q_bias + (size_t)g * M + m);
            const float2 b01 = __half22float2(u32_as_half2(bv.x));
            const float2 b23 = __half22float2(u32_as_half2(bv.y));
            acc[0] = fmaf(b01.x, ones_g, acc[0]);
            acc[1] = fmaf(b01.y, ones_g, acc[1]);
            acc[2] = fmaf(b23.x, ones_g, acc[2]);
            acc[3] = fmaf(b23.y, ones_g, acc[3]);
          }
        }
      }
    }
    // combine the four byte lanes of each column quad
#pragma unroll
    for (int c = 0; c < 4; c++) {
      acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
      acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
    }
    const float mine = j == 0 ? acc[0] : j == 1 ? acc[1] : j == 2 ? acc[2] : acc[3];
    if (active) red_add_f32(ws + m + j, mine);  // lane (cq,j) -> column ms + lane
  }

  // ---- last CTA converts the scratch row to fp16 and re-zeroes it ----
  __shared__ unsigned s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned total = gridDim.x * gridDim.y;
    const unsigned prev = atomicAdd(counter, 1u);
    s_last = (prev == total - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    for (int m = tid; m < M; m += kThreads) {
      const float v = __ldcg(ws + m);
      out[m] = __float2half_rn(v);
      ws[m] = 0.f;
    }
    if (tid == 0) *counter = 0u;
  }
}

template <int NB>
int launch_nb(int rpg_in_tile, dim3 grid, cudaStream_t st, const uint32_t* bW, const __half* alpha,
              const __half* q_bias, const __half* x, __half* out, float* ws, unsigned* counter,
              int M, int K, int rows_per_group, int cols_per_cta) {
#define HQ_LUT_LAUNCH(RPG)                                                                    \
  {                                                                                           \
    auto kern = lutgemm_kernel<NB, RPG>;                                                      \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                         (int)kSmemBytes);                                    \
    if (e != cudaSuccess) return cuda_status(e);                                              \
    kern<<<grid, kThreads, kSmemBytes, st>>>(bW, alpha, q_bias, x, out, ws, counter, M, K,     \
                                             rows_per_group, cols_per_cta);                   \
  }
  if (rpg_in_tile == 4) HQ_LUT_LAUNCH(4)
  else if (rpg_in_tile == 2) HQ_LUT_LAUNCH(2)
  else HQ_LUT_LAUNCH(1)
#undef HQ_LUT_LAUNCH
  return launch_status();
}

}  // namespace
}  // namespace hq

extern "C" {

size_t hq_lutgemm_workspace_bytes(int M) {
  if (M <= 0) return 0;
  return ((size_t)M * 4 + 255) / 256 * 256 + 256;
}

int hq_lutgemm_nqmv(void* out_half, const void* x_half, const uint32_t* bW, const void* alpha_half,
                    const void* q_bias_half, int M, int K, int nb, int group_size, void* workspace,
                    size_t workspace_bytes, hq_stream_t stream) {
  using namespace hq;
  if (!out_half || !x_half || !bW || !alpha_half) return HQ_ERR_NULL_POINTER;
  if (M <= 0 || K <= 0 || M % 4 != 0 || K % 32 != 0 || nb < 1 || nb > 8) return HQ_ERR_BAD_SHAPE;
  if (group_size <= 0 || group_size % 32 != 0 || K % group_size != 0) return HQ_ERR_BAD_SHAPE;
  if (!workspace || workspace_bytes < hq_lutgemm_workspace_bytes(M)) return HQ_ERR_WORKSPACE;
  if (!aligned16(bW) || !aligned8(alpha_half) || (q_bias_half && !aligned8(q_bias_half)) ||
      !aligned16(workspace))
    return HQ_ERR_MISALIGNED;
  const int rpg = group_size / 32;
  int rpg_in_tile;
  if (rpg % 4 == 0) rpg_in_tile = 4;
  else if (rpg == 2) rpg_in_tile = 2;
  else if (rpg == 1) rpg_in_tile = 1;
  else return HQ_ERR_UNSUPPORTED;  // groups of 96, 160, ... inputs straddle tiles

  const int tiles = (K / 32 + kTileRows - 1) / kTileRows;
  // columns per CTA: a multiple of 256 chosen so the grid is close to a
  // multiple of the SM count with at least ~2 CTAs per SM when M allows.
  const int sms = sm_count();
  int best_cols = 256;
  double best_score = -1.0;
  const int max_chunks = (M + 255) / 256;
  for (int chunk256 = 1; chunk256 <= max_chunks; chunk256++) {
    const int mblocks = (max_chunks + chunk256 - 1) / chunk256;
    const long ctas = (long)mblocks * tiles;
    const long waves = (ctas + sms - 1) / sms;
    // efficiency = useful lookups / (lookups + table build), times wave balance
    const double amort = (double)(chunk256 * 256) / (chunk256 * 256 + 700.0);
    const double balance = (double)ctas / (double)(waves * sms);
    const double score = amort * balance;
    if (score > best_score) { best_score = score; best_cols = chunk256 * 256; }
  }
  const int mblocks = (M + best_cols - 1) / best_cols;
  dim3 grid(mblocks, tiles);
  float* ws = reinterpret_cast<float*>(workspace);
  unsigned* counter =
      reinterpret_cast<unsigned*>(reinterpret_cast<char*>(workspace) +
                                  (hq_lutgemm_workspace_bytes(M) - 256));
  const __half* alpha = reinterpret_cast<const __half*>(alpha_half);
  const __half* qb = reinterpret_cast<const __half*>(q_bias_half);
  const __half* x = reinterpret_cast<const __half*>(x_half);
  __half* out = reinterpret_cast<__half*>(out_half);
  cudaStream_t st = (cudaStream_t)stream;
#define HQ_NB_CASE(NB)                                                                        \
  case NB:                                                                                    \
    return launch_nb<NB>(rpg_in_tile, grid, st, bW, alpha, qb, x, out, ws, counter, M, K, rpg, \
                         best_cols);
  switch (nb) {
    HQ_NB_CASE(1) HQ_NB_CASE(2) HQ_NB_CASE(3) HQ_NB_CASE(4)
    HQ_NB_CASE(5) HQ_NB_CASE(6) HQ_NB_CASE(7) HQ_NB_CASE(8)
  }
#undef HQ_NB_CASE
  return HQ_ERR_BAD_SHAPE;
}


// ---- entry point that allocates nothing ----------------------------------

}  // extern "C"

namespace hq {
namespace {

// Scratch row of the allocation-free entry point: fp32 partial sums for up to
// HQ_LUTGEMM_NOALLOC_MAX_M outputs plus the completion counter.  Every GPU
// that loads the library holds these 257 KiB until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[HQ_LUTGEMM_NOALLOC_MAX_M * 4 + 256];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kMaxDevices];  // device address of the array, per device; null = not set up

// Device address of g_noalloc_scratch on the current device.  In host code the
// array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int noalloc_scratch(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  if (dev < 0 || dev >= kMaxDevices) return HQ_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_status(e);
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return HQ_OK;
}

}  // namespace
}  // namespace hq

extern "C" int hq_lutgemm_nqmv_noalloc(void* out_half, const void* x_half, const uint32_t* bW,
                                       const void* alpha_half, const void* q_bias_half, int M,
                                       int K, int nb, int group_size, hq_stream_t stream) {
  using namespace hq;
  if (M > HQ_LUTGEMM_NOALLOC_MAX_M) return HQ_ERR_TOO_LARGE;
  if (M <= 0) return HQ_ERR_BAD_SHAPE;
  void* ws = nullptr;
  const int st = noalloc_scratch(&ws);
  if (st != HQ_OK) return st;
  const size_t bytes = hq_lutgemm_workspace_bytes(M);
  // The array keeps whatever the previous call (of any caller) left in it, and
  // the kernel needs partial sums and counter to start at zero.
  cudaError_t e = cudaMemsetAsync(ws, 0, bytes, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_status(e);
  return hq_lutgemm_nqmv(out_half, x_half, bW, alpha_half, q_bias_half, M, K, nb, group_size, ws,
                         bytes, stream);
}
