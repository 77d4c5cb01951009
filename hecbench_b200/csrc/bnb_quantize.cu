// bitsandbytes 8-bit dynamic-map quantize (quantBnB kQuantize) for sm_100a.
//
// out[i] = index that dQuantize<0> (quantBnB-cuda/main.cu:13-66) selects for
// A[i] in a 256-entry code table: a 7-step pivot search from index 127 with
// strides 64..1, then a midpoint test against the tightest bracket visited.
// The same sequence of fp32 compares is executed here, so the result is
// bit-exact for ANY table (sorted or not, NaN inputs included).
//
// Design.  5 bytes per element of HBM traffic; the search is 7 dependent
// table reads per element, so shared-memory bandwidth is the second wall.  The
// table is replicated once per bank (table[entry][lane]) so every lookup of a
// warp is conflict-free whatever the 32 pivots are, and the first two levels
// (pivots 127, 63/191) come from registers.  Each thread quantizes four
// consecutive elements (one 16-byte load, one 4-byte store).
#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t quantize_one(const float* __restrict__ tab_lane, float x,
                                                 float c127, float c63, float c191, float c0,
                                                 float c255) {
  // tab_lane points at table[0][lane]; entry p is tab_lane[p * 32].
  int pivot, upper_pivot = 255, lower_pivot = 0;
  float lower = -1.0f, upper = 1.0f, val;
  // step i = 64 (val = code[127])
  if (x > c127) { lower_pivot = 127; lower = c127; pivot = 191; val = c191; }
  else          { upper_pivot = 127; upper = c127; pivot = 63;  val = c63; }
#pragma unroll
  for (int i = 32; i > 0; i >>= 1) {
    if (x > val) { lower_pivot = pivot; lower = val; pivot += i; }
    else         { upper_pivot = pivot; upper = val; pivot -= i; }
    val = tab_lane[pivot * 32];
  }
  if (upper_pivot == 255) upper = c255;
  if (lower_pivot == 0) lower = c0;
  if (x > val) {
    const float midpoint = (upper + val) * 0.5f;
    return x > midpoint ? upper_pivot : pivot;
  } else {
    const float midpoint = (lower + val) * 0.5f;
    return x < midpoint ? lower_pivot : pivot;
  }
}

__global__ void __launch_bounds__(kThreads)
bnb_quantize_kernel(const float* __restrict__ code, const float* __restrict__ A,
                    uint8_t* __restrict__ out, size_t n) {
  extern __shared__ __align__(16) float table[];  // [256][32]
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  {
    // thread t replicates entry t into its 32-word row
    const float v = code[tid];
    float4 v4 = make_float4(v, v, v, v);
    float4* row = reinterpret_cast<float4*>(table + tid * 32);
#pragma unroll
    for (int q = 0; q < 8; q++) row[(q + tid) & 7] = v4;  // rotate to spread banks
  }
  __syncthreads();
  const float* tab_lane = table + lane;
  const float c127 = tab_lane[127 * 32], c63 = tab_lane[63 * 32], c191 = tab_lane[191 * 32];
  const float c0 = tab_lane[0], c255 = tab_lane[255 * 32];

  const size_t nvec = n >> 2;
  const size_t stride = (size_t)gridDim.x * kThreads;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(A) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 3u) == 0;
  if (vec_ok) {
    for (size_t v = (size_t)blockIdx.x * kThreads + tid; v < nvec; v += stride) {
      uint4 raw = ldg_stream_u4(A + 4 * v);
      uint32_t q0 = quantize_one(tab_lane, __uint_as_float(raw.x), c127, c63, c191, c0, c255);
      uint32_t q1 = quantize_one(tab_lane, __uint_as_float(raw.y), c127, c63, c191, c0, c255);
      uint32_t q2 = quantize_one(tab_lane, __uint_as_float(raw.z), c127, c63, c191, c0, c255);
      uint32_t q3 = quantize_one(tab_lane, __uint_as_float(raw.w), c127, c63, c191, c0, c255);
      reinterpret_cast<uint32_t*>(out)[v] = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
    }
    // tail (n % 4 elements)
    if (blockIdx.x == 0 && tid < (int)(n & 3)) {
      const size_t i = (nvec << 2) + tid;
      out[i] = (uint8_t)quantize_one(tab_lane, A[i], c127, c63, c191, c0, c255);
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * kThreads + tid; i < n; i += stride)
      out[i] = (uint8_t)quantize_one(tab_lane, A[i], c127, c63, c191, c0, c255);
  }
}

}  // namespace
}  // namespace hq

extern "C" int hq_bnb_quantize_u8(const float* code256, const float* A, uint8_t* out, size_t n,
                                  hq_stream_t stream) {
  using namespace hq;
  if (!code256 || (n && (!A || !out))) return HQ_ERR_NULL_POINTER;
  if (n == 0) return HQ_OK;
  if (!aligned4(A) || !aligned4(code256)) return HQ_ERR_MISALIGNED;
  const size_t smem = 256 * 32 * sizeof(float);
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  if (configured_device != dev) {
    // the attribute is per function per device; setting it again is harmless
    e = cudaFuncSetAttribute(bnb_quantize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return cuda_status(e);
    configured_device = dev;
  }
  const size_t want = (n / 4 + kThreads - 1) / kThreads;
  const size_t cap = (size_t)sm_count() * 6;
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
  bnb_quantize_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(code256, A, out, n);
  return launch_status();
}
