// bitsandbytes 8-bit dynamic-map quantize (quantBnB kQuantize) for sm_100a.
//
// out[i] = index that dQuantize<0> (quantBnB-cuda/main.cu:13-66) selects for
// A[i] in a 256-entry code table: a 7-step pivot search from index 127 with
// strides 64..1, then a midpoint test against the tightest bracket visited.
// The same sequence of fp32 compares is executed here, so the result is
// bit-exact for ANY table (sorted or not, NaN inputs included).
//
// Design.  5 bytes per element of HBM traffic; the search is a chain of
// dependent table reads per element, so instruction issue and shared-memory
// bandwidth are the second wall.  The table is replicated once per bank
// (table[entry][lane]) so every lookup of a warp is conflict-free whatever the
// 32 pivots are, and the first two levels (pivots 127, 63/191) come from
// registers.  Each thread quantizes four consecutive elements (one 16-byte
// load, one 4-byte store).
//
// Only the pivot is tracked through the search.  The reference also carries
// (lower_pivot, lower) and (upper_pivot, upper), the last pivots at which the
// compare went up resp. down, but with strides 64, 32, .., 1 these are
// functions of the final pivot P alone: after the last "down" at pivot p with
// stride s every later step goes up, so P = p - s + (s - 1) = p - 1, i.e.
// upper_pivot = P + 1 (and P = 254, upper_pivot = 255 when no step went down);
// symmetrically lower_pivot = P - 1, or 0 when no step went up (then P = 0).
// `upper` and `lower` are the table entries at those indices - for any table,
// sorted or not, because the argument is about indices only.  So the final
// test reads ONE neighbour, code[P + 1] or code[max(P - 1, 0)], and the result
// is the one the reference's compare sequence gives, NaN inputs included.
//
// The integer side of the search runs on the half-rate integer pipe, which is
// what bounds the kernel once the loads are covered, so a level costs one
// compare, ONE predicated add and one table read: only the "went up" strides
// are accumulated, and the constant rest of the pivot's address is an
// immediate of the shared-memory load.
#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;

template <int IMM>
__device__ __forceinline__ float lds_f32_imm(uint32_t addr) {
  // not volatile: the table is constant after the barrier that follows its set-up
  float v;
  asm("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(IMM));
  return v;
}

// One search level with stride D (in table rows of 128 bytes): a compare, one
// predicated add and the next pivot's value.  With acc = lane address + (sum of
// 2*d*128 over the levels that went up), the pivot after this level is at
// acc + (D - 1) * 128, and the constant part rides in the load's immediate.
template <int D>
__device__ __forceinline__ void search_level(uint32_t& acc, float& val, float x) {
  if (x > val) acc += 2u * D * 128u;
  val = lds_f32_imm<(D - 1) * 128>(acc);
}

// lane_addr: shared-window address of table[0][lane]; entry p is at lane_addr +
// p * 128, and the row before entry 0 holds a copy of entry 0 (so that the
// "lower neighbour" of pivot 0 can be read without a clamp on the address).
__device__ __forceinline__ uint32_t quantize_one(uint32_t lane_addr, float x, float c127, float c63,
                                                 float c191) {
  // step i = 64 (val = code[127]): decided from registers
  const bool up0 = x > c127;
  float val = up0 ? c191 : c63;
  uint32_t acc = lane_addr + (up0 ? 128u * 128u : 0u);
  search_level<32>(acc, val, x);
  search_level<16>(acc, val, x);
  search_level<8>(acc, val, x);
  search_level<4>(acc, val, x);
  search_level<2>(acc, val, x);
  search_level<1>(acc, val, x);
  // (acc - lane_addr) / 128 is the final pivot P, val = code[P].  The neighbour is
  // one row up or down: ONE load from a selected address (two loads under a
  // condition compile to a branch), and the answer is the row of the pivot or of
  // the neighbour - the guard row in front of entry 0 stands for "stay at 0".
  const bool gt = x > val;
  const uint32_t nb_addr = gt ? acc + 128u : acc - 128u;
  const float nb = lds_f32_imm<0>(nb_addr);
  const float midpoint = (nb + val) * 0.5f;
  const bool step = gt ? (x > midpoint) : (x < midpoint);
  const int row = (int)((step ? nb_addr : acc) - lane_addr) >> 7;  // -1 for the guard row
  return (uint32_t)max(row, 0);
}

__global__ void __launch_bounds__(kThreads)
bnb_quantize_kernel(const float* __restrict__ code, const float* __restrict__ A,
                    uint8_t* __restrict__ out, size_t n) {
  extern __shared__ __align__(16) float table_raw[];  // one guard row, then [256][32]
  float* table = table_raw + 32;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  {
    // thread t replicates entry t into its 32-word row
    const float v = code[tid];
    float4 v4 = make_float4(v, v, v, v);
    float4* row = reinterpret_cast<float4*>(table + tid * 32);
#pragma unroll
    for (int q = 0; q < 8; q++) row[(q + tid) & 7] = v4;  // rotate to spread banks
    if (tid < 32) table_raw[tid] = code[0];  // the guard row in front of entry 0
  }
  __syncthreads();
  const uint32_t tab_lane = (uint32_t)__cvta_generic_to_shared(table + lane);
  const float c127 = table[127 * 32 + lane], c63 = table[63 * 32 + lane],
              c191 = table[191 * 32 + lane];

  const size_t nvec = n >> 2;
  const size_t stride = (size_t)gridDim.x * kThreads;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(A) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 3u) == 0;
  if (vec_ok) {
    for (size_t v = (size_t)blockIdx.x * kThreads + tid; v < nvec; v += stride) {
      if (!HQ_IN_BOUNDS(A + 4 * v, 16, A, n * 4, 301) ||
          !HQ_IN_BOUNDS(reinterpret_cast<uint32_t*>(out) + v, 4, out, n, 302))
        continue;
      uint4 raw = ldg_stream_u4(A + 4 * v);
      uint32_t q0 = quantize_one(tab_lane, __uint_as_float(raw.x), c127, c63, c191);
      uint32_t q1 = quantize_one(tab_lane, __uint_as_float(raw.y), c127, c63, c191);
      uint32_t q2 = quantize_one(tab_lane, __uint_as_float(raw.z), c127, c63, c191);
      uint32_t q3 = quantize_one(tab_lane, __uint_as_float(raw.w), c127, c63, c191);
      reinterpret_cast<uint32_t*>(out)[v] = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
    }
    // tail (n % 4 elements)
    if (blockIdx.x == 0 && tid < (int)(n & 3)) {
      const size_t i = (nvec << 2) + tid;
      out[i] = (uint8_t)quantize_one(tab_lane, A[i], c127, c63, c191);
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * kThreads + tid; i < n; i += stride)
      out[i] = (uint8_t)quantize_one(tab_lane, A[i], c127, c63, c191);
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
  const size_t smem = 257 * 32 * sizeof(float);  // guard row + table
  constexpr auto kern = bnb_quantize_kernel;
  const cudaError_t e = ensure_dynamic_smem<kern>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  const size_t want = (n / 4 + kThreads - 1) / kThreads;
  const size_t cap = (size_t)sm_count() * 6;
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
  bnb_quantize_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(code256, A, out, n);
  return launch_status();
}
