// Per-token int8 activation quantization (quantVLLM) for sm_100a: the step in
// front of a W8A8 linear layer.
//
// Replaces the launchers static_scaled_int8_quant / dynamic_scaled_int8_quant
// of quantVLLM-cuda/main.cu:137-172 and their four kernels (main.cu:12-134):
//   static            out = sat8(rint(x / scale))
//   static + azp      out = sat8(sat32(rint(x / scale)) + azp)
//   dynamic           scale[t] = absmax_t / 127, out = sat8(rint(x * (127 / absmax_t)))
//   dynamic + azp     scale[t] = (max_t - min_t) / 255, azp[t] = rint(-128 - min_t / scale[t]),
//                     out = sat8(sat32(rint(x / scale[t])) + azp[t])
// for fp16, bf16 or fp32 inputs x[num_tokens][hidden_size].  Every arithmetic
// step is the reference's (IEEE division, round-half-even, the same order of
// saturations; the running maximum of the azp form starts at FLT_MIN like
// utils.h / reference.h:66), so the outputs are byte-exact.
//
// Design.  Pure streaming, 2-4 bytes in and 1 byte out per element:
//  * static forms have no per-token state: the tensor is processed flat, 16
//    elements per thread and turn (16-byte loads, one 16-byte store);
//  * dynamic forms: one CTA per token row; the row is read ONCE, kept in
//    registers (up to 32 elements per thread), reduced with warp shuffles and
//    one shared-memory exchange, and quantized from the registers - the
//    reference reads every row twice.  Rows are contiguous but start at any
//    element (the reference's own run uses hidden_size = 5137), so the CTA
//    works on the aligned 16-byte chunks that overlap its row and masks the
//    neighbours' elements: full-width loads and 8-byte stores at any row
//    offset, all loads of a row in flight together.  An element-wise form
//    covers unaligned buffers and rows beyond the register cache.
#include <cuda_bf16.h>

#include <cfloat>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }

// utils.h:9-28: nearbyint, clamp to [-128, 127], convert (NaN gives 0)
__device__ __forceinline__ int f2i8_rn(float x) {
  return max(-128, min(127, __float2int_rn(x)));  // the conversion saturates at int32 first
}
// utils.h:30-63: sat32(rint(x)) + azp (wrapping, as two's complement does), clamp
__device__ __forceinline__ int f2i8_azp(float x, int azp) {
  const int q = (int)((unsigned)__float2int_rn(x) + (unsigned)azp);
  return max(-128, min(127, q));
}

// ---- static forms: flat over num_tokens * hidden_size elements ----
template <typename T, bool AZP>
__global__ void __launch_bounds__(kThreads)
vllm_static_kernel(const T* __restrict__ in, int8_t* __restrict__ out, size_t n, float scale,
                   int azp, int vec_ok) {
  constexpr int kPerLoad = 16 / sizeof(T);  // elements per 16-byte load
  constexpr int kLoads = 16 / kPerLoad;     // loads per 16 outputs
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t nvec = vec_ok ? n / 16 : 0;
  for (size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
    if (!HQ_IN_BOUNDS(reinterpret_cast<const uint4*>(in) + v * kLoads, 16 * kLoads, in,
                      n * sizeof(T), 401) ||
        !HQ_IN_BOUNDS(reinterpret_cast<uint4*>(out) + v, 16, out, n, 402))
      continue;
    uint4 raw[kLoads];
#pragma unroll
    for (int l = 0; l < kLoads; l++)
      raw[l] = ldg_stream_u4(reinterpret_cast<const uint4*>(in) + v * kLoads + l);
    const T* e = reinterpret_cast<const T*>(raw);
    uint32_t o[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
      uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const float q = __fdiv_rn(to_float<T>(e[4 * w + b]), scale);
        const int r = AZP ? f2i8_azp(q, azp) : f2i8_rn(q);
        word |= (uint32_t)(r & 0xff) << (8 * b);
      }
      o[w] = word;
    }
    reinterpret_cast<uint4*>(out)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  // tail (and everything, when the buffers are not 16-byte aligned)
  for (size_t i = nvec * 16 + (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    const float q = __fdiv_rn(to_float<T>(in[i]), scale);
    out[i] = (int8_t)(AZP ? f2i8_azp(q, azp) : f2i8_rn(q));
  }
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : fminf(v, u);
  }
  __syncthreads();  // sh may still be read from an earlier reduction
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = sh[0];
#pragma unroll
  for (int w = 1; w < kWarps; w++) r = is_max ? fmaxf(r, sh[w]) : fminf(r, sh[w]);
  return r;
}

// ---- dynamic forms: one CTA per token row (rows dealt round-robin) ----
// Vector form.  The tensor is viewed as aligned 16-byte chunks (EPC = 8 or 4
// elements); the CTA of row t takes the chunks that overlap [t*hidden,
// (t+1)*hidden) - a chunk on a row boundary is read by both rows' CTAs and each
// masks the elements of the other row.  A thread keeps CPT chunks in registers
// (chunks tid, tid + 256, ...), so the row is read once, with full-width
// loads whatever the row's starting address is.  The eight (four) results of a
// chunk inside the row leave as one 8-byte (4-byte) store; a boundary chunk
// stores its in-row bytes one by one.
template <typename T, bool AZP, int CPT>
__global__ void __launch_bounds__(kThreads)
vllm_dynamic_vec_kernel(const T* __restrict__ in, int8_t* __restrict__ out,
                        float* __restrict__ scale_out, int* __restrict__ azp_out, int num_tokens,
                        int hidden) {
  constexpr int EPC = 16 / sizeof(T);
  __shared__ float sh[kWarps];
  const int tid = threadIdx.x;
  const size_t total = (size_t)num_tokens * hidden;
  for (int t = blockIdx.x; t < num_tokens; t += gridDim.x) {
    const size_t e0 = (size_t)t * hidden, e1 = e0 + hidden;  // the row's elements, flat
    const size_t c0 = e0 / EPC;                               // first chunk that overlaps it
    float v[CPT][EPC];
    float mx = AZP ? FLT_MIN : 0.f, mn = FLT_MAX;
#pragma unroll
    for (int j = 0; j < CPT; j++) {
      const size_t c = c0 + tid + (size_t)j * kThreads;
      const size_t first = c * EPC;
      uint4 raw = make_uint4(0, 0, 0, 0);
      // the last chunk of the tensor may be partial: it is fetched element-wise
      if (first < e1) {
        if (first + EPC <= total) {
          if (HQ_IN_BOUNDS(reinterpret_cast<const uint4*>(in) + c, 16, in, total * sizeof(T), 403))
            raw = ldg_stream_u4(reinterpret_cast<const uint4*>(in) + c);
        } else {
          T* r = reinterpret_cast<T*>(&raw);
          for (int k = 0; k < EPC; k++)
            if (first + k < total) r[k] = in[first + k];
        }
      }
      const T* e = reinterpret_cast<const T*>(&raw);
      // position of the chunk's first element inside the row (-EPC < lo < hidden)
      const int lo = first < e1 ? (int)((long long)first - (long long)e0) : hidden;
      if (lo >= 0 && lo + EPC <= hidden) {  // wholly inside the row: no masks
#pragma unroll
        for (int k = 0; k < EPC; k++) {
          const float x = to_float<T>(e[k]);
          v[j][k] = x;
          if (AZP) { mx = fmaxf(mx, x); mn = fminf(mn, x); }
          else mx = fmaxf(mx, fabsf(x));
        }
      } else {
#pragma unroll
        for (int k = 0; k < EPC; k++) {
          const bool mine = (unsigned)(lo + k) < (unsigned)hidden;
          const float x = to_float<T>(e[k]);
          v[j][k] = x;
          if (AZP) {
            mx = fmaxf(mx, mine ? x : FLT_MIN);
            mn = fminf(mn, mine ? x : FLT_MAX);
          } else {
            mx = fmaxf(mx, mine ? fabsf(x) : 0.f);
          }
        }
      }
    }
    mx = block_reduce(mx, true, sh);
    float scale, mul = 0.f;
    int azp = 0;
    if (AZP) {
      mn = block_reduce(mn, false, sh);
      scale = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
      azp = __float2int_rz(rintf(__fsub_rn(-128.0f, __fdiv_rn(mn, scale))));
    } else {
      scale = __fdiv_rn(mx, 127.0f);
      mul = __fdiv_rn(127.0f, mx);
    }
    if (tid == 0) {
      scale_out[t] = scale;
      if (AZP) azp_out[t] = azp;
    }
#pragma unroll
    for (int j = 0; j < CPT; j++) {
      const size_t first = (c0 + tid + (size_t)j * kThreads) * EPC;
      if (first >= e1) continue;
      uint32_t q[EPC / 4] = {};
#pragma unroll
      for (int k = 0; k < EPC; k++) {
        const int r = AZP ? f2i8_azp(__fdiv_rn(v[j][k], scale), azp) : f2i8_rn(__fmul_rn(v[j][k], mul));
        q[k / 4] |= (uint32_t)(r & 0xff) << (8 * (k & 3));
      }
      if (first >= e0 && first + EPC <= e1) {  // wholly inside the row: one aligned store
        if (HQ_IN_BOUNDS(out + first, EPC, out, total, 404)) {
          if (EPC == 8) *reinterpret_cast<uint2*>(out + first) = make_uint2(q[0], q[EPC / 4 - 1]);
          else *reinterpret_cast<uint32_t*>(out + first) = q[0];
        }
      } else {
#pragma unroll
        for (int k = 0; k < EPC; k++)
          if (first + k >= e0 && first + k < e1)
            out[first + k] = (int8_t)((q[k / 4] >> (8 * (k & 3))) & 0xff);
      }
    }
  }
}

// Element-wise form for buffers that are not 16 / 8-byte aligned and for rows
// longer than the register cache.  EPT: elements per thread kept in registers;
// EPT == 0 re-reads the row.
template <typename T, bool AZP, int EPT>
__global__ void __launch_bounds__(kThreads)
vllm_dynamic_kernel(const T* __restrict__ in, int8_t* __restrict__ out,
                    float* __restrict__ scale_out, int* __restrict__ azp_out, int num_tokens,
                    int hidden) {
  __shared__ float sh[kWarps];
  const int tid = threadIdx.x;
  for (int t = blockIdx.x; t < num_tokens; t += gridDim.x) {
    const T* row = in + (size_t)t * hidden;
    int8_t* orow = out + (size_t)t * hidden;
    float v[EPT > 0 ? EPT : 1];
    // reference.h:40-46 / :66-72: NaN inputs never win a compare
    float mx = AZP ? FLT_MIN : 0.f, mn = FLT_MAX;
    if (EPT > 0) {
#pragma unroll
      for (int j = 0; j < EPT; j++) {
        const int i = tid + j * kThreads;
        v[j] = i < hidden ? to_float<T>(row[i]) : (AZP ? FLT_MIN : 0.f);
      }
#pragma unroll
      for (int j = 0; j < EPT; j++) {
        if (AZP) {
          mx = fmaxf(mx, v[j]);
          if (tid + j * kThreads < hidden) mn = fminf(mn, v[j]);
        } else {
          mx = fmaxf(mx, fabsf(v[j]));
        }
      }
    } else {
      for (int i = tid; i < hidden; i += kThreads) {
        const float x = to_float<T>(row[i]);
        if (AZP) { mx = fmaxf(mx, x); mn = fminf(mn, x); }
        else mx = fmaxf(mx, fabsf(x));
      }
    }
    mx = block_reduce(mx, true, sh);
    float scale, mul = 0.f;
    int azp = 0;
    if (AZP) {
      mn = block_reduce(mn, false, sh);
      scale = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
      azp = __float2int_rz(rintf(__fsub_rn(-128.0f, __fdiv_rn(mn, scale))));
    } else {
      scale = __fdiv_rn(mx, 127.0f);
      mul = __fdiv_rn(127.0f, mx);
    }
    if (tid == 0) {
      scale_out[t] = scale;
      if (AZP) azp_out[t] = azp;
    }
    if (EPT > 0) {
#pragma unroll
      for (int j = 0; j < EPT; j++) {
        const int i = tid + j * kThreads;
        if (i < hidden)
          orow[i] = (int8_t)(AZP ? f2i8_azp(__fdiv_rn(v[j], scale), azp)
                                 : f2i8_rn(__fmul_rn(v[j], mul)));
      }
    } else {
      for (int i = tid; i < hidden; i += kThreads) {
        const float x = to_float<T>(row[i]);
        orow[i] = (int8_t)(AZP ? f2i8_azp(__fdiv_rn(x, scale), azp) : f2i8_rn(__fmul_rn(x, mul)));
      }
    }
  }
}

template <typename T>
int static_launch(int8_t* out, const void* in, size_t n, float scale, int azp, cudaStream_t st) {
  const int vec_ok = aligned16(in) && aligned16(out);
  const size_t want = (n / 16 + kThreads - 1) / kThreads;
  const size_t cap = (size_t)sm_count() * 16;
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
  const T* x = reinterpret_cast<const T*>(in);
  if (azp == 0)  // the launcher's choice, main.cu:147-152
    vllm_static_kernel<T, false><<<grid, kThreads, 0, st>>>(x, out, n, scale, azp, vec_ok);
  else
    vllm_static_kernel<T, true><<<grid, kThreads, 0, st>>>(x, out, n, scale, azp, vec_ok);
  return launch_status();
}

template <typename T, bool AZP>
int dynamic_launch_ept(int8_t* out, const T* x, float* scales, int* azp, int tokens, int hidden,
                       cudaStream_t st) {
  const unsigned grid = (unsigned)std::min(tokens, sm_count() * 32);
  constexpr int EPC = 16 / sizeof(T);
  // chunks a row can overlap: its elements plus one partial chunk at either end
  const long chunks = ((long)hidden + EPC - 1) / EPC + 1;
  const bool vec_ok = aligned16(x) && aligned8(out);
  if (vec_ok && chunks <= 1L * kThreads)
    vllm_dynamic_vec_kernel<T, AZP, 1><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  else if (vec_ok && chunks <= 2L * kThreads)
    vllm_dynamic_vec_kernel<T, AZP, 2><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  else if (vec_ok && chunks <= 4L * kThreads)
    vllm_dynamic_vec_kernel<T, AZP, 4><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  else if (vec_ok && sizeof(T) == 4 && chunks <= 8L * kThreads)
    vllm_dynamic_vec_kernel<T, AZP, 8><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  else if (hidden <= 8 * kThreads)
    vllm_dynamic_kernel<T, AZP, 8><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  else if (hidden <= 16 * kThreads)
    vllm_dynamic_kernel<T, AZP, 16><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  else if (hidden <= 32 * kThreads)
    vllm_dynamic_kernel<T, AZP, 32><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  else
    vllm_dynamic_kernel<T, AZP, 0><<<grid, kThreads, 0, st>>>(x, out, scales, azp, tokens, hidden);
  return launch_status();
}

template <typename T>
int dynamic_launch(int8_t* out, const void* in, float* scales, int* azp, int tokens, int hidden,
                   cudaStream_t st) {
  const T* x = reinterpret_cast<const T*>(in);
  return azp == nullptr ? dynamic_launch_ept<T, false>(out, x, scales, nullptr, tokens, hidden, st)
                        : dynamic_launch_ept<T, true>(out, x, scales, azp, tokens, hidden, st);
}

int check_common(const void* out, const void* in, int dtype, int hidden, int tokens) {
  if (!out || !in) return HQ_ERR_NULL_POINTER;
  if (hidden <= 0 || tokens <= 0) return HQ_ERR_BAD_SHAPE;
  if (dtype != HQ_DTYPE_F16 && dtype != HQ_DTYPE_BF16 && dtype != HQ_DTYPE_F32)
    return HQ_ERR_UNSUPPORTED;
  const uintptr_t a = reinterpret_cast<uintptr_t>(in);
  if (a & (dtype == HQ_DTYPE_F32 ? 3u : 1u)) return HQ_ERR_MISALIGNED;
  return HQ_OK;
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_vllm_static_scaled_int8_quant(int8_t* out, const void* input, int dtype, int hidden_size,
                                     int num_tokens, float scale, int32_t azp,
                                     hq_stream_t stream) {
  using namespace hq;
  const int st = check_common(out, input, dtype, hidden_size, num_tokens);
  if (st != HQ_OK) return st;
  const size_t n = (size_t)num_tokens * (size_t)hidden_size;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == HQ_DTYPE_F16) return static_launch<__half>(out, input, n, scale, azp, s);
  if (dtype == HQ_DTYPE_BF16) return static_launch<__nv_bfloat16>(out, input, n, scale, azp, s);
  return static_launch<float>(out, input, n, scale, azp, s);
}

int hq_vllm_dynamic_scaled_int8_quant(int8_t* out, const void* input, int dtype, int hidden_size,
                                      int num_tokens, float* scales, int32_t* azp,
                                      hq_stream_t stream) {
  using namespace hq;
  const int st = check_common(out, input, dtype, hidden_size, num_tokens);
  if (st != HQ_OK) return st;
  if (!scales) return HQ_ERR_NULL_POINTER;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == HQ_DTYPE_F16)
    return dynamic_launch<__half>(out, input, scales, azp, num_tokens, hidden_size, s);
  if (dtype == HQ_DTYPE_BF16)
    return dynamic_launch<__nv_bfloat16>(out, input, scales, azp, num_tokens, hidden_size, s);
  return dynamic_launch<float>(out, input, scales, azp, num_tokens, hidden_size, s);
}

}  // extern "C"
