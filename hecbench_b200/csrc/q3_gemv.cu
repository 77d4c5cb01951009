// GPTQ 3-bit packed mat-vec for sm_100a.
//
// Packed layout (quant3MatMul-cuda/kernels.h:41-87): mat is int32[height][width];
// for output column c and K-group r (32 inputs) rows 3r..3r+2 of mat[:,c] form a
// 96-bit little-endian stream, code j at bits 3j..3j+2.
//
// Design.  HBM-bound on the packed words, but at 12 bytes per 32 weights the
// instruction issue rate is the second wall, so the unpack costs one logic op
// per weight (fp32 path) or per two weights (fp16 path):
//  * a thread owns four adjacent columns and reads one 16-byte vector per
//    packed row, so a warp reads 512 contiguous bytes of each row;
//  * a 3-bit field left in place inside a zero word IS a denormal number:
//    (w & (7 << p)) read as fp32 is q * 2^(p-149); read as a half in either
//    half of the word it is q * 2^(p-24).  Multiplying by an input that was
//    pre-scaled by the matching power of two (done once per CTA in shared
//    memory) gives q*x directly from AND + FMA, no shift, no int->float;
//  * the affine part is factored: sum (s*q - z)*x = s*sum(q*x) - z*sum(x);
//  * K is split over the 8 warps of a CTA and over gridDim.y; partial sums are
//    combined in shared memory and added to mul with one atomicAdd per column
//    per CTA (the reference API accumulates into mul).
#include "hq_common.cuh"

namespace hq {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kColsPerCta = 128;  // 32 lanes x 4 columns
constexpr int kF16Words = 20;     // 18 half2 input pairs per group + 2 pad (16-byte rows)

__device__ __forceinline__ float pow2f(int e) { return __int_as_float((e + 127) << 23); }

// Window starts (in codes) of the six 32-bit windows of the fp16 path.  Window a
// holds codes a..a+2 at bits 1,4,7 of its low half and codes a+5..a+7 at bits
// 0,3,6 of its high half.
__device__ __forceinline__ int f16_window_start(int w) {
  return w == 0 ? 0 : w == 1 ? 3 : w == 2 ? 11 : w == 3 ? 14 : w == 4 ? 22 : 25;
}

// MULTI: a CTA takes several column blocks one after the other (a separate
// instantiation: the single-block form keeps its code).
template <bool F16IN, bool MULTI>
__global__ void __launch_bounds__(kThreads)
q3_gemv_kernel(const void* __restrict__ vec_, const int32_t* __restrict__ mat,
               float* __restrict__ mul, const float* __restrict__ scales,
               const float* __restrict__ zeros, int groups, int width, int groups_per_cta,
               int colblocks_per_cta) {
  // the next kernel of the stream may become resident while this grid runs;
  // nothing is read or written before every earlier kernel has completed
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g0 = blockIdx.y * groups_per_cta;
  const int ng = min(groups_per_cta, groups - g0);

  // shared layout: [xp table][gsum ng floats][red kWarps*128 floats][misc 4 floats]
  const int xp_words = F16IN ? kF16Words : 32;
  uint32_t* xp = reinterpret_cast<uint32_t*>(smem_raw);
  float* gsum = reinterpret_cast<float*>(xp + (size_t)groups_per_cta * xp_words);
  float* red = gsum + ((groups_per_cta + 3) & ~3);
  float* misc = red + kWarps * kColsPerCta;

  __shared__ float s_sumx[kWarps];
  // ---- prologue: per-CTA scaling exponent, pre-scaled inputs, group sums ----
  const float* xf = reinterpret_cast<const float*>(vec_);
  const __half* xh = reinterpret_cast<const __half*>(vec_);
  auto load_x = [&](int k) -> float {
    return F16IN ? __half2float(ld_dependent_f16(xh + (size_t)g0 * 32 + k))
                 : ld_dependent_f32(xf + (size_t)g0 * 32 + k);
  };
  float amax = 0.f;
  for (int i = tid; i < ng * 32; i += kThreads) amax = fmaxf(amax, fabsf(load_x(i)));
  amax = warp_max(amax);
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  if (tid == 0) {
    float m = red[0];
    for (int w = 1; w < kWarps; w++) m = fmaxf(m, red[w]);
    misc[0] = m;
  }
  __syncthreads();
  amax = misc[0];
  int e = ((__float_as_int(amax) >> 23) & 0xff) - 126;  // amax < 2^e
  if (F16IN) e = max(-24, min(e, 17));
  else e = max(-20, min(e, 100));

  for (int gi = warp; gi < ng; gi += kWarps) {
    float x = load_x(gi * 32 + lane);
    float s = warp_sum(x);
    if (lane == 0) gsum[gi] = s;
    if (!F16IN) {
      // field position of code j inside its fp32 window is 3*(j%7)
      xp[gi * 32 + lane] = __float_as_uint(x * pow2f(100 - e - 3 * (lane % 7)));
    } else {
      // all lanes take part in the shuffles; lanes 0..17 own one input pair each
      const int t = min(lane, 17);
      const int w = t / 3, i = t - 3 * w;
      const int a = f16_window_start(w);
      const bool skip_lo = (i == 2) && (w == 1 || w == 3 || w == 5);
      const bool skip_hi = (i == 2) && (w == 5);
      const float xlo = __shfl_sync(0xffffffffu, x, a + i);
      const float xhi = __shfl_sync(0xffffffffu, x, min(a + 5 + i, 31));
      const __half hlo =
          skip_lo ? __float2half(0.f) : __float2half(xlo * pow2f(15 - e - (1 + 3 * i)));
      const __half hhi = skip_hi ? __float2half(0.f) : __float2half(xhi * pow2f(15 - e - 3 * i));
      if (lane < 18) xp[gi * kF16Words + lane] = half2_as_u32(__halves2half2(hlo, hhi));
      else if (lane < 20) xp[gi * kF16Words + lane] = 0u;
    }
  }
  __syncthreads();

  // The staged inputs serve colblocks_per_cta blocks of 128 columns one after the
  // other: the staging is about a third of a block's main loop, so a CTA that
  // takes several blocks of a shorter K slice spends less of its time on it.
  const int ncb = MULTI ? colblocks_per_cta : 1;
  for (int cb = 0; cb < ncb; cb++) {
    const int colblock = blockIdx.x * ncb + cb;
    const int col0 = colblock * kColsPerCta + lane * 4;
    if (colblock * kColsPerCta >= width) break;
    // ---- main loop: this warp takes groups warp, warp+8, ... of the CTA slice ----
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float sumx = 0.f;
    const bool active = col0 < width;
    const int32_t* base = mat + (size_t)g0 * 3 * width + col0;

    // software pipeline: the three packed rows of the next group are requested
    // before the current group is unpacked
    uint4 n0 = make_uint4(0, 0, 0, 0), n1 = n0, n2 = n0;
    if (active && warp < ng) {
      const int32_t* p = base + (size_t)warp * 3 * width;
      n0 = ldg_stream_u4(p);
      n1 = ldg_stream_u4(p + width);
      n2 = ldg_stream_u4(p + 2 * (size_t)width);
    }
    for (int gi = warp; gi < ng; gi += kWarps) {
      const uint4 u0 = n0, u1 = n1, u2 = n2;
      if (active && gi + kWarps < ng) {
        const int32_t* p = base + (size_t)(gi + kWarps) * 3 * width;
        n0 = ldg_stream_u4(p);
        n1 = ldg_stream_u4(p + width);
        n2 = ldg_stream_u4(p + 2 * (size_t)width);
      }
      sumx += gsum[gi];
      const uint32_t w0s[4] = {u0.x, u0.y, u0.z, u0.w};
      const uint32_t w1s[4] = {u1.x, u1.y, u1.z, u1.w};
      const uint32_t w2s[4] = {u2.x, u2.y, u2.z, u2.w};

      if (!F16IN) {
        float x[32];
        const float4* xv = reinterpret_cast<const float4*>(xp + gi * 32);
  #pragma unroll
        for (int q = 0; q < 8; q++) {
          float4 t = xv[q];
          x[4 * q] = t.x; x[4 * q + 1] = t.y; x[4 * q + 2] = t.z; x[4 * q + 3] = t.w;
        }
  #pragma unroll
        for (int c = 0; c < 4; c++) {
          uint32_t win[5];
          win[0] = w0s[c];
          win[1] = __funnelshift_r(w0s[c], w1s[c], 21);
          win[2] = __funnelshift_r(w1s[c], w2s[c], 10);
          win[3] = __funnelshift_r(w1s[c], w2s[c], 31);
          win[4] = w2s[c] >> 20;
          float a = acc[c];
  #pragma unroll
          for (int j = 0; j < 32; j++) {
            const int w = j / 7, i = j % 7;
            a = fmaf(__uint_as_float(win[w] & (7u << (3 * i))), x[j], a);
          }
          acc[c] = a;
        }
      } else {
        uint32_t x2[kF16Words];
        const uint4* xv = reinterpret_cast<const uint4*>(xp + gi * kF16Words);
  #pragma unroll
        for (int q = 0; q < 5; q++) {
          uint4 t = xv[q];
          x2[4 * q] = t.x; x2[4 * q + 1] = t.y; x2[4 * q + 2] = t.z; x2[4 * q + 3] = t.w;
        }
  #pragma unroll
        for (int c = 0; c < 4; c++) {
          uint32_t win[6];
          win[0] = w0s[c] << 1;
          win[1] = __funnelshift_r(w0s[c], w1s[c], 8);
          win[2] = w1s[c];
          win[3] = __funnelshift_r(w1s[c], w2s[c], 9);
          win[4] = w2s[c] >> 1;
          win[5] = w2s[c] >> 10;
          __half2 a2 = __float2half2_rn(0.f);
  #pragma unroll
          for (int w = 0; w < 6; w++) {
  #pragma unroll
            for (int i = 0; i < 3; i++) {
              const uint32_t m = (7u << (1 + 3 * i)) | (7u << (16 + 3 * i));
              a2 = __hfma2(u32_as_half2(win[w] & m), u32_as_half2(x2[3 * w + i]), a2);
            }
          }
          acc[c] += __low2float(a2) + __high2float(a2);
        }
      }
    }

    // ---- epilogue: combine the 8 warps, apply scale/zero, accumulate into mul ----
  #pragma unroll
    for (int c = 0; c < 4; c++) red[warp * kColsPerCta + lane * 4 + c] = acc[c];
    __syncthreads();
    if (lane == 0) s_sumx[warp] = sumx;
    __syncthreads();
    if (tid < kColsPerCta) {
      const int col = colblock * kColsPerCta + tid;
      if (col < width) {
        float q = 0.f, sx = 0.f;
  #pragma unroll
        for (int w = 0; w < kWarps; w++) {
          q += red[w * kColsPerCta + tid];
          sx += s_sumx[w];
        }
        // undo the input pre-scaling: fp32 path 2^(49+e), fp16 path 2^(9+e)
        q = F16IN ? q * pow2f(9 + e) : (q * pow2f(49)) * pow2f(e);
        float sc, nz;
        if (F16IN) {
          // the reference rounds both parameters to fp16 (kernels.h:121-122)
          sc = __half2float(__float2half_rn(scales[col]));
          nz = __half2float(__float2half_rn(-zeros[col]));
        } else {
          sc = scales[col];
          nz = -zeros[col];
        }
        atomicAdd(&mul[col], fmaf(sc, q, nz * sx));
      }
    }
    if (MULTI) __syncthreads();  // `red` and the warp sums are reused by the next column block
  }
}

// W[k][c] for one (group, 4 columns) per thread; bit-exact dequant rules.
template <bool F16OUT>
__global__ void __launch_bounds__(256)
q3_dequant_kernel(const int32_t* __restrict__ mat, const float* __restrict__ scales,
                  const float* __restrict__ zeros, void* __restrict__ W_, int groups,
                  int width) {
  const int c = (blockIdx.x * 256 + threadIdx.x);
  const int r = blockIdx.y;
  if (c >= width) return;
  const uint32_t w0 = (uint32_t)mat[(size_t)(3 * r) * width + c];
  const uint32_t w1 = (uint32_t)mat[(size_t)(3 * r + 1) * width + c];
  const uint32_t w2 = (uint32_t)mat[(size_t)(3 * r + 2) * width + c];
  const float sc = scales[c], z = zeros[c];
  const __half sch = __float2half_rn(sc), nzh = __float2half_rn(-z);
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const int bit = 3 * j;
    uint32_t q;
    if (bit + 3 <= 32) q = (w0 >> bit) & 7u;
    else if (bit < 32) q = __funnelshift_r(w0, w1, bit) & 7u;
    else if (bit + 3 <= 64) q = (w1 >> (bit - 32)) & 7u;
    else if (bit < 64) q = __funnelshift_r(w1, w2, bit - 32) & 7u;
    else q = (w2 >> (bit - 64)) & 7u;
    const size_t o = (size_t)(32 * r + j) * width + c;
    if (F16OUT) {
      reinterpret_cast<__half*>(W_)[o] = __hfma(__int2half_rn((int)q), sch, nzh);
    } else {
      reinterpret_cast<float*>(W_)[o] = fmaf(sc, (float)q, -z);
    }
  }
}

template <bool F16IN>
int q3_gemv_launch(const void* vec, const int32_t* mat, float* mul, const float* scales,
                   const float* zeros, int height, int width, hq_stream_t stream) {
  if (!vec || !mat || !mul || !scales || !zeros) return HQ_ERR_NULL_POINTER;
  if (height <= 0 || width <= 0 || height % 3 != 0 || width % 4 != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(mat)) return HQ_ERR_MISALIGNED;
  if (!aligned4(vec) || !aligned4(mul)) return HQ_ERR_MISALIGNED;
  const int groups = height / 3;
  const int colblocks_total = (width + kColsPerCta - 1) / kColsPerCta;
  // Grid = (column blocks / CB) x (K split).  A slice holds at most 256 groups
  // (8192 inputs: the pre-scaled inputs fit shared memory) and at least one
  // group per warp.  Cost model per CTA, in group iterations of one column block:
  // 6 fixed + g * (CB + 0.34) - staging a group's inputs costs about a third of
  // using them for one block - times the number of waves the grid needs on the
  // resident CTA slots (a grid of 2.1 waves runs as long as one of 3).
  const int sms = sm_count();
  const int slots = sms * (F16IN ? 4 : 3);  // resident CTAs at 59 / 74 registers per thread
  const int k_lo = max(1, (groups + 255) / 256);
  int ksplit = k_lo, cbs = 1;
  double best = 1e30;
  // (fp32 inputs: staging is cheap there and several blocks per CTA measured slower)
  for (int cb = 1; cb <= (F16IN ? 4 : 1); cb *= 2) {
    const int colblocks = (colblocks_total + cb - 1) / cb;
    const int k_hi =
        max(k_lo, min((groups + kWarps - 1) / kWarps, (16 * sms + colblocks - 1) / colblocks));
    for (int k = k_lo; k <= k_hi; k++) {
      const int g = (groups + k - 1) / k;
      const int kk = (groups + g - 1) / g;
      const long ctas = (long)colblocks * kk;
      const long waves = (ctas + slots - 1) / slots;
      // a grid that leaves most slots of its last wave empty pays with idle SMs
      const double fill = (double)ctas / (double)(waves * slots);
      const double cost = (double)waves * (6.0 + g * (cb + 0.34)) / (fill > 0.5 ? 1.0 : 2.0 * fill);
      if (cost < best - 1e-9) { best = cost; ksplit = kk; cbs = cb; }
    }
  }
  const int colblocks = (colblocks_total + cbs - 1) / cbs;
  int gpc = (groups + ksplit - 1) / ksplit;
  ksplit = (groups + gpc - 1) / gpc;
  const int xp_words = F16IN ? kF16Words : 32;
  size_t smem = (size_t)gpc * xp_words * 4 + (size_t)((gpc + 3) & ~3) * 4 +
                (size_t)kWarps * kColsPerCta * 4 + 16;
  dim3 grid(colblocks, ksplit);
  if (cbs > 1) {
    constexpr auto kern = q3_gemv_kernel<F16IN, true>;
    if (smem > 48 * 1024) {
      cudaError_t e = ensure_dynamic_smem<kern>(smem);
      if (e != cudaSuccess) return cuda_status(e);
    }
    return cuda_status(launch_pdl(kern, grid, dim3(kThreads), smem, (cudaStream_t)stream, vec, mat,
                                  mul, scales, zeros, groups, width, gpc, cbs));
  }
  constexpr auto kern = q3_gemv_kernel<F16IN, false>;
  if (smem > 48 * 1024) {
    cudaError_t e = ensure_dynamic_smem<kern>(smem);
    if (e != cudaSuccess) return cuda_status(e);
  }
  return cuda_status(launch_pdl(kern, grid, dim3(kThreads), smem, (cudaStream_t)stream, vec, mat,
                                mul, scales, zeros, groups, width, gpc, 1));
}

template <bool F16OUT>
int q3_dequant_launch(const int32_t* mat, const float* scales, const float* zeros, void* W,
                      int height, int width, hq_stream_t stream) {
  if (!mat || !scales || !zeros || !W) return HQ_ERR_NULL_POINTER;
  if (height <= 0 || width <= 0 || height % 3 != 0) return HQ_ERR_BAD_SHAPE;
  dim3 grid((width + 255) / 256, height / 3);
  q3_dequant_kernel<F16OUT><<<grid, 256, 0, (cudaStream_t)stream>>>(mat, scales, zeros, W,
                                                                  height / 3, width);
  return launch_status();
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_q3_gemv_f32(const float* vec, const int32_t* mat, float* mul, const float* scales,
                   const float* zeros, int height, int width, hq_stream_t stream) {
  return hq::q3_gemv_launch<false>(vec, mat, mul, scales, zeros, height, width, stream);
}

int hq_q3_gemv_f16in(const void* vec_half, const int32_t* mat, float* mul, const float* scales,
                     const float* zeros, int height, int width, hq_stream_t stream) {
  return hq::q3_gemv_launch<true>(vec_half, mat, mul, scales, zeros, height, width, stream);
}

int hq_q3_dequant_f32(const int32_t* mat, const float* scales, const float* zeros, float* W,
                      int height, int width, hq_stream_t stream) {
  return hq::q3_dequant_launch<false>(mat, scales, zeros, W, height, width, stream);
}

int hq_q3_dequant_f16(const int32_t* mat, const float* scales, const float* zeros, void* W_half,
                      int height, int width, hq_stream_t stream) {
  return hq::q3_dequant_launch<true>(mat, scales, zeros, W_half, height, width, stream);
}

}  // extern "C"
