/*
 * CPU oracle for the weight-only quantized mat-vec family.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * algorithms of four HeCBench benchmarks (quant3MatMul, quantBnB, lut-gemm,
 * quantAQLM) plus the written semantics of the pieces that have no reference
 * implementation (NF4 dequantize / 4-bit GEMV, AQLM 2x8, per-output scales,
 * batched dequant-GEMM).  It is used as the checker by the tests, by the smoke
 * entry and as the timed CPU baseline of the bench.  Nothing in the shipped
 * library calls it, and it is never a fallback for a missing GPU.
 *
 * Parity pins:
 *   q3    - known-answer vector of quant3MatMul-cuda/main.cu:28-53,86 (-49152).
 *   bnb   - byte-exact against the reference dQuantize compiled from
 *           quantBnB-omp/main.cpp (see oracle/ref_cpu.cpp and tests/golden).
 *   lut-gemm, aqlm 1x16 - no usable known-answer test exists in the reference;
 *           pinned on the GPU box against the reference CUDA kernels compiled
 *           from their own sources (oracle/ref_gpu.cu).
 *   nf4, aqlm 2x8, scales, batched - PARITY UNPINNED: the reference has no
 *           implementation or test of these; semantics are the ones written in
 *           each function's comment.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the HeCBench source tree).
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ */
/* fp16 helpers (IEEE binary16, round-to-nearest-even), bit exact      */
/* ------------------------------------------------------------------ */

static inline float orc_h2f(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* double -> half, RN-even, single rounding (the argument is exact). */
static inline uint16_t orc_d2h(double d) {
  uint16_t sign = 0;
  if (d != d) return 0x7fffu;
  if (signbit(d)) { sign = 0x8000u; d = -d; }
  if (d == 0.0) return sign;
  if (isinf(d)) return sign | 0x7c00u;
  int e;
  double m = frexp(d, &e); /* d = m * 2^e, m in [0.5,1) */
  /* value = (2m) * 2^(e-1); half normal exponent range -14..15 */
  int he = e - 1;
  double q;
  if (he < -14) {
    /* subnormal: units of 2^-24 */
    q = ldexp(d, 24);
    double r = nearbyint(q); /* default rounding mode = RN-even */
    uint32_t mi = (uint32_t)r;
    if (mi >= 0x400u) return sign | 0x0400u; /* rounded up to min normal */
    return sign | (uint16_t)mi;
  }
  q = ldexp(d, 10 - he); /* in [1024, 2048) */
  double r = nearbyint(q);
  uint32_t mi = (uint32_t)r;
  if (mi >= 2048u) { mi >>= 1; he++; }
  if (he > 15) return sign | 0x7c00u;
  return sign | (uint16_t)(((uint32_t)(he + 15) << 10) | (mi & 0x3ffu));
}

static inline uint16_t orc_f2h(float f) { return orc_d2h((double)f); }

/* fp16 fused multiply-add: one rounding of a*b+c (done in double; the
 * product of two halves is exact in double, the sum is rounded to 53 bits
 * before the final rounding to 11 bits - a double rounding that can differ
 * only on exact 53-bit ties, which 22+11-bit operands cannot produce unless
 * the exponent gap exceeds 30 binades). */
static inline uint16_t orc_hfma(uint16_t a, uint16_t b, uint16_t c) {
  return orc_d2h(fma((double)orc_h2f(a), (double)orc_h2f(b), (double)orc_h2f(c)));
}
static inline uint16_t orc_hadd(uint16_t a, uint16_t b) {
  return orc_d2h((double)orc_h2f(a) + (double)orc_h2f(b));
}
static inline uint16_t orc_hmul(uint16_t a, uint16_t b) {
  return orc_d2h((double)orc_h2f(a) * (double)orc_h2f(b));
}

void orc_f32_to_f16(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; i++) dst[i] = orc_f2h(src[i]);
}
void orc_f16_to_f32(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; i++) dst[i] = orc_h2f(src[i]);
}

/* ------------------------------------------------------------------ */
/* GPTQ 3-bit (quant3MatMul)                                           */
/* ------------------------------------------------------------------ */

/* Code j (0..31) of K-group r for column c lives in the 96-bit little-endian
 * integer formed by rows 3r,3r+1,3r+2 of mat[:,c], at bits 3j..3j+2.
 * Follows the extraction order of quant3MatMul-cuda/kernels.h:41-87
 * (codes 10 and 21 straddle the word boundaries, :55 and :71). */
static inline unsigned q3_code(const int32_t* mat, int width, int r, int c, int j) {
  uint32_t w0 = (uint32_t)mat[(size_t)(3 * r + 0) * width + c];
  uint32_t w1 = (uint32_t)mat[(size_t)(3 * r + 1) * width + c];
  uint32_t w2 = (uint32_t)mat[(size_t)(3 * r + 2) * width + c];
  int bit = 3 * j;
  uint64_t lo = (uint64_t)w0 | ((uint64_t)w1 << 32);
  if (bit + 3 <= 64) return (unsigned)((lo >> bit) & 7u);
  uint64_t hi = (uint64_t)w1 | ((uint64_t)w2 << 32); /* bits 32..95 */
  return (unsigned)((hi >> (bit - 32)) & 7u);
}

/* codes[K][width] (uint8, 0..7) -> mat[K*3/32][width]. K multiple of 32. */
void orc_q3_pack(const uint8_t* codes, int32_t* mat, int K, int width) {
  int groups = K / 32;
  memset(mat, 0, (size_t)groups * 3 * width * sizeof(int32_t));
  for (int r = 0; r < groups; r++)
    for (int c = 0; c < width; c++) {
      uint32_t w[3] = {0, 0, 0};
      for (int j = 0; j < 32; j++) {
        uint32_t q = codes[(size_t)(32 * r + j) * width + c] & 7u;
        int bit = 3 * j;
        w[bit >> 5] |= q << (bit & 31);
        if ((bit & 31) > 29) w[(bit >> 5) + 1] |= q >> (32 - (bit & 31));
      }
      for (int t = 0; t < 3; t++) mat[(size_t)(3 * r + t) * width + c] = (int32_t)w[t];
    }
}

/* Round-to-nearest 3-bit quantizer, W[K][width] fp32 (widened weights) -> the
 * packed matrix, scales and zeros of the 3-bit mat-vec.  No counterpart in the
 * reference tree (it holds only the consumer, quant3MatMul-cuda/kernels.h); the
 * rule is GPTQ's per-column min / max quantizer without its error search:
 * lo = min(column, 0), hi = max(column, 0) (-1, 1 if both are 0); scale = (hi -
 * lo) / 7; z = rint(-lo / scale); q = clamp(rint(w / scale) + z, 0, 7), all fp32;
 * scales[c] = scale, zeros[c] = scale * z. */
void orc_q3_quantize(const float* W, int K, int width, int32_t* mat, float* scales, float* zeros) {
  uint8_t* codes = (uint8_t*)malloc((size_t)K * width);
#pragma omp parallel for
  for (int c = 0; c < width; c++) {
    float lo = 0.f, hi = 0.f;
    for (int k = 0; k < K; k++) {
      const float w = W[(size_t)k * width + c];
      if (w < lo) lo = w;
      if (w > hi) hi = w;
    }
    if (lo == 0.f && hi == 0.f) {
      lo = -1.f;
      hi = 1.f;
    }
    const float scale = (hi - lo) / 7.f;
    const float z = rintf(-lo / scale);
    scales[c] = scale;
    zeros[c] = scale * z;
    for (int k = 0; k < K; k++) {
      float q = rintf(W[(size_t)k * width + c] / scale) + z;
      if (q < 0.f) q = 0.f;
      if (q > 7.f) q = 7.f;
      codes[(size_t)k * width + c] = (uint8_t)q;
    }
  }
  orc_q3_pack(codes, mat, K, width);
  free(codes);
}

void orc_q3_unpack(const int32_t* mat, uint8_t* codes, int height, int width) {
  int groups = height / 3;
  for (int r = 0; r < groups; r++)
    for (int j = 0; j < 32; j++)
      for (int c = 0; c < width; c++)
        codes[(size_t)(32 * r + j) * width + c] = (uint8_t)q3_code(mat, width, r, c, j);
}

/* fp32 dequant rule of VecQuant3MatMulKernel<float>: the expression
 * (scale * float(q) - zero) of kernels.h:43 is contracted by nvcc's default
 * -fmad=true into one fused multiply-add.  W is [K][width]. */
void orc_q3_dequant_f32(const int32_t* mat, const float* scales, const float* zeros,
                        float* W, int height, int width) {
  int groups = height / 3;
#pragma omp parallel for
  for (int r = 0; r < groups; r++)
    for (int j = 0; j < 32; j++)
      for (int c = 0; c < width; c++)
        W[(size_t)(32 * r + j) * width + c] =
            fmaf(scales[c], (float)q3_code(mat, width, r, c, j), -zeros[c]);
}

/* fp16 dequant rule of VecQuant3MatMulKernelFaster (kernels.h:121-122,137):
 * W = hfma(half(q), half_rn(scale), half_rn(-zero)), one fp16 rounding. */
void orc_q3_dequant_f16(const int32_t* mat, const float* scales, const float* zeros,
                        uint16_t* W, int height, int width) {
  int groups = height / 3;
#pragma omp parallel for
  for (int r = 0; r < groups; r++)
    for (int j = 0; j < 32; j++)
      for (int c = 0; c < width; c++) {
        uint16_t q = orc_f2h((float)q3_code(mat, width, r, c, j));
        W[(size_t)(32 * r + j) * width + c] =
            orc_hfma(q, orc_f2h(scales[c]), orc_f2h(-zeros[c]));
      }
}

/* mul[c] += sum_k W[k][c]*vec[k] in the reference's fp32 order
 * (kernels.h:33-89): one fp32 running sum per 256-deep K slab, each term
 * fma(fma(scale,q,-zero), vec[k], res); slabs are added to mul in slab order
 * (the reference uses atomicAdd, whose order is unspecified). */
void orc_q3_gemv_f32(const float* vec, const int32_t* mat, float* mul,
                     const float* scales, const float* zeros, int height, int width) {
  int slabs = height / 24;
#pragma omp parallel for
  for (int c = 0; c < width; c++) {
    float out = mul[c];
    for (int s = 0; s < slabs; s++) {
      float res = 0.f;
      for (int g = 0; g < 8; g++)
        for (int j = 0; j < 32; j++) {
          int r = s * 8 + g;
          float w = fmaf(scales[c], (float)q3_code(mat, width, r, c, j), -zeros[c]);
          res = fmaf(w, vec[(size_t)s * 256 + g * 32 + j], res);
        }
      out += res;
    }
    mul[c] = out;
  }
}

/* The fp16 "faster" kernel restated (kernels.h:93-169): per 32 weights a
 * half2 accumulator starts at zero, res2 = hfma2(hfma2(q2,scale,-zero),x2,res2)
 * for the 16 pairs (even k in .x, odd k in .y), then
 * res += float(res2.x) + float(res2.y) in fp32; slabs added in slab order. */
void orc_q3_gemv_f16in(const uint16_t* vec, const int32_t* mat, float* mul,
                       const float* scales, const float* zeros, int height, int width) {
  int slabs = height / 24;
#pragma omp parallel for
  for (int c = 0; c < width; c++) {
    uint16_t sc = orc_f2h(scales[c]);
    uint16_t nz = orc_f2h(-zeros[c]);
    float out = mul[c];
    for (int s = 0; s < slabs; s++) {
      float res = 0.f;
      for (int g = 0; g < 8; g++) {
        int r = s * 8 + g;
        uint16_t ax = 0, ay = 0;
        for (int p = 0; p < 16; p++) {
          uint16_t q0 = orc_f2h((float)q3_code(mat, width, r, c, 2 * p));
          uint16_t q1 = orc_f2h((float)q3_code(mat, width, r, c, 2 * p + 1));
          size_t k = (size_t)s * 256 + g * 32 + 2 * p;
          ax = orc_hfma(orc_hfma(q0, sc, nz), vec[k], ax);
          ay = orc_hfma(orc_hfma(q1, sc, nz), vec[k + 1], ay);
        }
        res += orc_h2f(ax) + orc_h2f(ay);
      }
      out += res;
    }
    mul[c] = out;
  }
}

/* fp64 truth: mul64[c] = sum_k W32[k][c]*vec[k], W32 by the fp32 dequant rule
 * (f16in = 0) or the fp16 rule (f16in = 1, vec given as fp32 values that are
 * exactly representable in fp16). */
void orc_q3_gemv_f64(const float* vec, const int32_t* mat, double* out,
                     const float* scales, const float* zeros, int height, int width,
                     int f16rule) {
  int groups = height / 3;
#pragma omp parallel for
  for (int c = 0; c < width; c++) {
    double acc = 0.0;
    uint16_t sc = orc_f2h(scales[c]), nz = orc_f2h(-zeros[c]);
    for (int r = 0; r < groups; r++)
      for (int j = 0; j < 32; j++) {
        unsigned q = q3_code(mat, width, r, c, j);
        double w = f16rule ? (double)orc_h2f(orc_hfma(orc_f2h((float)q), sc, nz))
                           : (double)fmaf(scales[c], (float)q, -zeros[c]);
        acc += w * (double)vec[(size_t)32 * r + j];
      }
    out[c] = acc;
  }
}

/* ------------------------------------------------------------------ */
/* bitsandbytes 8-bit dynamic-map blockwise quantize (quantBnB)        */
/* ------------------------------------------------------------------ */

/* dQuantize<0> restated (quantBnB-cuda/main.cu:13-66): seven-step pivot
 * search from index 127 with strides 64..1 over a 256-entry table, then a
 * midpoint test against the nearest bracket that was visited. */
static inline uint8_t bnb_quantize_one(const float* code, float x) {
  int pivot = 127, upper_pivot = 255, lower_pivot = 0;
  float lower = -1.0f, upper = 1.0f;
  float val = code[pivot];
  for (int i = 64; i > 0; i >>= 1) {
    if (x > val) { lower_pivot = pivot; lower = val; pivot += i; }
    else         { upper_pivot = pivot; upper = val; pivot -= i; }
    val = code[pivot];
  }
  if (upper_pivot == 255) upper = code[upper_pivot];
  if (lower_pivot == 0) lower = code[lower_pivot];
  if (x > val) {
    float midpoint = (upper + val) * 0.5f;
    return (uint8_t)(x > midpoint ? upper_pivot : pivot);
  } else {
    float midpoint = (lower + val) * 0.5f;
    return (uint8_t)(x < midpoint ? lower_pivot : pivot);
  }
}

/* Loop of quantBnB-omp/main.cpp:105-108,119-122 under a host parallel-for. */
void orc_bnb_quantize(const float* code, const float* A, uint8_t* out, size_t n) {
#pragma omp parallel for
  for (size_t i = 0; i < n; i++) out[i] = bnb_quantize_one(code, A[i]);
}

/* ------------------------------------------------------------------ */
/* NF4 blockwise 4-bit (no reference implementation - parity unpinned) */
/* ------------------------------------------------------------------ */

/* Semantics (ours): element e of the flattened [N][K] matrix has its 4-bit
 * code in byte e/2; with low_first == 0 the even element is the HIGH nibble,
 * with low_first != 0 it is the LOW nibble.  The 16 levels are a runtime
 * table lut16 (fp32).  One fp32 absmax per `blocksize` consecutive elements. */
static inline unsigned nf4_code(const uint8_t* B, size_t e, int low_first) {
  uint8_t b = B[e >> 1];
  int want_low = ((e & 1) != 0) ^ (low_first != 0);
  return want_low ? (b & 15u) : (b >> 4);
}

/* out[e] = half_rn( lut16[code_e] * absmax[e / blocksize] ), fp32 multiply. */
void orc_nf4_dequant_f16(const uint8_t* B, const float* absmax, const float* lut16,
                         uint16_t* out, size_t n, int blocksize, int low_first) {
#pragma omp parallel for
  for (size_t e = 0; e < n; e++)
    out[e] = orc_f2h(lut16[nf4_code(B, e, low_first)] * absmax[e / (size_t)blocksize]);
}

/* Blockwise 4-bit quantizer, the inverse of the dequantisation above (no
 * counterpart in the reference tree): absmax[b] = max |w| over the block, x = w *
 * (1 / absmax[b]) in fp32 (0 where absmax is zero, denormal or infinite), code =
 * how many of the 15 midpoints (lut16[j] + lut16[j+1]) / 2 (fp32) are < x - the
 * nearest level, a tie going to the lower one.  w: the weights widened to fp32
 * (exact for fp16 / bf16). */
void orc_nf4_quantize(const float* w, size_t n, int blocksize, const float* lut16, int low_first,
                      uint8_t* B, float* absmax) {
  float mid[15];
  for (int j = 0; j < 15; j++) mid[j] = 0.5f * (lut16[j] + lut16[j + 1]);
  for (size_t i = 0; i < n / 2; i++) B[i] = 0;
  for (size_t b = 0; b < n / (size_t)blocksize; b++) {
    float m = 0.f;
    for (int j = 0; j < blocksize; j++) {
      const float a = fabsf(w[b * blocksize + j]);
      if (a > m) m = a;
    }
    absmax[b] = m;
    const float inv = (m >= FLT_MIN && m <= FLT_MAX) ? 1.f / m : 0.f;
    for (int j = 0; j < blocksize; j++) {
      const size_t e = b * blocksize + j;
      const float x = w[e] * inv;
      unsigned code = 0;
      for (int k = 0; k < 15; k++) code += x > mid[k];
      const int low = ((e & 1) != 0) ^ (low_first != 0);
      B[e >> 1] |= (uint8_t)(low ? code : code << 4);
    }
  }
}

/* fp64 truth of the 4-bit GEMV: out[n] = sum_k A[k] * (lut16[c]*absmax) with
 * the weight taken as the exact fp32 product (not rounded to fp16). */
void orc_nf4_gemv_f64(const uint16_t* A, const uint8_t* B, const float* absmax,
                      const float* lut16, double* out, int N, int K, int blocksize,
                      int low_first) {
#pragma omp parallel for
  for (int n = 0; n < N; n++) {
    double acc = 0.0;
    for (int k = 0; k < K; k++) {
      size_t e = (size_t)n * K + k;
      float w = lut16[nf4_code(B, e, low_first)] * absmax[e / (size_t)blocksize];
      acc += (double)w * (double)orc_h2f(A[k]);
    }
    out[n] = acc;
  }
}

/* fp32-accumulating version used as the timed CPU baseline. */
void orc_nf4_gemv_f32(const uint16_t* A, const uint8_t* B, const float* absmax,
                      const float* lut16, uint16_t* out, int N, int K, int blocksize,
                      int low_first) {
  float* Af = (float*)malloc((size_t)K * sizeof(float));
  for (int k = 0; k < K; k++) Af[k] = orc_h2f(A[k]);
#pragma omp parallel for
  for (int n = 0; n < N; n++) {
    float acc = 0.f;
    size_t e0 = (size_t)n * K;
    if ((e0 % (size_t)blocksize) == 0 && (K % blocksize) == 0 && (blocksize % 2) == 0) {
      for (int kb = 0; kb < K; kb += blocksize) {
        float part = 0.f;
        const uint8_t* bp = B + ((e0 + kb) >> 1);
        for (int j = 0; j < blocksize; j += 2) {
          uint8_t b = bp[j >> 1];
          unsigned c0 = low_first ? (b & 15u) : (b >> 4);
          unsigned c1 = low_first ? (b >> 4) : (b & 15u);
          part += lut16[c0] * Af[kb + j] + lut16[c1] * Af[kb + j + 1];
        }
        acc += part * absmax[(e0 + kb) / (size_t)blocksize];
      }
    } else {
      for (int k = 0; k < K; k++) {
        size_t e = e0 + k;
        acc += lut16[nf4_code(B, e, low_first)] * absmax[e / (size_t)blocksize] * Af[k];
      }
    }
    out[n] = orc_f2h(acc);
  }
  free(Af);
}

/* ------------------------------------------------------------------ */
/* LUT-GEMM binary-coding mat-vec (lut-gemm)                           */
/* ------------------------------------------------------------------ */

/* Layouts of lut-gemm-cuda/main.cu:27-30,118-134 and nQWeight_fp16.h:24-26:
 * bW[K/32][nb][M] (bit t of a word <-> k = 32*row + t, 1 => +1, 0 => -1),
 * alpha[K/group][nb][M], q_bias[K/group][M] (nullable).  The dequantised
 * weight (main.cu:136-146, with the [K][M] layout the check intended) is
 * W[k][m] = q_bias[g][m] + sum_b alpha[g][b][m]*(2*bit-1).  Everything fp16
 * in storage; the truth is accumulated in fp64 from the exact fp16 values. */
void orc_lutgemm_dequant_f32(const uint32_t* bW, const uint16_t* alpha,
                             const uint16_t* q_bias, float* W, int M, int K, int nb,
                             int group_size) {
#pragma omp parallel for
  for (int k = 0; k < K; k++) {
    int g = k / group_size;
    for (int m = 0; m < M; m++) {
      double w = q_bias ? (double)orc_h2f(q_bias[(size_t)g * M + m]) : 0.0;
      for (int b = 0; b < nb; b++) {
        uint32_t word = bW[((size_t)(k >> 5) * nb + b) * M + m];
        double s = ((word >> (k & 31)) & 1u) ? 1.0 : -1.0;
        w += s * (double)orc_h2f(alpha[((size_t)g * nb + b) * M + m]);
      }
      W[(size_t)k * M + m] = (float)w;
    }
  }
}

/* Greedy binary-coding quantizer, W[K][M] fp32 (widened weights) -> the layouts
 * above.  No counterpart in the reference tree (it holds only the consumer).  Per
 * column and group, fp32: q_bias = half(mean) (when asked for); r = w - q_bias;
 * per plane alpha = half(mean |r|), bit = r >= 0, r -= +-alpha (the rounded
 * value).  A sum over a group is one sum per 32 consecutive inputs (ascending k)
 * and those partial sums added in ascending order. */
static float bcq_group_sum(const float* r, int n, int magnitude) {
  float s = 0.f;
  for (int k0 = 0; k0 < n; k0 += 32) {
    float p = 0.f;
    for (int k = k0; k < k0 + 32; k++) p += magnitude ? fabsf(r[k]) : r[k];
    s += p;
  }
  return s;
}
void orc_lutgemm_quantize(const float* W, int K, int M, int nb, int group_size, uint32_t* bW,
                          uint16_t* alpha, uint16_t* q_bias) {
  const int G = K / group_size;
  memset(bW, 0, (size_t)(K / 32) * nb * M * sizeof(uint32_t));
#pragma omp parallel for
  for (int m = 0; m < M; m++) {
    float* r = (float*)malloc((size_t)group_size * sizeof(float));
    for (int g = 0; g < G; g++) {
      for (int k = 0; k < group_size; k++) r[k] = W[(size_t)(g * group_size + k) * M + m];
      if (q_bias) {
        const uint16_t bh = orc_f2h(bcq_group_sum(r, group_size, 0) / (float)group_size);
        q_bias[(size_t)g * M + m] = bh;
        const float bias = orc_h2f(bh);
        for (int k = 0; k < group_size; k++) r[k] = r[k] - bias;
      }
      for (int b = 0; b < nb; b++) {
        const uint16_t ah = orc_f2h(bcq_group_sum(r, group_size, 1) / (float)group_size);
        alpha[((size_t)g * nb + b) * M + m] = ah;
        const float a = orc_h2f(ah);
        for (int k = 0; k < group_size; k++) {
          const int up = r[k] >= 0.f;
          const int kk = g * group_size + k;
          if (up) bW[((size_t)(kk >> 5) * nb + b) * M + m] |= 1u << (kk & 31);
          r[k] = r[k] - (up ? a : -a);
        }
      }
    }
    free(r);
  }
}

void orc_lutgemm_gemv_f64(const uint16_t* x, const uint32_t* bW, const uint16_t* alpha,
                          const uint16_t* q_bias, double* out, int M, int K, int nb,
                          int group_size) {
  int G = K / group_size;
  double* xs = (double*)malloc((size_t)K * sizeof(double));
  for (int k = 0; k < K; k++) xs[k] = (double)orc_h2f(x[k]);
#pragma omp parallel for
  for (int m = 0; m < M; m++) {
    double acc = 0.0;
    for (int g = 0; g < G; g++) {
      double sumx = 0.0;
      for (int k = g * group_size; k < (g + 1) * group_size; k++) sumx += xs[k];
      if (q_bias) acc += (double)orc_h2f(q_bias[(size_t)g * M + m]) * sumx;
      for (int b = 0; b < nb; b++) {
        double pos = 0.0; /* sum of x where bit = 1 */
        for (int k = g * group_size; k < (g + 1) * group_size; k++) {
          uint32_t word = bW[((size_t)(k >> 5) * nb + b) * M + m];
          if ((word >> (k & 31)) & 1u) pos += xs[k];
        }
        acc += (double)orc_h2f(alpha[((size_t)g * nb + b) * M + m]) * (2.0 * pos - sumx);
      }
    }
    out[m] = acc;
  }
  free(xs);
}

/* fp32 version for CPU timing (same loop nest, float accumulators). */
void orc_lutgemm_gemv_f32(const uint16_t* x, const uint32_t* bW, const uint16_t* alpha,
                          const uint16_t* q_bias, uint16_t* out, int M, int K, int nb,
                          int group_size) {
  int G = K / group_size;
  float* xs = (float*)malloc((size_t)K * sizeof(float));
  for (int k = 0; k < K; k++) xs[k] = orc_h2f(x[k]);
#pragma omp parallel for
  for (int m = 0; m < M; m++) {
    float acc = 0.f;
    for (int g = 0; g < G; g++) {
      float sumx = 0.f;
      for (int k = g * group_size; k < (g + 1) * group_size; k++) sumx += xs[k];
      if (q_bias) acc += orc_h2f(q_bias[(size_t)g * M + m]) * sumx;
      for (int b = 0; b < nb; b++) {
        float pos = 0.f;
        for (int k0 = g * group_size; k0 < (g + 1) * group_size; k0 += 32) {
          uint32_t word = bW[((size_t)(k0 >> 5) * nb + b) * M + m];
          int lim = (g + 1) * group_size - k0;
          if (lim > 32) lim = 32;
          for (int t = 0; t < lim; t++)
            if ((word >> t) & 1u) pos += xs[k0 + t];
        }
        acc += orc_h2f(alpha[((size_t)g * nb + b) * M + m]) * (2.f * pos - sumx);
      }
    }
    out[m] = orc_f2h(acc);
  }
  free(xs);
}

/* ------------------------------------------------------------------ */
/* AQLM additive codebooks (quantAQLM)                                 */
/* ------------------------------------------------------------------ */

/* Code1x16MatVec restated bit for bit (quantAQLM-cuda/main.cu:39-108).
 * Row m has prob_k/8 uint16 codes, read as int4 (8 codes); lane l of the
 * row's warp takes int4 indices l, l+32, ...; code i of int4 idx multiplies
 * inputs 8*(8*idx+i)..+7 with four fp16 hfma2 (main.cu:94-96), whose two
 * halves are added to the lane's fp32 sum (:97); lanes are combined with the
 * shfl_down tree 16,8,4,2,1 (:106); lane 0 stores half_rn (:108).  The
 * codebook of a row is picked by the cumulative row ranges cb_sizes
 * (:43-51).  `scales` (nullable, fp16 per output) is OUR extension: the fp32
 * sum is multiplied by float(scale[m]) before the final rounding. */
void orc_aqlm_1x16_ref(const uint16_t* codes, const uint16_t* x, uint16_t* out,
                       const uint16_t* codebook, int prob_m, int prob_k,
                       const int* cb_sizes, int cb_stride_int4, const uint16_t* scales) {
  int n_int4 = prob_k / 64; /* int4 per row */
#pragma omp parallel for
  for (int m = 0; m < prob_m; m++) {
    const uint16_t* cb = codebook;
    int s = 0;
    while (s < 3 && m >= cb_sizes[s]) { cb += (size_t)cb_stride_int4 * 8; s++; }
    float lane[32];
    for (int l = 0; l < 32; l++) {
      float res = 0.f;
      for (int idx = l; idx < n_int4; idx += 32) {
        for (int i = 0; i < 8; i++) {
          uint16_t code = codes[(size_t)m * (prob_k / 8) + (size_t)idx * 8 + i];
          const uint16_t* a = cb + (size_t)code * 8;
          const uint16_t* b = x + (size_t)8 * (8 * idx + i);
          uint16_t rx = 0, ry = 0;
          for (int j = 0; j < 4; j++) {
            rx = orc_hfma(a[2 * j], b[2 * j], rx);
            ry = orc_hfma(a[2 * j + 1], b[2 * j + 1], ry);
          }
          res += orc_h2f(rx) + orc_h2f(ry);
        }
      }
      lane[l] = res;
    }
    for (int off = 16; off > 0; off >>= 1)
      for (int l = 0; l < off; l++) lane[l] += lane[l + off];
    float r = lane[0];
    if (scales) r *= orc_h2f(scales[m]);
    out[m] = orc_f2h(r);
  }
}

/* fp64 truth for 1x16 (same indexing, exact products). */
void orc_aqlm_1x16_f64(const uint16_t* codes, const uint16_t* x, double* out,
                       const uint16_t* codebook, int prob_m, int prob_k,
                       const int* cb_sizes, int cb_stride_int4, const uint16_t* scales) {
  int groups = prob_k / 8;
#pragma omp parallel for
  for (int m = 0; m < prob_m; m++) {
    const uint16_t* cb = codebook;
    int s = 0;
    while (s < 3 && m >= cb_sizes[s]) { cb += (size_t)cb_stride_int4 * 8; s++; }
    double acc = 0.0;
    for (int g = 0; g < groups; g++) {
      const uint16_t* a = cb + (size_t)codes[(size_t)m * groups + g] * 8;
      for (int j = 0; j < 8; j++)
        acc += (double)orc_h2f(a[j]) * (double)orc_h2f(x[(size_t)8 * g + j]);
    }
    if (scales) acc *= (double)orc_h2f(scales[m]);
    out[m] = acc;
  }
}

/* AQLM 2x8 (no reference implementation - parity unpinned).  Semantics
 * (ours): codes uint8[prob_m][prob_k/8][2]; codebooks fp16[2][256][8];
 * out[m] = scale[m] * sum_g sum_{c<2} codebooks[c][codes[m][g][c]] . x[8g..8g+7]. */
void orc_aqlm_2x8_f64(const uint8_t* codes, const uint16_t* x, double* out,
                      const uint16_t* codebooks, int prob_m, int prob_k,
                      const uint16_t* scales) {
  int groups = prob_k / 8;
#pragma omp parallel for
  for (int m = 0; m < prob_m; m++) {
    double acc = 0.0;
    for (int g = 0; g < groups; g++)
      for (int c = 0; c < 2; c++) {
        const uint16_t* a =
            codebooks + ((size_t)c * 256 + codes[((size_t)m * groups + g) * 2 + c]) * 8;
        for (int j = 0; j < 8; j++)
          acc += (double)orc_h2f(a[j]) * (double)orc_h2f(x[(size_t)8 * g + j]);
      }
    if (scales) acc *= (double)orc_h2f(scales[m]);
    out[m] = acc;
  }
}

/* fp32 versions for CPU timing. */
void orc_aqlm_1x16_f32(const uint16_t* codes, const uint16_t* x, uint16_t* out,
                       const uint16_t* codebook, int prob_m, int prob_k,
                       const int* cb_sizes, int cb_stride_int4, const uint16_t* scales) {
  int groups = prob_k / 8;
  float* xs = (float*)malloc((size_t)prob_k * sizeof(float));
  for (int k = 0; k < prob_k; k++) xs[k] = orc_h2f(x[k]);
#pragma omp parallel for
  for (int m = 0; m < prob_m; m++) {
    const uint16_t* cb = codebook;
    int s = 0;
    while (s < 3 && m >= cb_sizes[s]) { cb += (size_t)cb_stride_int4 * 8; s++; }
    float acc = 0.f;
    for (int g = 0; g < groups; g++) {
      const uint16_t* a = cb + (size_t)codes[(size_t)m * groups + g] * 8;
      for (int j = 0; j < 8; j++) acc += orc_h2f(a[j]) * xs[8 * g + j];
    }
    if (scales) acc *= orc_h2f(scales[m]);
    out[m] = orc_f2h(acc);
  }
  free(xs);
}

/* ------------------------------------------------------------------ */
/* Batched dequant-GEMM (no reference implementation - parity unpinned)*/
/* ------------------------------------------------------------------ */

/* Y[Mb][N] = X[Mb][K] * Wd[K][N] in fp64 from fp16 operands; Wd is a
 * dequantised fp16 weight matrix produced by one of the dequant rules above
 * (row-major [K][N]). */
void orc_gemm_f16_f64(const uint16_t* X, const uint16_t* Wd, double* Y, int Mb, int N,
                      int K) {
#pragma omp parallel for
  for (int n0 = 0; n0 < N; n0 += 64) {
    int n1 = n0 + 64 < N ? n0 + 64 : N;
    for (int i = 0; i < Mb; i++) {
      double acc[64];
      for (int n = n0; n < n1; n++) acc[n - n0] = 0.0;
      for (int k = 0; k < K; k++) {
        double xv = (double)orc_h2f(X[(size_t)i * K + k]);
        const uint16_t* wr = Wd + (size_t)k * N;
        for (int n = n0; n < n1; n++) acc[n - n0] += xv * (double)orc_h2f(wr[n]);
      }
      for (int n = n0; n < n1; n++) Y[(size_t)i * N + n] = acc[n - n0];
    }
  }
}

/* Same with Wd stored [N][K] (the NF4 dequant output orientation). */
void orc_gemm_f16_nk_f64(const uint16_t* X, const uint16_t* Wd, double* Y, int Mb, int N,
                         int K) {
#pragma omp parallel for
  for (int n = 0; n < N; n++)
    for (int i = 0; i < Mb; i++) {
      double acc = 0.0;
      for (int k = 0; k < K; k++)
        acc += (double)orc_h2f(X[(size_t)i * K + k]) * (double)orc_h2f(Wd[(size_t)n * K + k]);
      Y[(size_t)i * N + n] = acc;
    }
}

/* Group-wise 3-bit dequant for the batched path (ours): same packed layout as
 * quant3MatMul (mat[K*3/32][N]); per-group fp16 scale and zero,
 * scales/zeros[K/group][N]; W[k][n] = hfma(half(q), scale, -zero) in fp16
 * (the rule of kernels.h:121-122,137 with the column parameters replaced by
 * the (group, column) ones). */
void orc_q3g_dequant_f16(const int32_t* mat, const uint16_t* scales, const uint16_t* zeros,
                         uint16_t* W, int K, int N, int group) {
#pragma omp parallel for
  for (int k = 0; k < K; k++) {
    int g = k / group;
    for (int n = 0; n < N; n++) {
      uint16_t q = orc_f2h((float)q3_code(mat, N, k >> 5, n, k & 31));
      uint16_t z = zeros[(size_t)g * N + n] ^ 0x8000u;
      W[(size_t)k * N + n] = orc_hfma(q, scales[(size_t)g * N + n], z);
    }
  }
}

/* ------------------------------------------------------------------------
 * gemv: uniform int8 / int4 weight-only mat-vec.  Restates the device-side
 * checks of gemv-cuda/gemv.cu:98-114 (int8) and :116-141 (int4) - the only
 * statement of the expected result in the reference: the weight is dequantised
 * in fp32 as (float(w) - float(zero_point_half)) * float(scale_half) - with the
 * accumulation carried in fp64 here.  bits = 16 (fp16 matrix, gemv.cu:83-96),
 * 8 (int8) or 4 (two codes per byte, element 2j in the low nibble:
 * kernels.h:17-23).  scale and zero_point arrive as fp16 bit patterns, which
 * is what the reference launchers make of their float arguments
 * (gemv.cu:21-22).
 * ------------------------------------------------------------------------ */
void orc_gemv_uniform_f64(const void* mat, const uint16_t* vec, double* out, int rows, int n,
                          int bits, uint16_t scale_h, uint16_t zero_h) {
  const float scale = orc_h2f(scale_h), zp = orc_h2f(zero_h);
#pragma omp parallel for
  for (int r = 0; r < rows; r++) {
    double acc = 0.0;
    for (int j = 0; j < n; j++) {
      float w;
      if (bits == 16) {
        w = orc_h2f(((const uint16_t*)mat)[(size_t)r * n + j]);
      } else if (bits == 8) {
        w = ((float)((const int8_t*)mat)[(size_t)r * n + j] - zp) * scale;
      } else {
        const uint8_t b = ((const uint8_t*)mat)[(size_t)r * (n / 2) + j / 2];
        w = ((float)((j & 1) ? (b >> 4) : (b & 15)) - zp) * scale;
      }
      acc += (double)w * (double)orc_h2f(vec[j]);
    }
    out[r] = acc;
  }
}

/* ------------------------------------------------------------------------
 * RMSNorm -> weight-only mat-vec -> gated activation, in fp64.  Restates
 * rmsnorm-cuda/reference.h:4-25 (xn = x * 1/sqrt(mean(x^2) + eps) * gamma; no
 * rounding of xn here), the mat-vec of the format (fmt 16 / 8 / 4 as
 * orc_gemv_uniform_f64, fmt 40 = NF4 as orc_nf4_gemv_f64) and, for act != 0,
 * the pairing of geglu-cuda/reference.h:8-16 per output feature (row 2m the
 * value, row 2m + 1 the gate) with act 1: v * g / (1 + exp(-g))
 * (swish-cuda/reference.h:4), act 2: v * 0.5 * g * (1 + erf(g / sqrt 2))
 * (geglu-cuda/reference.h:1-5).  gamma == NULL: no normalisation.
 * ------------------------------------------------------------------------ */
void orc_gemv_fused_f64(int fmt, const void* mat, const float* absmax, const float* lut16,
                        int low_first, int blocksize, const uint16_t* x, const uint16_t* gamma,
                        double eps, double* out, int rows_out, int n, int act, uint16_t scale_h,
                        uint16_t zero_h) {
  double* xn = (double*)malloc((size_t)n * sizeof(double));
  double ms = 0.0;
  for (int k = 0; k < n; k++) {
    const double v = (double)orc_h2f(x[k]);
    ms += v * v;
  }
  const double s = gamma ? 1.0 / sqrt(ms / n + eps) : 1.0;
  for (int k = 0; k < n; k++)
    xn[k] = (double)orc_h2f(x[k]) * s * (gamma ? (double)orc_h2f(gamma[k]) : 1.0);
  const float scale = orc_h2f(scale_h), zp = orc_h2f(zero_h);
  const int rows_mat = act ? 2 * rows_out : rows_out;
  double* y = (double*)malloc((size_t)rows_mat * sizeof(double));
#pragma omp parallel for
  for (int r = 0; r < rows_mat; r++) {
    double acc = 0.0;
    for (int j = 0; j < n; j++) {
      float w;
      if (fmt == 16) {
        w = orc_h2f(((const uint16_t*)mat)[(size_t)r * n + j]);
      } else if (fmt == 8) {
        w = ((float)((const int8_t*)mat)[(size_t)r * n + j] - zp) * scale;
      } else if (fmt == 4) {
        const uint8_t b = ((const uint8_t*)mat)[(size_t)r * (n / 2) + j / 2];
        w = ((float)((j & 1) ? (b >> 4) : (b & 15)) - zp) * scale;
      } else {
        const size_t e = (size_t)r * n + j;
        w = lut16[nf4_code((const uint8_t*)mat, e, low_first)] * absmax[e / (size_t)blocksize];
      }
      acc += (double)w * xn[j];
    }
    y[r] = acc;
  }
  for (int m = 0; m < rows_out; m++) {
    if (!act) {
      out[m] = y[m];
    } else {
      const double v = y[2 * m], g = y[2 * m + 1];
      out[m] = act == 1 ? v * g / (1.0 + exp(-g)) : v * 0.5 * g * (1.0 + erf(g * 0.70710678118654752440));
    }
  }
  free(y);
  free(xn);
}

/* ------------------------------------------------------------------------
 * MXFP4 quantize-dequantize (mxfp4-cuda/main.cu:112-150) and its packed form.
 * T is fp16 (bf16 = 0) or bf16 (bf16 = 1), passed as 16-bit patterns.
 * ------------------------------------------------------------------------ */
static inline float orc_bf2f(uint16_t b) {
  union { uint32_t u; float f; } v;
  v.u = (uint32_t)b << 16;
  return v.f;
}
static inline uint16_t orc_f2bf(float f) { /* round to nearest even */
  union { uint32_t u; float f; } v;
  v.f = f;
  if ((v.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((v.u >> 16) | 0x40u);
  return (uint16_t)((v.u + 0x7fffu + ((v.u >> 16) & 1u)) >> 16);
}
static inline float mx_t2f(uint16_t b, int bf16) { return bf16 ? orc_bf2f(b) : orc_h2f(b); }
static inline uint16_t mx_d2t(double d, int bf16) { return bf16 ? orc_f2bf((float)d) : orc_d2h(d); }

/* One value of T, already divided by the group's scale, rounded to the e2m1
 * grid and returned in T's encoding: the bit procedure of fp16_to_fp4_simulate
 * (main.cu:21-109) - E exponent bits, M mantissa bits, bias B.  The rounding
 * looks at the mantissa bits e2m1 drops (one more per binade below e2m1's
 * smallest normal, the lowest exponent bit standing in for the implicit one),
 * goes to the nearer neighbour and on a tie to the even mantissa; results are
 * clamped to the binades 2^-1 .. 2^2 and magnitudes beyond 6 become 6. */
static uint16_t mx_round_e2m1(uint16_t bits, int E, int M, int B) {
  const int exp = (bits >> M) & ((1 << E) - 1);
  const int sign = (bits >> (M + E)) & 1;
  const int top = (bits >> (M - 1)) & 1; /* the one mantissa bit e2m1 keeps */
  const int e4 = exp - B + 1;            /* exponent in e2m1's bias (main.cu:32-33) */
  const int below = e4 <= 0 ? 1 - e4 : 0;
  int cut = M - 1 + below;               /* bits the rounding discards (main.cu:39) */
  if (cut > 16) cut = 16;
  const uint32_t tail = (bits & ((1u << (M + 1)) - 1u)) & ((1u << cut) - 1u);
  const uint32_t half = 1u << (cut - 1);
  int new_exp, new_man;
  if (tail < half) { /* towards zero (main.cu:68-69) */
    new_exp = exp;
    new_man = e4 > 0 ? top : 0;
  } else if (tail > half) { /* away from zero (main.cu:82-83) */
    new_exp = exp + ((e4 <= 0 || top) ? 1 : 0);
    new_man = (e4 > 0 && !top) ? 1 : 0;
  } else { /* tie: to the even mantissa; .25 goes to 0 (main.cu:93) */
    new_exp = exp > B - 2 ? exp + top : 0;
    new_man = 0;
  }
  if (new_exp > B + 2 && new_man == 0) new_man = 1; /* main.cu:101 */
  if (new_exp < B - 2) new_exp = 0;                 /* main.cu:104 */
  else if (new_exp > B + 2) new_exp = B + 2;
  return (uint16_t)((sign << 15) | (new_exp << M) | (new_man << (M - 1)));
}

/* exponent k of the scale of one group from its largest magnitude (T's bits):
 * mantissa rounded up from 1.75 by adding a quarter of the mantissa range to the
 * bits and keeping the exponent field (main.cu:127-129), floor(log2) - 2,
 * clamped to E8M0's range (main.cu:131-135).  A field of 0 (a zero or small
 * denormal maximum, for which the reference takes log2 of zero) counts as 1,
 * the smallest field the reference's expression is defined for. */
static int mx_scale_exponent(uint16_t max_bits, int bf16) {
  const int M = bf16 ? 7 : 10, B = bf16 ? 127 : 15;
  int field = (int)(((uint32_t)max_bits + (1u << (M - 2))) >> M);
  if (field < 1) field = 1;
  int k = field - B - 2;
  if (k < -127) k = -127;
  if (k > 127) k = 127;
  return k;
}
/* the same from T's own bits, as the reference does it; -1000 where the
 * reference's expression is undefined (log2 of zero) */
int orc_mxfp4_scale_exponent_ref(uint16_t max_bits, int bf16) {
  const int M = bf16 ? 7 : 10, E = bf16 ? 8 : 5, B = bf16 ? 127 : 15;
  const uint32_t r = ((uint32_t)max_bits + (1u << (M - 2))) & (((1u << (E + 1)) - 1u) << M);
  const int exp = (int)(r >> M) & ((1 << E) - 1);
  if (exp == 0) return -1000;
  int k = exp - B - 2;
  if (k > 127) k = 127;
  if (k < -127) k = -127;
  return k;
}
int orc_mxfp4_scale_exponent(uint16_t max_bits, int bf16) { return mx_scale_exponent(max_bits, bf16); }

/* out (T) = quantize-dequantize of in; codes / scales (nullable): the packed
 * form, element 2j in the low nibble, nibble = sign << 3 | grid index, scale
 * byte = k + 127. */
void orc_mxfp4(const uint16_t* in, uint16_t* out, uint8_t* codes, uint8_t* scales, size_t numel,
               int bf16) {
  const int M = bf16 ? 7 : 10, E = bf16 ? 8 : 5, B = bf16 ? 127 : 15;
#pragma omp parallel for
  for (long long g = 0; g < (long long)(numel / 32); g++) {
    const uint16_t* x = in + (size_t)g * 32;
    uint16_t mx = 0;
    for (int j = 0; j < 32; j++) {
      const uint16_t a = x[j] & 0x7fffu;
      if (a > mx) mx = a;
    }
    const int k = mx_scale_exponent(mx, bf16);
    if (scales) scales[g] = (uint8_t)(k + 127);
    for (int j = 0; j < 32; j++) {
      /* x / scale in T (exact, or a denormal of T, which rounds to 0 below) */
      const uint16_t a = mx_d2t(ldexp((double)mx_t2f(x[j], bf16), -k), bf16);
      const uint16_t q = mx_round_e2m1(a, E, M, B);
      if (out) out[(size_t)g * 32 + j] = mx_d2t(ldexp((double)mx_t2f(q, bf16), k), bf16);
      if (codes) {
        const float mag = fabsf(mx_t2f(q, bf16));
        const int idx = mag < 2.f ? (int)(mag * 2.f) : (mag < 4.f ? (int)mag + 2 : (int)(mag / 2.f) + 4);
        const uint8_t nib = (uint8_t)(((q >> 15) << 3) | idx);
        uint8_t* c = codes + ((size_t)g * 32 + j) / 2;
        if (j & 1) *c = (uint8_t)((*c & 0x0f) | (nib << 4));
        else *c = (uint8_t)((*c & 0xf0) | nib);
      }
    }
  }
}

/* packed form -> T */
void orc_mxfp4_dequant(const uint8_t* codes, const uint8_t* scales, uint16_t* out, size_t numel,
                       int bf16) {
  static const float grid[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  for (size_t i = 0; i < numel; i++) {
    const uint8_t nib = (i & 1) ? (codes[i / 2] >> 4) : (codes[i / 2] & 15);
    const double v = ldexp((double)grid[nib & 7], (int)scales[i / 32] - 127);
    out[i] = mx_d2t((nib & 8) ? -v : v, bf16);
  }
}

/* ------------------------------------------------------------------------
 * Scale and zero point per channel from its minimum and maximum: restates
 * zeropoint-cuda/reference.h:1-71 (the kernel main.cu:10-80 is the same
 * arithmetic).  The mixed fp32 / fp64 arithmetic is the reference's.
 * ------------------------------------------------------------------------ */
void orc_zero_point(const float* x_min, const float* x_max, int32_t qmin, int32_t qmax, int size,
                    int preserve_sparsity, float* scale, int32_t* zero_point) {
  const int span = qmax - qmin;
  const int sym_lo = -(span / 2 + 1), sym_hi = span / 2;
  for (int i = 0; i < size; i++) {
    float lo = x_min[i], hi = x_max[i];
    if (preserve_sparsity && lo < 0 && hi > 0) { /* reference.h:15-22 */
      const float a = fabsf(lo / (float)sym_lo), b = fabsf(hi / (float)sym_hi);
      const double m = (double)(a > b ? a : b);
      lo = (float)(m * (double)sym_lo);
      hi = (float)(m * (double)sym_hi);
    }
    if (!(lo < 0.f)) lo = 0.f; /* reference.h:27-28: the range contains 0 */
    if (!(hi > 0.f)) hi = 0.f;
    float sc = (float)(((double)hi - (double)lo) / (double)span); /* reference.h:29 */
    if (sc == 0.f || isinf(1.f / sc)) sc = 0.1f;                  /* reference.h:33-35 */
    const double s = (double)sc;
    const double from_lo = (double)qmin - (double)lo / s, from_hi = (double)qmax - (double)hi / s;
    const double err_lo = (double)abs(qmin) + fabs((double)lo / s);
    const double err_hi = (double)abs(qmax) + fabs((double)hi / s);
    double z = err_lo < err_hi ? from_lo : from_hi; /* reference.h:37-46 */
    if (preserve_sparsity && lo < 0 && hi > 0) z = (double)(qmin + qmax) / 2.0; /* :52-54 */
    int32_t nudged;
    if (z < (double)qmin) nudged = qmin;
    else if (z > (double)qmax) nudged = qmax;
    else nudged = (int32_t)nearbyint(z); /* reference.h:60-67 */
    scale[i] = sc;
    zero_point[i] = nudged;
  }
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------
 * Per-token int8 activation quantization (quantVLLM).  Restates the host
 * reference loops of quantVLLM-cuda/reference.h:1-93 with the helpers of
 * quantVLLM-cuda/utils.h:9-63 (float_to_int8_rn, float_to_int32_rn,
 * int32_to_int8); the CUDA kernels of main.cu:12-134 compute the same values
 * and the reference driver compares the two with memcmp (main.cu:222-267).
 * dtype: 0 = fp16, 1 = bf16, 2 = fp32 input.  Conversions of NaN to an integer,
 * undefined in the host reference, give 0 here (what the device gives).
 * ------------------------------------------------------------------------ */
static inline float vllm_in(const void* in, int dtype, size_t i) {
  if (dtype == 0) return orc_h2f(((const uint16_t*)in)[i]);
  if (dtype == 1) {
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)((const uint16_t*)in)[i] << 16;
    return v.f;
  }
  return ((const float*)in)[i];
}
/* utils.h:9-28 */
static inline int8_t vllm_f2i8_rn(float x) {
  float dst = nearbyintf(x);
  if (dst != dst) return 0;
  dst = dst < -128.0f ? -128.0f : (127.0f < dst ? 127.0f : dst);
  return (int8_t)dst;
}
/* utils.h:30-53 */
static inline int32_t vllm_f2i32_rn(float x) {
  float dst = nearbyintf(x);
  if (dst != dst) return 0;
  if (dst >= 2147483648.0f) return INT32_MAX;
  if (dst <= -2147483648.0f) return INT32_MIN;
  return (int32_t)dst;
}
/* utils.h:55-63 */
static inline int8_t vllm_i32_to_i8(int32_t x) {
  return (int8_t)(x < -128 ? -128 : (127 < x ? 127 : x));
}

/* reference.h:1-31: azp == 0 selects the form without zero point, as the
 * launcher does (main.cu:147-152) */
void orc_vllm_static_quant(const void* in, int dtype, int8_t* out, float scale, int32_t azp,
                           long long num_tokens, int hidden) {
#pragma omp parallel for
  for (long long t = 0; t < num_tokens; t++)
    for (int i = 0; i < hidden; i++) {
      size_t idx = (size_t)t * hidden + i;
      float val = vllm_in(in, dtype, idx);
      if (azp == 0) out[idx] = vllm_f2i8_rn(val / scale);
      else out[idx] = vllm_i32_to_i8((int32_t)((uint32_t)vllm_f2i32_rn(val / scale) + (uint32_t)azp));
    }
}

/* reference.h:33-58 (azp_out == NULL) and :60-93 */
void orc_vllm_dynamic_quant(const void* in, int dtype, int8_t* out, float* scale_out,
                            int32_t* azp_out, long long num_tokens, int hidden) {
#pragma omp parallel for
  for (long long t = 0; t < num_tokens; t++) {
    size_t row = (size_t)t * hidden;
    if (azp_out == NULL) {
      float absmax_val = 0.0f;
      for (int i = 0; i < hidden; i++) {
        float val = vllm_in(in, dtype, row + i);
        val = val > 0.0f ? val : -val;
        absmax_val = val > absmax_val ? val : absmax_val;
      }
      scale_out[t] = absmax_val / 127.0f;
      float tmp_scale = 127.0f / absmax_val;
      for (int i = 0; i < hidden; i++)
        out[row + i] = vllm_f2i8_rn(vllm_in(in, dtype, row + i) * tmp_scale);
    } else {
      /* the reference starts the maximum at the smallest positive normal float */
      float max_val = FLT_MIN, min_val = FLT_MAX;
      for (int i = 0; i < hidden; i++) {
        float val = vllm_in(in, dtype, row + i);
        max_val = max_val < val ? val : max_val;
        min_val = val < min_val ? val : min_val;
      }
      float scale_val = (max_val - min_val) / 255.0f;
      float azp_float = nearbyintf(-128.0f - min_val / scale_val);
      int32_t azp_val = azp_float != azp_float ? 0 : (int32_t)azp_float;
      scale_out[t] = scale_val;
      azp_out[t] = azp_val;
      for (int i = 0; i < hidden; i++) {
        float val = vllm_in(in, dtype, row + i);
        out[row + i] =
            vllm_i32_to_i8((int32_t)((uint32_t)vllm_f2i32_rn(val / scale_val) + (uint32_t)azp_val));
      }
    }
  }
}
