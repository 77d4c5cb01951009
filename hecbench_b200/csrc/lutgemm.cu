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
//  * a CTA of 512 threads owns a K tile of 128 inputs (4 packed rows; 64 inputs
//    for alpha groups of 192, 320, ... inputs) and a range of columns; lane
//    (c,j) of a warp handles byte j of the words of columns 4c..4c+3 and reads
//    replica c of table (row, j): the 16 tables are stored with one 256-byte
//    line per (row pair, byte value) holding [row parity][replica c][byte-lane
//    j], so every lane of a warp reads its own bank - no lookup ever conflicts
//    - and, the table block sitting at a FIXED address of the shared window,
//    the address of a lookup is ONE byte-permute of the packed word and a
//    per-lane constant, plus an immediate offset that selects the row;
//  * shared memory carries the lookups and nothing else: packed words, alphas
//    and bias go from global memory straight into registers (128-bit streaming
//    loads, the four lanes of a column quad reading the same 16 bytes), one
//    column step ahead of their use, and the first step is requested before
//    the tables are built;
//  * table entries and all sums are fp32 (the reference uses fp16 throughout
//    and half2 atomics on the output);
//  * the four lanes of a column quad are combined with two shuffles, each CTA
//    adds its tile's partial sums to an fp32 scratch row with one 16-byte
//    vector reduction per column quad, and the last CTA of each column range to
//    finish converts that range of the scratch to fp16, stores the output and
//    re-zeroes the scratch.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "hq_common.cuh"

namespace hq {
namespace {

// CTA shapes: 512 threads with a 128-input tile (one CTA per SM), or 256 threads
// with a 64-input tile and two CTAs per SM - the two then run out of phase, one
// streaming packed words while the other builds its tables.
// Shared-window address at which a CTA's dynamic region starts: the 1 KiB the
// system reserves per CTA (the kernels have no static shared memory).  The
// host checks the device attribute before launching; kSlack bytes of padding
// absorb a start up to kSlack later.
constexpr int kDynBase = 1024;
constexpr int kSlack = 256;
// completion counters at the end of the workspace: one per column range
constexpr int kCounterWords = 64;

// Compile-time layout of one variant.  TR: packed rows (32 inputs each) per K
// tile.  Dynamic shared memory:
//   [flag 16 B][build scratch: compact tables + inputs][padding][tables TR/2 x 64 KiB]
// The tables start at the FIXED shared-window address kLutImm so that the
// address of a lookup is a byte-permute plus an immediate.
template <int TR>
struct Layout {
  static constexpr int kCompactWords = TR * 256 * 4;  // [row][byte value][j]
  static constexpr int kBuildBytes = kCompactWords * 4 + TR * 32 * 4;
  static constexpr int kFlagBytes = 16;
  static constexpr int kLutBytes = (TR / 2) * 65536;
  static constexpr int kLutImm = (kDynBase + kSlack + kFlagBytes + kBuildBytes + 255) / 256 * 256;
  static constexpr int kSmem = kLutImm - kDynBase + kLutBytes;
  static_assert(kSmem <= 227 * 1024, "shared memory budget");
};

__device__ __forceinline__ void red_add_v4_f32(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}
template <int IMM>
__device__ __forceinline__ float lds_f32_imm(uint32_t addr) {
  // not volatile: the tables are constant once built, so the scheduler is free
  // to batch these loads
  float v;
  asm("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(IMM));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// One launch handles NB bit planes b0 .. b0+NB-1 of nb_total (more planes than
// fit the register budget are split over launches that accumulate into the
// same scratch row; only the last one converts it).  RPG: packed rows that
// share one alpha group inside a tile.  counters: one completion counter per
// column range (per_range != 0) or a single one.
template <int TR, int NB, int RPG, int kThreads>
__global__ void __launch_bounds__(kThreads, (kThreads == 256 ? 2 : 1))
lutgemm_kernel(const uint32_t* __restrict__ bW, const __half* __restrict__ alpha,
               const __half* __restrict__ q_bias, const __half* __restrict__ x,
               __half* __restrict__ out, float* __restrict__ ws, unsigned* __restrict__ counters,
               int M, int K, int rows_per_group, int cols_per_cta, int nb_total, int b0,
               int finalize, int per_range) {
  using L = Layout<TR>;
  constexpr int kWarps = kThreads / 32;
  constexpr int kGroups = TR / RPG;
  constexpr int kLutImm = L::kLutImm;
  extern __shared__ __align__(16) unsigned char dsm[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t dsm_addr = (uint32_t)__cvta_generic_to_shared(dsm);
  // the host has checked where the dynamic region starts; never taken
  if (dsm_addr < (uint32_t)kDynBase || dsm_addr > (uint32_t)(kDynBase + kSlack)) return;
  unsigned char* lut = dsm + ((uint32_t)kLutImm - dsm_addr);
  unsigned* s_last = reinterpret_cast<unsigned*>(dsm);
  float* compact = reinterpret_cast<float*>(dsm + L::kFlagBytes);
  float* xs = compact + L::kCompactWords;  // the tile's inputs
  const int tile = blockIdx.y;
  const int row0 = tile * TR;  // first packed row of the tile
  const int total_rows = K >> 5;
  const int nrows = min(TR, total_rows - row0);
  const int m_begin = blockIdx.x * cols_per_cta;
  const int m_end = min(M, m_begin + cols_per_cta);
  const int g0 = row0 / rows_per_group;  // alpha group of the tile's first row

  // ---- stage the tile's inputs (zero beyond K) ----
  if (tid < TR * 32) {
    const int k = row0 * 32 + tid;
    xs[tid] = (k < K && HQ_IN_BOUNDS(x + k, 2, x, (size_t)K * 2, 206)) ? __half2float(x[k]) : 0.f;
  }
  // ---- column steps of this warp: step s handles columns m0 + s*kWarps*32 ..+3 ----
  const int j = lane & 3;   // byte of the word this lane looks up
  const int cq = lane >> 2; // column quad inside the 32-column step
  const int m0 = m_begin + warp * 32 + cq * 4;
  const int nsteps = (m_end - (m_begin + warp * 32) + kWarps * 32 - 1) / (kWarps * 32);
  const uint32_t* src0 = bW + ((size_t)row0 * nb_total + b0) * M + m0;

  uint4 wv[TR][NB];
  uint2 av[kGroups][NB + 1];
#pragma unroll
  for (int r = 0; r < TR; r++)
#pragma unroll
    for (int b = 0; b < NB; b++) wv[r][b] = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int gi = 0; gi < kGroups; gi++)
#pragma unroll
    for (int b = 0; b <= NB; b++) av[gi][b] = make_uint2(0, 0);

  // packed words of row r for the step whose first column (for this quad) is m
  // extents of the caller's buffers, used only by the index-checked build
  const size_t bw_bytes = (size_t)total_rows * nb_total * M * 4;
  const size_t alpha_bytes = (size_t)(total_rows / rows_per_group) * nb_total * M * 2;
  const size_t bias_bytes = (size_t)(total_rows / rows_per_group) * M * 2;
  (void)bw_bytes; (void)alpha_bytes; (void)bias_bytes;
  auto load_row = [&](int r, int m) {
    if (r < nrows) {
#pragma unroll
      for (int b = 0; b < NB; b++) {
        const uint32_t* src = src0 + (size_t)(r * nb_total + b) * M + (m - m0);
        if (HQ_IN_BOUNDS(src, 16, bW, bw_bytes, 201)) wv[r][b] = ldg_stream_u4(src);
      }
    }
  };
  auto load_group = [&](int gi, int m) {
    if (gi * RPG < nrows) {
      const int g = g0 + gi;
#pragma unroll
      for (int b = 0; b < NB; b++) {
        const __half* src = alpha + ((size_t)g * nb_total + b0 + b) * M + m;
        if (HQ_IN_BOUNDS(src, 8, alpha, alpha_bytes, 202)) av[gi][b] = ldg_nc_u2(src);
      }
      if (q_bias != nullptr && HQ_IN_BOUNDS(q_bias + (size_t)g * M + m, 8, q_bias, bias_bytes, 203))
        av[gi][NB] = ldg_nc_u2(q_bias + (size_t)g * M + m);
    }
  };
  if (nsteps > 0 && m0 < m_end) {
#pragma unroll
    for (int r = 0; r < TR; r++) load_row(r, m0);
#pragma unroll
    for (int gi = 0; gi < kGroups; gi++) load_group(gi, m0);
  }
  __syncthreads();

  // ---- phase A: thread = (byte value, some of the rows); signed sums of 8 inputs ----
  {
    constexpr int kRowSets = kThreads / 256;      // threads per byte value
    constexpr int kRowsEach = TR / kRowSets;      // rows per thread
    const int bv = tid & 255, rp = tid >> 8;
    uint32_t sgn[8];
#pragma unroll
    for (int t = 0; t < 8; t++) sgn[t] = ((bv >> t) & 1) ? 0u : 0x80000000u;
#pragma unroll
    for (int rr = 0; rr < kRowsEach; rr++) {
      const int r = rp * kRowsEach + rr;
      float v[4];
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const float4 xa = *reinterpret_cast<const float4*>(xs + r * 32 + jj * 8);
        const float4 xb = *reinterpret_cast<const float4*>(xs + r * 32 + jj * 8 + 4);
        const float s0 = __uint_as_float(__float_as_uint(xa.x) ^ sgn[0]) +
                         __uint_as_float(__float_as_uint(xa.y) ^ sgn[1]);
        const float s1 = __uint_as_float(__float_as_uint(xa.z) ^ sgn[2]) +
                         __uint_as_float(__float_as_uint(xa.w) ^ sgn[3]);
        const float s2 = __uint_as_float(__float_as_uint(xb.x) ^ sgn[4]) +
                         __uint_as_float(__float_as_uint(xb.y) ^ sgn[5]);
        const float s3 = __uint_as_float(__float_as_uint(xb.z) ^ sgn[6]) +
                         __uint_as_float(__float_as_uint(xb.w) ^ sgn[7]);
        v[jj] = (s0 + s1) + (s2 + s3);
      }
      *reinterpret_cast<float4*>(compact + (r * 256 + bv) * 4) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
  __syncthreads();
  // ---- phase B: replicate each (row, byte) entry 8 times into its table line ----
  // line (row pair p, byte b) at lut + p*65536 + b*256; inside: [row parity][c][j] floats
  {
    const int c = lane & 7, bl = lane >> 3;
#pragma unroll 4
    for (int it = 0; it < TR * 256 / (kWarps * 4); it++) {
      const int e = (it * kWarps + warp) * 4 + bl;  // row*256 + byte
      const int r = e >> 8, b = e & 255;
      const float4 v = *reinterpret_cast<const float4*>(compact + e * 4);
      *reinterpret_cast<float4*>(lut + (r >> 1) * 65536 + b * 256 + (r & 1) * 128 + c * 16) = v;
    }
  }
  __syncthreads();

  // ---- lookup phase ----
  // lookup of byte value b in row r: [byteperm(word, lane*4, sel) + kLutImm + (r>>1)*65536 + (r&1)*128]
  const uint32_t hi = (uint32_t)(lane * 4);
  const uint32_t sel = 0x7604u | ((uint32_t)j << 4);

  // bias uses the all-ones entry (byte 255): sum of this lane's 8 inputs per row
  float ones[kGroups];
#pragma unroll
  for (int gi = 0; gi < kGroups; gi++) {
    float o = 0.f;
#pragma unroll
    for (int r = gi * RPG; r < (gi + 1) * RPG; r++)
      o += *reinterpret_cast<const float*>(lut + (r >> 1) * 65536 + 255 * 256 + (r & 1) * 128 +
                                           lane * 4);
    ones[gi] = o;
  }

  for (int s = 0; s < nsteps; s++) {
    const int m = m0 + s * (kWarps * 32);
    const bool active = m < m_end;
    const int m_next = m + kWarps * 32;
    const bool next = (s + 1 < nsteps) && m_next < m_end;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (active) {
#pragma unroll
      for (int gi = 0; gi < kGroups; gi++) {
        float t[NB][4];
#pragma unroll
        for (int rr = 0; rr < RPG; rr++) {
          const int r = gi * RPG + rr;
#pragma unroll
          for (int b = 0; b < NB; b++) {
            const uint32_t w4[4] = {wv[r][b].x, wv[r][b].y, wv[r][b].z, wv[r][b].w};
#pragma unroll
            for (int c = 0; c < 4; c++) {
              const uint32_t a = __byte_perm(w4[c], hi, sel);
              float v;
              if (r == 0) v = lds_f32_imm<kLutImm>(a);
              else if (r == 1) v = lds_f32_imm<kLutImm + 128>(a);
              else if (r == 2) v = lds_f32_imm<kLutImm + 65536>(a);
              else v = lds_f32_imm<kLutImm + 65536 + 128>(a);
              t[b][c] = (rr == 0) ? v : t[b][c] + v;
            }
          }
          if (next) load_row(r, m_next);  // the registers of this row are free again
        }
        if (gi * RPG < nrows) {  // rows past the end of K have no alpha
#pragma unroll
          for (int b = 0; b < NB; b++) {
            const float2 a01 = __half22float2(u32_as_half2(av[gi][b].x));
            const float2 a23 = __half22float2(u32_as_half2(av[gi][b].y));
            acc[0] = fmaf(a01.x, t[b][0], acc[0]);
            acc[1] = fmaf(a01.y, t[b][1], acc[1]);
            acc[2] = fmaf(a23.x, t[b][2], acc[2]);
            acc[3] = fmaf(a23.y, t[b][3], acc[3]);
          }
          if (q_bias != nullptr) {
            const float2 b01 = __half22float2(u32_as_half2(av[gi][NB].x));
            const float2 b23 = __half22float2(u32_as_half2(av[gi][NB].y));
            acc[0] = fmaf(b01.x, ones[gi], acc[0]);
            acc[1] = fmaf(b01.y, ones[gi], acc[1]);
            acc[2] = fmaf(b23.x, ones[gi], acc[2]);
            acc[3] = fmaf(b23.y, ones[gi], acc[3]);
          }
        }
        if (next) load_group(gi, m_next);
      }
    }
    // combine the four byte lanes of each column quad
#pragma unroll
    for (int c = 0; c < 4; c++) {
      acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
      acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
    }
    // every lane of the quad now holds the four column sums: lane j == 0 adds
    // them to the scratch row with one 16-byte reduction
    if (active && j == 0 && HQ_IN_BOUNDS(ws + m, 16, ws, (size_t)M * 4, 204))
      red_add_v4_f32(ws + m, acc[0], acc[1], acc[2], acc[3]);
  }

  // ---- the last CTA of a column range converts it to fp16 and re-zeroes the scratch ----
  if (!finalize) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned total = per_range ? gridDim.y : gridDim.x * gridDim.y;
    const unsigned prev = atomicAdd(counters + (per_range ? blockIdx.x : 0), 1u);
    *s_last = (prev == total - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (*s_last) {
    __threadfence();
    const int lo = per_range ? m_begin : 0, hi_m = per_range ? m_end : M;
    for (int mm = lo + tid * 4; mm < hi_m; mm += kThreads * 4) {
      if (!HQ_IN_BOUNDS(out + mm, 8, out, (size_t)M * 2, 205)) continue;
      const float4 v = __ldcg(reinterpret_cast<const float4*>(ws + mm));
      const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
      *reinterpret_cast<uint2*>(out + mm) = make_uint2(half2_as_u32(h01), half2_as_u32(h23));
      *reinterpret_cast<float4*>(ws + mm) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (tid == 0) counters[per_range ? blockIdx.x : 0] = 0u;
  }
}

// ---- bulk-copy form ---------------------------------------------------------
// The register form above keeps one column step of packed words in flight per
// warp, about 29 KB per SM, and waits out the HBM latency at every step.  This
// form asks the copy engine for the CTA's WHOLE column range right at the
// start: a CTA owns a 64-input K tile (two packed rows, 64 KB of tables) and up
// to kMaxStages steps of 512 columns.  Each of the 2*NB packed-word runs, NB
// alpha runs and the bias run of that range is contiguous in global memory and
// is fetched by TWO large bulk copies (cp.async.bulk, global -> shared), one
// per half of the range, each half completing on its own mbarrier - few large
// copies is what the copy engine is good at.  All copies are in flight while
// the tables are built, HBM streams without gaps, the first half is looked up
// while the second one lands, and the lookup phase reads its operands with
// quad-broadcast shared-memory loads (one wavefront per load).  Needs M % 8 == 0, alpha groups
// of a multiple of 64 inputs and 16-byte aligned alpha / bias (the alpha runs
// are copied in 16-byte units); other shapes take the register form.
constexpr int kBulkThreads = 512;
constexpr int kBulkWarps = kBulkThreads / 32;
constexpr int kBulkCols = kBulkWarps * 32;  // columns per step
constexpr int kMaxStages = 8;
constexpr uint32_t kMbarSpins = 1u << 22;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kMbarSpins; i++) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds_u2(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// Shared memory: [flag 16 B][mbarriers 8 x 8 B][build scratch][padding][tables 64 KiB at
// kLutImm][2*NB word runs of the column range][NB alpha runs][bias run]
struct BulkLayout {
  static constexpr int kCompactWords = 2 * 256 * 4;
  static constexpr int kBuildBytes = kCompactWords * 4 + 2 * 32 * 4;
  static constexpr int kHeadBytes = 16 + kMaxStages * 8;
  static constexpr int kLutBytes = 65536;
  static constexpr int kLutImm = (kDynBase + kSlack + kHeadBytes + kBuildBytes + 255) / 256 * 256;
  static constexpr int kStage0 = kLutImm + kLutBytes;  // shared-window address of stage 0
};
template <int NB>
struct BulkStage {
  static constexpr int kBytes = 2 * NB * kBulkCols * 4 + (NB + 1) * kBulkCols * 2;
};

template <int NB>
__global__ void __launch_bounds__(kBulkThreads, 1)
lutgemm_bulk_kernel(const uint32_t* __restrict__ bW, const __half* __restrict__ alpha,
                    const __half* __restrict__ q_bias, const __half* __restrict__ x,
                    __half* __restrict__ out, float* __restrict__ ws,
                    unsigned* __restrict__ counters, int M, int K, int rows_per_group,
                    int cols_per_cta, int nb_total, int b0, int finalize, int per_range) {
  using L = BulkLayout;
  constexpr int kLutImm = L::kLutImm;
  extern __shared__ __align__(16) unsigned char dsm[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t dsm_addr = (uint32_t)__cvta_generic_to_shared(dsm);
  // the host has checked where the dynamic region starts; never taken
  if (dsm_addr < (uint32_t)kDynBase || dsm_addr > (uint32_t)(kDynBase + kSlack)) return;
  unsigned char* base0 = dsm - dsm_addr;  // generic address of shared-window address 0
  unsigned char* lut = base0 + kLutImm;
  unsigned* s_last = reinterpret_cast<unsigned*>(dsm);
  const uint32_t bars = dsm_addr + 16;
  float* compact = reinterpret_cast<float*>(dsm + L::kHeadBytes);
  float* xs = compact + L::kCompactWords;
  const int row0 = blockIdx.y * 2;  // first packed row of the tile
  const int total_rows = K >> 5;
  const int nrows = min(2, total_rows - row0);
  const int m_begin = blockIdx.x * cols_per_cta;
  const int m_end = min(M, m_begin + cols_per_cta);
  const int nsteps = (m_end - m_begin + kBulkCols - 1) / kBulkCols;
  const int g = row0 / rows_per_group;  // the tile's alpha group

  if (tid < 64) {
    const int k = row0 * 32 + tid;
    xs[tid] = (k < K) ? __half2float(x[k]) : 0.f;
  }
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; s++) mbar_init(bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // ---- request the whole column range: warp h asks for half h of every run ----
  const int steps_half = (nsteps + 1) / 2;            // steps in the first half
  const uint32_t range_cols = (uint32_t)cols_per_cta;  // run pitch in shared memory (columns)
  const uint32_t alpha_off = 2u * NB * range_cols * 4u;
  if (warp < 2 && warp * steps_half < nsteps) {
    const int h = warp;
    const int m = m_begin + h * steps_half * kBulkCols;
    const int m_hi = h == 0 ? min(m_end, m_begin + steps_half * kBulkCols) : m_end;
    const uint32_t cols = (uint32_t)(m_hi - m);  // multiple of 8
    const uint32_t stage = (uint32_t)L::kStage0;
    const uint32_t col0 = (uint32_t)(m - m_begin);
    const uint32_t bar = bars + 8 * h;
    const bool bias_on = q_bias != nullptr;
    // this lane's copy: packed words of (row r, plane b), alpha of plane b, or the bias
    const void* src = nullptr;
    uint32_t dst = 0, bytes = 0;
    if (lane < 2 * NB) {
      const int r = lane / NB, b = lane - r * NB;
      if (r < nrows) {
        src = bW + ((size_t)(row0 + r) * nb_total + b0 + b) * M + m;
        dst = stage + ((uint32_t)lane * range_cols + col0) * 4u;
        bytes = cols * 4u;
      }
    } else if (lane < 3 * NB) {
      const int b = lane - 2 * NB;
      src = alpha + ((size_t)g * nb_total + b0 + b) * M + m;
      dst = stage + alpha_off + ((uint32_t)b * range_cols + col0) * 2u;
      bytes = cols * 2u;
    } else if (lane == 3 * NB && bias_on) {
      src = q_bias + (size_t)g * M + m;
      dst = stage + alpha_off + ((uint32_t)NB * range_cols + col0) * 2u;
      bytes = cols * 2u;
    }
#ifdef HQ_BOUNDS_CHECK
    {
      // a copy that leaves its buffer is recorded and the whole stage is skipped
      const size_t groups = (size_t)(total_rows / rows_per_group);
      bool fine = true;
      if (bytes != 0) {
        if (lane < 2 * NB) fine = HQ_IN_BOUNDS(src, bytes, bW, (size_t)total_rows * nb_total * M * 4, 211);
        else if (lane < 3 * NB) fine = HQ_IN_BOUNDS(src, bytes, alpha, groups * nb_total * M * 2, 212);
        else fine = HQ_IN_BOUNDS(src, bytes, q_bias, groups * M * 2, 213);
      }
      if (__ballot_sync(0xffffffffu, !fine) != 0u) bytes = 0;
    }
#endif
    uint32_t total = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) mbar_expect_tx(bar, total);
    __syncwarp();
    if (bytes != 0) bulk_load(dst, src, bytes, bar);
  }

  // ---- phase A: thread = (byte value, row); signed sums of 8 inputs ----
  {
    const int bv = tid & 255, r = tid >> 8;
    uint32_t sgn[8];
#pragma unroll
    for (int t = 0; t < 8; t++) sgn[t] = ((bv >> t) & 1) ? 0u : 0x80000000u;
    float v[4];
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
      const float4 xa = *reinterpret_cast<const float4*>(xs + r * 32 + jj * 8);
      const float4 xb = *reinterpret_cast<const float4*>(xs + r * 32 + jj * 8 + 4);
      const float s0 = __uint_as_float(__float_as_uint(xa.x) ^ sgn[0]) +
                       __uint_as_float(__float_as_uint(xa.y) ^ sgn[1]);
      const float s1 = __uint_as_float(__float_as_uint(xa.z) ^ sgn[2]) +
                       __uint_as_float(__float_as_uint(xa.w) ^ sgn[3]);
      const float s2 = __uint_as_float(__float_as_uint(xb.x) ^ sgn[4]) +
                       __uint_as_float(__float_as_uint(xb.y) ^ sgn[5]);
      const float s3 = __uint_as_float(__float_as_uint(xb.z) ^ sgn[6]) +
                       __uint_as_float(__float_as_uint(xb.w) ^ sgn[7]);
      v[jj] = (s0 + s1) + (s2 + s3);
    }
    *reinterpret_cast<float4*>(compact + (r * 256 + bv) * 4) = make_float4(v[0], v[1], v[2], v[3]);
  }
  __syncthreads();
  // ---- phase B: replicate each (row, byte) entry 8 times into its table line ----
  // line (byte b) at lut + b*256; inside: [row parity][c][j] floats
  {
    const int c = lane & 7, bl = lane >> 3;
#pragma unroll 4
    for (int it = 0; it < 2 * 256 / (kBulkWarps * 4); it++) {
      const int e = (it * kBulkWarps + warp) * 4 + bl;  // row*256 + byte
      const int r = e >> 8, b = e & 255;
      const float4 v = *reinterpret_cast<const float4*>(compact + e * 4);
      *reinterpret_cast<float4*>(lut + b * 256 + (r & 1) * 128 + c * 16) = v;
    }
  }
  __syncthreads();

  // ---- lookup phase ----
  const int j = lane & 3;   // byte of the word this lane looks up
  const int cq = lane >> 2; // column quad inside the warp's 32 columns
  const uint32_t hi = (uint32_t)(lane * 4);
  const uint32_t sel = 0x7604u | ((uint32_t)j << 4);
  // bias uses the all-ones entry (byte 255): sum of this lane's 8 inputs per row
  const float ones = *reinterpret_cast<const float*>(lut + 255 * 256 + lane * 4) +
                     *reinterpret_cast<const float*>(lut + 255 * 256 + 128 + lane * 4);
  const uint32_t col_off = (uint32_t)(warp * 32 + cq * 4);  // column inside the step
  bool ok = true;
  for (int s = 0; s < nsteps; s++) {
    const int m = m_begin + s * kBulkCols + (int)col_off;
    if (ok && !mbar_wait(bars + 8 * (s >= steps_half ? 1 : 0), 0)) ok = false;
    const bool active = m < m_end;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (active) {
      const uint32_t stage = (uint32_t)L::kStage0;
      const uint32_t col = (uint32_t)(s * kBulkCols) + col_off;  // column inside the range
      float t[NB][4];
#pragma unroll
      for (int r = 0; r < 2; r++) {
#pragma unroll
        for (int b = 0; b < NB; b++) {
          // rows past the end of K were not copied: their tables are zero, any word will do
          const uint4 wv = lds_u4(stage + ((uint32_t)(r * NB + b) * range_cols + col) * 4u);
          const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int c = 0; c < 4; c++) {
            const uint32_t a = __byte_perm(w4[c], hi, sel);
            const float v = r == 0 ? lds_f32_imm<kLutImm>(a) : lds_f32_imm<kLutImm + 128>(a);
            t[b][c] = (r == 0) ? v : t[b][c] + v;
          }
        }
      }
#pragma unroll
      for (int b = 0; b < NB; b++) {
        const uint2 av = lds_u2(stage + alpha_off + ((uint32_t)b * range_cols + col) * 2u);
        const float2 a01 = __half22float2(u32_as_half2(av.x));
        const float2 a23 = __half22float2(u32_as_half2(av.y));
        acc[0] = fmaf(a01.x, t[b][0], acc[0]);
        acc[1] = fmaf(a01.y, t[b][1], acc[1]);
        acc[2] = fmaf(a23.x, t[b][2], acc[2]);
        acc[3] = fmaf(a23.y, t[b][3], acc[3]);
      }
      if (q_bias != nullptr) {
        const uint2 bv = lds_u2(stage + alpha_off + ((uint32_t)NB * range_cols + col) * 2u);
        const float2 b01 = __half22float2(u32_as_half2(bv.x));
        const float2 b23 = __half22float2(u32_as_half2(bv.y));
        acc[0] = fmaf(b01.x, ones, acc[0]);
        acc[1] = fmaf(b01.y, ones, acc[1]);
        acc[2] = fmaf(b23.x, ones, acc[2]);
        acc[3] = fmaf(b23.y, ones, acc[3]);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; c++) {
      acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
      acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
    }
    if (active && j == 0 && HQ_IN_BOUNDS(ws + m, 16, ws, (size_t)M * 4, 214))
      red_add_v4_f32(ws + m, acc[0], acc[1], acc[2], acc[3]);
  }
  // a wait that ran out: word kCounterWords - 1 of the counter block tells the host
  if (!ok && lane == 0) atomicExch(counters + (kCounterWords - 1), 1u);

  // ---- the last CTA of a column range converts it to fp16 and re-zeroes the scratch ----
  if (!finalize) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned total = per_range ? gridDim.y : gridDim.x * gridDim.y;
    const unsigned prev = atomicAdd(counters + (per_range ? blockIdx.x : 0), 1u);
    *s_last = (prev == total - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (*s_last) {
    __threadfence();
    const int lo = per_range ? m_begin : 0, hi_m = per_range ? m_end : M;
    for (int mm = lo + tid * 4; mm < hi_m; mm += kBulkThreads * 4) {
      if (!HQ_IN_BOUNDS(out + mm, 8, out, (size_t)M * 2, 215)) continue;
      const float4 v = __ldcg(reinterpret_cast<const float4*>(ws + mm));
      const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
      *reinterpret_cast<uint2*>(out + mm) = make_uint2(half2_as_u32(h01), half2_as_u32(h23));
      *reinterpret_cast<float4*>(ws + mm) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (tid == 0) counters[per_range ? blockIdx.x : 0] = 0u;
  }
}

struct LaunchArgs {
  dim3 grid;
  cudaStream_t st;
  const uint32_t* bW;
  const __half* alpha;
  const __half* q_bias;
  const __half* x;
  __half* out;
  float* ws;
  unsigned* counters;
  int M, K, rows_per_group, cols_per_cta, nb_total, per_range;
};

template <int TR, int NB, int RPG>
int launch_one(const LaunchArgs& a, int b0, const __half* bias, int finalize) {
  using L = Layout<TR>;
  constexpr int kThreads = TR == 4 ? 512 : 256;
  constexpr auto kern = lutgemm_kernel<TR, NB, RPG, kThreads>;
  cudaError_t e = ensure_dynamic_smem<kern>(L::kSmem);
  if (e != cudaSuccess) return cuda_status(e);
  kern<<<a.grid, kThreads, L::kSmem, a.st>>>(a.bW, a.alpha, bias, a.x, a.out, a.ws, a.counters,
                                             a.M, a.K, a.rows_per_group, a.cols_per_cta,
                                             a.nb_total, b0, finalize, a.per_range);
  return launch_status();
}

// Bit planes are handled up to kMax at a time (what the register budget of the
// one-step-ahead loads allows); further planes go to follow-up launches that
// accumulate into the same scratch row.  Only the first launch adds the bias
// term, only the last one converts the scratch row.
template <int TR, int RPG>
int launch_planes(const LaunchArgs& a) {
  constexpr int kMax = TR == 4 ? 3 : 4;
  const int nb = a.nb_total;
  for (int b0 = 0; b0 < nb; b0 += kMax) {
    const int n = nb - b0 < kMax ? nb - b0 : kMax;
    const int last = (b0 + n == nb) ? 1 : 0;
    const __half* bias = b0 == 0 ? a.q_bias : nullptr;
    int st;
    if (n == 1) st = launch_one<TR, 1, RPG>(a, b0, bias, last);
    else if (n == 2) st = launch_one<TR, 2, RPG>(a, b0, bias, last);
    else if (n == 3) st = launch_one<TR, 3, RPG>(a, b0, bias, last);
    else st = launch_one<TR, (kMax >= 4 ? 4 : 3), RPG>(a, b0, bias, last);
    if (st != HQ_OK) return st;
  }
  return HQ_OK;
}

template <int NB>
int launch_bulk_one(const LaunchArgs& a, int b0, const __half* bias, int finalize) {
  constexpr auto kern = lutgemm_bulk_kernel<NB>;
  const int stages = (a.cols_per_cta + kBulkCols - 1) / kBulkCols;
  const size_t smem = (size_t)BulkLayout::kStage0 - kDynBase + (size_t)stages * BulkStage<NB>::kBytes;
  cudaError_t e = ensure_dynamic_smem<kern>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  kern<<<a.grid, kBulkThreads, smem, a.st>>>(a.bW, a.alpha, bias, a.x, a.out, a.ws, a.counters, a.M,
                                             a.K, a.rows_per_group, a.cols_per_cta, a.nb_total, b0,
                                             finalize, a.per_range);
  return launch_status();
}

// stages of 512 columns that fit beside the tables for NB planes per launch
inline int bulk_max_stages(int nb) {
  const int stage = 2 * nb * kBulkCols * 4 + (nb + 1) * kBulkCols * 2;
  const int room = 227 * 1024 - (BulkLayout::kStage0 - kDynBase);
  return std::min(kMaxStages, room / stage);
}

// Planes in groups of up to 3 per launch (what leaves room for 8 stages)
int launch_bulk_planes(const LaunchArgs& a) {
  constexpr int kMax = 3;
  const int nb = a.nb_total;
  for (int b0 = 0; b0 < nb; b0 += kMax) {
    const int n = nb - b0 < kMax ? nb - b0 : kMax;
    const int last = (b0 + n == nb) ? 1 : 0;
    const __half* bias = b0 == 0 ? a.q_bias : nullptr;
    int st;
    if (n == 1) st = launch_bulk_one<1>(a, b0, bias, last);
    else if (n == 2) st = launch_bulk_one<2>(a, b0, bias, last);
    else st = launch_bulk_one<3>(a, b0, bias, last);
    if (st != HQ_OK) return st;
  }
  return HQ_OK;
}

// Argument rules shared by both entry points; nothing is launched or touched
// when they fail.
int check_args(const void* out_half, const void* x_half, const uint32_t* bW, const void* alpha_half,
               const void* q_bias_half, int M, int K, int nb, int group_size) {
  if (!out_half || !x_half || !bW || !alpha_half) return HQ_ERR_NULL_POINTER;
  if (M <= 0 || K <= 0 || M % 4 != 0 || K % 32 != 0 || nb < 1 || nb > 8) return HQ_ERR_BAD_SHAPE;
  if (group_size <= 0 || group_size % 32 != 0 || K % group_size != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(bW) || !aligned8(alpha_half) || (q_bias_half && !aligned8(q_bias_half)) ||
      !aligned8(out_half))
    return HQ_ERR_MISALIGNED;
  const int rpg = group_size / 32;
  // groups of 96, 160, ... inputs would straddle tiles
  if (rpg != 1 && rpg % 2 != 0) return HQ_ERR_UNSUPPORTED;
  return HQ_OK;
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
  const int cst = check_args(out_half, x_half, bW, alpha_half, q_bias_half, M, K, nb, group_size);
  if (cst != HQ_OK) return cst;
  if (!workspace || workspace_bytes < hq_lutgemm_workspace_bytes(M)) return HQ_ERR_WORKSPACE;
  if (!aligned16(workspace)) return HQ_ERR_MISALIGNED;
  const int rpg = group_size / 32;
  const int reserved = reserved_smem_per_block();
  if (reserved < kDynBase || reserved > kDynBase + kSlack) return HQ_ERR_UNSUPPORTED;

  // Bulk-copy form: 64-input tiles, the whole column range of a CTA requested up
  // front.  Opt-in (environment HQ_LUT_BULK=1): on B200 it measured 37.1 us
  // against 29.7 us for the register form on a 12288 x 12288, 3-plane layer.
  if (env_flag("HQ_LUT_BULK") && M % 8 == 0 && rpg % 2 == 0 && aligned16(alpha_half) &&
      (!q_bias_half || aligned16(q_bias_half))) {
    const int tiles2 = (K / 32 + 1) / 2;
    const int max_cols = bulk_max_stages(std::min(nb, 3)) * kBulkCols;
    // balanced column ranges of at most max_cols columns, multiples of 512
    const int steps_total = (M + kBulkCols - 1) / kBulkCols;
    const int ranges = (steps_total * kBulkCols + max_cols - 1) / max_cols;
    const int steps_per_range = (steps_total + ranges - 1) / ranges;
    LaunchArgs a;
    a.cols_per_cta = steps_per_range * kBulkCols;
    const int mblocks = (M + a.cols_per_cta - 1) / a.cols_per_cta;
    a.grid = dim3(mblocks, tiles2);
    a.st = (cudaStream_t)stream;
    a.bW = bW;
    a.alpha = reinterpret_cast<const __half*>(alpha_half);
    a.q_bias = reinterpret_cast<const __half*>(q_bias_half);
    a.x = reinterpret_cast<const __half*>(x_half);
    a.out = reinterpret_cast<__half*>(out_half);
    a.ws = reinterpret_cast<float*>(workspace);
    a.counters = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(workspace) +
                                             (hq_lutgemm_workspace_bytes(M) - 256));
    a.M = M;
    a.K = K;
    a.rows_per_group = rpg;
    a.nb_total = nb;
    a.per_range = mblocks <= kCounterWords - 1 ? 1 : 0;
    return launch_bulk_planes(a);
  }
  // K tile: 128 inputs wherever alpha groups do not straddle it; 64 inputs for
  // groups of 192, 320, ... inputs
  int tile_rows = (rpg % 4 == 0 || rpg <= 2) ? 4 : 2;
  const int tiles = (K / 32 + tile_rows - 1) / tile_rows;
  // columns per CTA: a multiple of 256 chosen so the grid is close to a
  // multiple of the resident CTA slots while the table build stays amortised.
  const int slots = sm_count() * (tile_rows == 2 ? 2 : 1);
  int best_cols = 256;
  double best_score = -1.0;
  const int max_chunks = (M + 255) / 256;
  for (int mb = 1; mb <= max_chunks; mb++) {
    const int chunk256 = (max_chunks + mb - 1) / mb;  // balanced ranges
    const long ctas = (long)((max_chunks + chunk256 - 1) / chunk256) * tiles;
    const long waves = (ctas + slots - 1) / slots;
    // efficiency = useful lookups / (lookups + table build), times wave balance
    const double amort = (double)(chunk256 * 256) / (chunk256 * 256 + 2000.0);
    const double balance = (double)ctas / (double)(waves * slots);
    const double score = amort * balance;
    if (score > best_score) { best_score = score; best_cols = chunk256 * 256; }
  }
  const int mblocks = (M + best_cols - 1) / best_cols;
  LaunchArgs a;
  a.grid = dim3(mblocks, tiles);
  a.st = (cudaStream_t)stream;
  a.bW = bW;
  a.alpha = reinterpret_cast<const __half*>(alpha_half);
  a.q_bias = reinterpret_cast<const __half*>(q_bias_half);
  a.x = reinterpret_cast<const __half*>(x_half);
  a.out = reinterpret_cast<__half*>(out_half);
  a.ws = reinterpret_cast<float*>(workspace);
  a.counters = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(workspace) +
                                           (hq_lutgemm_workspace_bytes(M) - 256));
  a.M = M;
  a.K = K;
  a.rows_per_group = rpg;
  a.cols_per_cta = best_cols;
  a.nb_total = nb;
  a.per_range = mblocks <= kCounterWords ? 1 : 0;
  if (tile_rows == 4) {
    if (rpg % 4 == 0) return launch_planes<4, 4>(a);
    if (rpg == 2) return launch_planes<4, 2>(a);
    return launch_planes<4, 1>(a);
  }
  if (rpg % 2 == 0) return launch_planes<2, 2>(a);
  return launch_planes<2, 1>(a);
}

// ---- entry point that allocates nothing ----------------------------------

}  // extern "C"

namespace hq {
namespace {

// Scratch row of the allocation-free entry point: fp32 partial sums for up to
// HQ_LUTGEMM_NOALLOC_MAX_M outputs plus the completion counter.  Every GPU
// that loads the library holds these 257 KiB until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[HQ_LUTGEMM_NOALLOC_MAX_M * 4 + 256];

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
  // every argument rule is checked before the shared array is looked up or touched
  const int cst = check_args(out_half, x_half, bW, alpha_half, q_bias_half, M, K, nb, group_size);
  if (cst != HQ_OK) return cst;
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
