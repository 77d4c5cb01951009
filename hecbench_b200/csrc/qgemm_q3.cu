// Batched dequant-GEMM for the GPTQ 3-bit layout on the sm_100a tensor cores:
//   Y[Mb][N] = X[Mb][K] * W[K][N],  W[k][n] = hfma(half(q[k][n]), scale[g][n], -zero[g][n])
// X, Y, scale, zero are fp16, q is the packed 3-bit stream of quant3MatMul
// (mat int32[K*3/32][N], 32 codes per 3 consecutive rows), g = k / group_size,
// accumulation is fp32 in tensor memory.  No counterpart in the reference tree:
// the dequant rule is the fp16 rule of quant3MatMul-cuda/kernels.h:121-122,137
// with per-(group, column) parameters.
//
// The contraction is computed transposed so that the weight dimension fills
// the 128 rows of a tcgen05.mma tile and the token batch is its N dimension:
//   D[128 n][Mb] += A[128 n][16 k] * B[16 k][Mb],  A = W^T (K-major), B = X^T (K-major)
// One CTA owns 128 output features and walks K in blocks of 64:
//   warps 0-3  producers: each thread owns one output feature, reads its six
//              packed words of the block (coalesced across the warp), turns
//              every 6-bit pair into half2(q0, q1) with one lookup in a
//              bank-replicated shared table, applies hfma2 with the group's
//              scale / -zero, and stores the 64 halves of its row into the
//              stage's A tile in the 128-byte-swizzled K-major layout the
//              tensor core reads; the same threads copy the X block into the
//              B tile; then fence.proxy.async + mbarrier arrive;
//   warp 4     one elected lane waits for the stage, issues four
//              tcgen05.mma.cta_group::1.kind::f16 (K = 16 each) with shared
//              memory descriptors, and commits them to the stage's "empty"
//              mbarrier; after the last block it commits to the accumulator
//              barrier;
//   warps 0-3  epilogue: tcgen05.ld of the warp's 32 TMEM lanes, fp32 -> fp16,
//              transposed store into Y.
// Every mbarrier wait is bounded: when the limit is hit the thread records a
// status code, stops waiting and carries on, so the kernel always terminates
// and frees its tensor memory; the host reads the status word.
#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kStages = 4;
constexpr int kBlockK = 64;                 // halves per smem row (128 bytes)
constexpr int kTileN = 128;                 // output features per CTA (UMMA M)
constexpr int kMaxTokens = 128;             // UMMA N upper bound handled here
constexpr int kATile = kTileN * 128;        // bytes
constexpr int kBTile = kMaxTokens * 128;    // bytes
constexpr int kDeqLut = 64 * 128;           // 64 pair values x 32 lane copies x 4 B
constexpr int kProducerThreads = 128;
constexpr int kThreads = 160;
constexpr uint32_t kSpinLimit = 1u << 20;   // bounded mbarrier polls
constexpr int kSmemBytes = 1024 + kStages * (kATile + kBTile) + kDeqLut + 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait; returns false when the limit was reached.  A thread that has
// already given up once (healthy == false) does not wait again.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, bool healthy) {
  if (!healthy) return false;
  for (uint32_t i = 0; i < kSpinLimit; i++) {
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
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// 64-bit shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128
// bytes, 8-row groups 1024 bytes apart (stride byte offset 64 in 16-byte units),
// leading byte offset 1, descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fffu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)64 << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

struct QgemmParams {
  const __half* X;
  const int32_t* mat;
  const __half* scales;
  const __half* zeros;
  __half* Y;
  int* status;
  int Mb, N, K, group_size, tokens_padded;
};

__global__ void __launch_bounds__(kThreads, 1) qgemm_q3_kernel(const QgemmParams p) {
  extern __shared__ unsigned char dsm_raw[];
  // 1024-byte aligned tiles (the swizzle pattern repeats every 1024 bytes)
  const uint32_t raw = smem_u32(dsm_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = dsm_raw + (base - raw);
  const uint32_t a_tiles = base;
  const uint32_t b_tiles = base + kStages * kATile;
  unsigned char* deq_lut = sm + kStages * (kATile + kBTile);
  const uint32_t bars = base + kStages * (kATile + kBTile) + kDeqLut;
  // barrier slots (8 bytes each): full[kStages], empty[kStages], accum; then the TMEM address
  const uint32_t full0 = bars, empty0 = bars + 8 * kStages, accum_bar = bars + 16 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kStages * (kATile + kBTile) + kDeqLut +
                                                    16 * kStages + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN;
  const int nkb = p.K / kBlockK;
  bool ok = true;

  if (tid == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(full0 + 8 * s, kProducerThreads);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // pair table: entry v (6 bits) = half2(v & 7, v >> 3), one copy per bank
  for (int i = tid; i < 64 * 32; i += kThreads) {
    const int v = i >> 5;
    reinterpret_cast<uint32_t*>(deq_lut)[i] =
        half2_as_u32(__halves2half2(__int2half_rn(v & 7), __int2half_rn(v >> 3)));
  }
  if (warp == 4) {
    // 128 columns of tensor memory: accumulator D[128 lanes][tokens <= 128] fp32
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(128)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;

  if (warp < 4) {
    // ------------------------------ producers ------------------------------
    const int t = tid;              // output feature n0 + t, A-tile row t
    const int n = n0 + t;
    const unsigned char* lut_lane = deq_lut + lane * 4;
    const uint32_t a_row = (uint32_t)((t >> 3) * 1024 + (t & 7) * 128);
    const int swz = t & 7;
    __half2 sc2 = __float2half2_rn(0.f), nz2 = sc2;
    int cur_group = -1;
    for (int kb = 0; kb < nkb; kb++) {
      const int s = kb % kStages;
      const uint32_t round = (uint32_t)(kb / kStages);
      // packed words of this block: rows 6*kb .. 6*kb+5 (two groups of 32 inputs)
      uint32_t w[6];
#pragma unroll
      for (int i = 0; i < 6; i++) w[i] = ldg_stream_u32(p.mat + (size_t)(6 * kb + i) * p.N + n);
      const int g = (kb * kBlockK) / p.group_size;
      if (g != cur_group) {
        cur_group = g;
        const __half sc = p.scales[(size_t)g * p.N + n];
        const __half z = p.zeros[(size_t)g * p.N + n];
        sc2 = __half2half2(sc);
        nz2 = __half2half2(__hneg(z));
      }
      if (!mbar_wait(empty0 + 8 * s, (round & 1u) ^ 1u, ok)) ok = false;

      // ---- A tile: 64 weights of row t, 8 chunks of 16 bytes ----
      const uint32_t a_stage = a_tiles + s * kATile + a_row;
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const uint32_t w0 = w[3 * half], w1 = w[3 * half + 1], w2 = w[3 * half + 2];
        // sixteen 6-bit pair values of the 96-bit stream
        uint32_t pv[16];
#pragma unroll
        for (int i = 0; i < 5; i++) pv[i] = (w0 >> (6 * i)) & 63u;
        pv[5] = __funnelshift_r(w0, w1, 30) & 63u;
#pragma unroll
        for (int i = 0; i < 4; i++) pv[6 + i] = (w1 >> (4 + 6 * i)) & 63u;
        pv[10] = __funnelshift_r(w1, w2, 28) & 63u;
#pragma unroll
        for (int i = 0; i < 5; i++) pv[11 + i] = (w2 >> (2 + 6 * i)) & 63u;
#pragma unroll
        for (int c = 0; c < 4; c++) {
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const uint32_t q2 = *reinterpret_cast<const uint32_t*>(lut_lane + (pv[4 * c + e] << 7));
            o[e] = half2_as_u32(__hfma2(u32_as_half2(q2), sc2, nz2));
          }
          const int chunk = half * 4 + c;  // 16-byte chunk (8 halves) of the 128-byte row
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                           a_stage + (uint32_t)((chunk ^ swz) * 16)),
                       "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                       : "memory");
        }
      }
      // ---- B tile: X[token][kb*64 .. +63], tokens_padded rows of 8 chunks ----
      const uint32_t b_stage = b_tiles + s * kBTile;
      for (int idx = t; idx < p.tokens_padded * 8; idx += kProducerThreads) {
        const int row = idx >> 3, c = idx & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < p.Mb)
          v = __ldg(reinterpret_cast<const uint4*>(p.X + (size_t)row * p.K + kb * kBlockK) + c);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                         b_stage + (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 +
                                              ((c ^ (row & 7)) * 16))),
                     "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                     : "memory");
      }
      fence_async_smem();
      mbar_arrive(full0 + 8 * s);
    }
  } else if (lane == 0) {
    // ------------------------------ MMA issuer ------------------------------
    // instruction descriptor: D fp32, A/B fp16, both K-major, N = tokens_padded, M = 128
    const uint32_t idesc = (1u << 4) | ((uint32_t)(p.tokens_padded >> 3) << 17) |
                           ((uint32_t)(kTileN >> 4) << 24);
    for (int kb = 0; kb < nkb; kb++) {
      const int s = kb % kStages;
      const uint32_t round = (uint32_t)(kb / kStages);
      if (!mbar_wait(full0 + 8 * s, round & 1u, ok)) ok = false;
      tc_fence_after();
      const uint64_t adesc = smem_desc(a_tiles + s * kATile);
      const uint64_t bdesc = smem_desc(b_tiles + s * kBTile);
#pragma unroll
      for (int i = 0; i < kBlockK / 16; i++)
        umma_f16(tmem_d, adesc + 2 * i, bdesc + 2 * i, idesc, (kb | i) != 0 ? 1u : 0u);
      umma_commit(empty0 + 8 * s);
    }
    umma_commit(accum_bar);
  }

  if (warp < 4) {
    // ------------------------------ epilogue ------------------------------
    if (!mbar_wait(accum_bar, 0, ok)) ok = false;
    tc_fence_after();
    const int n = n0 + tid;  // TMEM lane = D row = output feature
    const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16);
    for (int j0 = 0; j0 < p.tokens_padded; j0 += 16) {
      uint32_t r[16];
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
          "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
            "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
            "=r"(r[14]), "=r"(r[15])
          : "r"(taddr + (uint32_t)j0));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 16; j++)
        if (j0 + j < p.Mb) p.Y[(size_t)(j0 + j) * p.N + n] = __float2half_rn(__uint_as_float(r[j]));
    }
  }
  if (!ok && p.status != nullptr) atomicExch(p.status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(128)
                 : "memory");
  }
}

}  // namespace
}  // namespace hq

extern "C" int hq_qgemm_q3_f16(const void* X_half, const int32_t* mat, const void* scales_half,
                               const void* zeros_half, void* Y_half, int Mb, int N, int K,
                               int group_size, int* status_word, hq_stream_t stream) {
  using namespace hq;
  if (!X_half || !mat || !scales_half || !zeros_half || !Y_half) return HQ_ERR_NULL_POINTER;
  if (Mb <= 0 || Mb > kMaxTokens || N <= 0 || K <= 0 || N % kTileN != 0 || K % kBlockK != 0)
    return HQ_ERR_BAD_SHAPE;
  if (group_size <= 0 || group_size % kBlockK != 0 || K % group_size != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(X_half) || !aligned4(mat) || (K % 8) != 0) return HQ_ERR_MISALIGNED;
  cudaError_t e = cudaFuncSetAttribute(qgemm_q3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemBytes);
  if (e != cudaSuccess) return cuda_status(e);
  QgemmParams prm;
  prm.X = reinterpret_cast<const __half*>(X_half);
  prm.mat = mat;
  prm.scales = reinterpret_cast<const __half*>(scales_half);
  prm.zeros = reinterpret_cast<const __half*>(zeros_half);
  prm.Y = reinterpret_cast<__half*>(Y_half);
  prm.status = status_word;
  prm.Mb = Mb;
  prm.N = N;
  prm.K = K;
  prm.group_size = group_size;
  prm.tokens_padded = (Mb + 15) / 16 * 16;
  qgemm_q3_kernel<<<N / kTileN, kThreads, kSmemBytes, (cudaStream_t)stream>>>(prm);
  return launch_status();
}
