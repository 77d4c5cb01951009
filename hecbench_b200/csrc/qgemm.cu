// Batched dequant-GEMM on the sm_100a tensor cores, Y[Mb][N] = X[Mb][K] * W[K][N]
// with fp16 X and Y and fp32 accumulation in tensor memory, for two packed
// weight formats (no counterpart in the reference tree):
//  * GPTQ 3-bit: W[k][n] = hfma(half(q[k][n]), scale[g][n], -zero[g][n]), q the
//    packed 3-bit stream of quant3MatMul (mat int32[K*3/32][N], 32 codes per 3
//    consecutive rows), g = k / group_size, fp16 scale / zero per (group,
//    column): the fp16 rule of quant3MatMul-cuda/kernels.h:121-122,137;
//  * NF4: W[k][n] = half(lut16[code[n*K + k]] * absmax[(n*K + k) / blocksize]),
//    two 4-bit codes per byte in output-feature-major order B uint8[N][K/2]
//    (even element in the high nibble unless the low-nibble-first flag is
//    given): the dequantisation rule of hq_nf4_dequant_f16.
// The description below is written for the 3-bit format; the NF4 form differs
// only in the box the word warps fetch (128 rows x 32 bytes), in the unpack
// arithmetic (one float2 table lookup per byte = two codes, one multiply per
// code, packed to half2 with round-to-nearest) and in the ring depths.
//
// The contraction is computed transposed so that the weight dimension fills
// the 128 rows of a tcgen05.mma tile and the token batch is its N dimension:
//   D[128 n][Mb] += A[128 n][16 k] * B[16 k][Mb],  A = W^T, B = X^T (K-major)
// with A in TENSOR MEMORY (the unpack warps write it there with tcgen05.st, so
// the dequantised weights never pass through shared memory) and B = X in shared
// memory.  One CTA (448 threads) owns 128 output features and a range of K
// blocks of 64 inputs, and runs two independent pipelines j = 0, 1 over the
// blocks j, j + 2, ...:
//   warps 9, 10  packed-word TMA of pipeline 0 / 1: per block lane 0 waits for
//              the ring slot and posts the byte count, lanes 0-2 issue the
//              boxes (6 rows x 128 columns of words, 128 scales, 128 zeros)
//              into the pipeline's slots of an 8-deep shared-memory ring;
//   warps 12, 13 X TMA of pipeline 0 / 1 (one lane): one box of 64 inputs x all
//              tokens per block into the pipeline's four X stages, in the
//              128-byte-swizzled K-major layout (rows beyond the token count
//              are zero-filled by the TMA unit);
//   warps 0-3, 4-7  unpack group of pipeline 0 / 1: thread = one output feature
//              = one tensor-memory lane; it reads its six packed words from the
//              ring, turns every 6-bit pair into half2(q0, q1) with one lookup
//              in a bank-replicated shared table, applies hfma2 with the
//              group's scale / -zero, and writes its 64 halves as 32 columns of
//              its lane of the pipeline's A stage (tcgen05.st 32x32b.x32), then
//              tcgen05.wait::st, tcgen05.fence::before_thread_sync and one
//              mbarrier arrival per warp;
//   warps 8, 11  MMA issuer of pipeline 0 / 1 (one lane): waits for the block's
//              "full" barrier (four unpack-warp arrivals + the X bytes), issues
//              four tcgen05.mma.cta_group::1.kind::f16 (K = 16 each, A from
//              tensor memory, B through a shared-memory descriptor) into the
//              pipeline's OWN accumulator columns, and commits them to the
//              "empty" barriers of the A stage and of the X stage;
//   warps 0-7  epilogue: tcgen05.ld of both accumulators for the warp's 32
//              lanes, their sum, then either fp32 -> fp16 and a transposed
//              store into Y, or (K split over several CTAs) fp32 reductions
//              into a scratch matrix that the last CTA of the tile converts
//              and re-zeroes.
// Tensor memory per CTA (up to 64 tokens): 2 x 64 accumulator columns + 4 A
// stages x 32 columns = 256 of the SM's 512 columns, so two CTAs share an SM
// (the shared-memory request is padded to keep it at two); beyond 64 tokens a
// CTA takes all 512 columns.  No TMA load uses cluster multicast.
// Every mbarrier wait is bounded: when the limit is hit the thread records a
// status code, stops waiting and carries on, so the kernel always terminates
// and frees its tensor memory; the host reads the status word.
#include <cuda.h>

#include <cstdlib>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kStages = 4;                  // A tiles in tensor memory, two per pipeline
constexpr int kBlockK = 64;                 // halves per smem row (128 bytes)
constexpr int kTileN = 128;                 // output features per CTA (UMMA M)
constexpr int kMaxTokens = 128;             // UMMA N upper bound handled here
constexpr int kAColumns = kBlockK / 2;      // tensor-memory columns of one A stage (2 halves each)
enum { kFmtQ3 = 0, kFmtNf4 = 1 };
// bytes of one block's packed weights in the ring
//   3-bit: 6 rows x 128 words, then 128 scales and 128 zeros;  NF4: 128 rows x 32 bytes
// Per format: depth of the two shared-memory rings and size of the lookup table.
// 3-bit: 8 X stages (four per pipeline), 8 word slots, table [64 pair values][32
// lane copies] of half2.  NF4: 6 X stages, 6 word slots, table [256 byte
// values][16 copies] of float2 (the two levels of the byte's codes), 32 KiB: the
// shallower rings pay for it inside the same two-CTAs-per-SM budget.
template <int FMT>
struct Rings {
#ifndef HQ_RING_X_Q3  // ring depths (even: half per pipeline); overridable for sweeps
#define HQ_RING_X_Q3 8
#define HQ_RING_W_Q3 8
#define HQ_RING_X_NF4 6
#define HQ_RING_W_NF4 6
#endif
  static constexpr int kXStages = FMT == 0 ? HQ_RING_X_Q3 : HQ_RING_X_NF4;
  static constexpr int kWordAhead = FMT == 0 ? HQ_RING_W_Q3 : HQ_RING_W_NF4;
  static constexpr int kLutWords = FMT == 0 ? 64 * 32 : 256 * 16 * 2;
};
template <int FMT>
struct WordSlot { static constexpr int kBytes = FMT == kFmtQ3 ? 6 * 512 + 2 * 256 : 128 * 32; };
constexpr int kProducerThreads = 256;
constexpr int kThreads = 448;               // 8 unpack, MMA, 2 word TMA, MMA, 2 X TMA warps
constexpr uint32_t kSpinLimit = 1u << 20;   // bounded mbarrier polls

template <int FMT>
inline size_t qgemm_smem_bytes(int tokens_padded) {
  const size_t need =
      1024 + (size_t)Rings<FMT>::kXStages * (tokens_padded * 128) +
      Rings<FMT>::kWordAhead * WordSlot<FMT>::kBytes + 512;
  // The request also sets the number of CTAs per SM to what tensor memory holds:
  // two CTAs of 256 columns up to 64 tokens, one CTA of 512 columns beyond.
  const size_t static_bytes = (size_t)Rings<FMT>::kLutWords * 4;
  const size_t floor_bytes = (tokens_padded <= 64 ? 98 * 1024 : 128 * 1024) - static_bytes;
  return need > floor_bytes ? need : floor_bytes;
}

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
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// 2-D tiled TMA load (no multicast) completing on an mbarrier of this CTA
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
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

// tcgen05.mma, A operand in tensor memory (128 lanes x 8 columns of two halves per K = 16)
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0)
      : "memory");
}
// 32 consecutive columns of the executing warp's 32 lanes, one lane per thread
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
      "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}



struct QgemmParams {
  __half* Y;
  // Sharded layers: when peer_Y is non-null the tile is stored, as soon as it is
  // finished, into the output slice of EVERY GPU of the node (peer_Y[r] + y_offset,
  // peer-mapped memory, the local GPU included) instead of Y.
  __half* const* peer_Y;
  long long y_offset;
  int world;
  float* ws;            // fp32 [Mb][N] scratch + per-tile counters, used when ksplit > 1
  unsigned* counters;
  int* status;
#ifdef HQ_QGEMM_TRACE
  long long* trace;  // development: [CTA][4 roles][8] accumulated clock cycles
#endif
  int Mb, N, K, group_size, tokens_padded, ksplit;
  // NF4 only (group_size is the absmax block size there)
  const float* absmax;
  const float* lut16;
  int low_first;
};

// output slice of this launch on GPU g (the table is constant during the launch)
__device__ __forceinline__ __half* peer_slice(const QgemmParams& p, int g) {
  return reinterpret_cast<__half*>(
             __ldg(reinterpret_cast<const unsigned long long*>(p.peer_Y) + g)) +
         p.y_offset;
}

// PEERS: the sharded form (tiles stored to every GPU's slice); a separate
// instantiation so that the plain form carries none of it.
template <int FMT, bool PEERS>
__global__ void __launch_bounds__(kThreads, 2)
qgemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_z,
                const QgemmParams p) {
  extern __shared__ unsigned char dsm_raw[];
  // 1024-byte aligned tiles (the swizzle pattern repeats every 1024 bytes)
  const uint32_t raw = smem_u32(dsm_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = dsm_raw + (base - raw);
  constexpr int kWordSlot = WordSlot<FMT>::kBytes;
  constexpr int kXStages = Rings<FMT>::kXStages, kWordAhead = Rings<FMT>::kWordAhead;
  constexpr int kWordRing = kWordAhead * kWordSlot;
  // lookup table.  3-bit: [pair value v (6 bits)][lane] = half2(v & 7, v >> 3), one
  // copy per bank.  NF4: [byte value][copy c < 16] = float2(level of the first
  // element, level of the second element): lane reads copy lane % 16, so the 16
  // lanes of a half-warp read 16 different bank pairs whatever their bytes are.
  __shared__ __align__(16) uint32_t lut_s[Rings<FMT>::kLutWords];
  const int kBTile = p.tokens_padded * 128;
  const uint32_t b_tiles = base;
  const uint32_t tiles_bytes = (uint32_t)(kXStages * kBTile);
  const uint32_t word_ring = base + tiles_bytes;  // [kWordAhead][6 rows][128 columns] words
  const uint32_t bars = base + tiles_bytes + kWordRing;
  // barrier slots (8 bytes each)
  // Pipeline j = unpack group j + MMA issuer j + two TMA warps handles blocks
  // j, j + 2, ...; its m-th block uses A stage j + 2 * (m & 1) (tensor memory)
  // and X stage j + 2 * (m & 3) (shared memory), so every barrier has one
  // producer side and one consumer side that take its phases strictly in order.
  // full[xs]:   both operands of the block are in place = one arrival per unpack
  //             warp of the group (4) + the X warp's expect_tx arrival + the X
  //             tile's bytes
  // empty[st]:  the issuer's instructions that read A stage st have completed
  // xempty[xs]: the issuer's instructions that read X stage xs have completed
  const uint32_t full0 = bars;
  const uint32_t empty0 = full0 + 8 * kXStages;
  const uint32_t xempty0 = empty0 + 8 * kStages;
  const uint32_t wfull0 = xempty0 + 8 * kXStages;       // word box landed (TMA bytes)
  const uint32_t wempty0 = wfull0 + 8 * kWordAhead;     // word box read by the group's 4 warps
  const uint32_t accum_bar = wempty0 + 8 * kWordAhead;  // both issuers committed their last block
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(
      sm + tiles_bytes + kWordRing + 8 * (2 * kXStages + kStages + 2 * kWordAhead + 1));
  __shared__ unsigned s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // tensor memory: two accumulators D[128 lanes][tokens] fp32 (one per MMA
  // issuer), then kStages A tiles of 128 lanes x 32 columns (64 halves per row)
  const uint32_t tmem_cols = p.tokens_padded <= 64 ? 256u : 512u;
  const uint32_t a_col0 = 2u * (uint32_t)p.tokens_padded;
  const int n0 = blockIdx.x * kTileN;
  // K blocks of this CTA: split index blockIdx.y of p.ksplit
  const int nkb_total = p.K / kBlockK;
  const int kb0 = (int)(((long long)nkb_total * blockIdx.y) / p.ksplit);
  const int kb1 = (int)(((long long)nkb_total * (blockIdx.y + 1)) / p.ksplit);
  const int nloc = kb1 - kb0;
  bool ok = true;
#ifdef HQ_QGEMM_TRACE
  long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long tmark = clock64();
#define HQ_TR(i) { const long long now_ = clock64(); tr[i] += now_ - tmark; tmark = now_; }
#else
#define HQ_TR(i)
#endif

  if (tid == 0) {
    for (int s = 0; s < kXStages; s++) {
      mbar_init(full0 + 8 * s, kProducerThreads / 64 + 1);
      mbar_init(xempty0 + 8 * s, 1);
    }
    for (int s = 0; s < kStages; s++) mbar_init(empty0 + 8 * s, 1);
    for (int s = 0; s < kWordAhead; s++) {
      mbar_init(wfull0 + 8 * s, 1);
      mbar_init(wempty0 + 8 * s, kProducerThreads / 64);
    }
    mbar_init(accum_bar, 2);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (FMT == kFmtQ3) {
    for (int i = tid; i < 64 * 32; i += kThreads) {
      const int v = i >> 5;
      lut_s[i] = half2_as_u32(__halves2half2(__int2half_rn(v & 7), __int2half_rn(v >> 3)));
    }
  } else {
    for (int i = tid; i < 256 * 16; i += kThreads) {
      const int b = i >> 4, hi = b >> 4, lo = b & 15;
      // even element = high nibble unless the low-nibble-first flag is given
      lut_s[2 * i] = __float_as_uint(p.lut16[p.low_first ? lo : hi]);
      lut_s[2 * i + 1] = __float_as_uint(p.lut16[p.low_first ? hi : lo]);
    }
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;

  if (warp < 8) {
    // ------------------------------ unpack warps ------------------------------
    // Two groups of four warps take alternate K blocks, so the groups (and the
    // two CTAs of the SM) sit in different phases of the loop and fill each
    // other's barrier and shared-memory latencies.  Thread = one output feature:
    // it unpacks the 64 weights of its row for the block.  The loop carries
    // running counters and phase bits (no division, no modulo).
    const int row = tid & 127;      // output feature n0 + row, A-tile row
    const int grp = tid >> 7;       // blocks grp, grp + 2, ...
    const unsigned char* lut = reinterpret_cast<const unsigned char*>(lut_s);
    const uint32_t lane8 = (uint32_t)(lane & 15) * 8u;  // NF4: this lane's copy of a table row
    const uint32_t lane4 = (uint32_t)lane * 4u;
    // this warp's 32 lanes of tensor memory (lane = A row), first A column
    const uint32_t a_lane = tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + a_col0;
    // word box: [6 rows][128 columns] words, then 128 scales, then 128 zeros
    const uint32_t my_words = word_ring + (uint32_t)(row * 4);
    const uint32_t my_param = word_ring + 6 * 512 + (uint32_t)(row * 2);

    // the group's m-th block uses stage grp + 2 * (m & 1) for the (m >> 1)-th time
    uint32_t a_stage = (uint32_t)grp, a_use = 0, x_stage = (uint32_t)grp;
    uint32_t w_slot = (uint32_t)grp, w_parity = 0;
    if constexpr (FMT == kFmtQ3) {
      HQ_TR(0)
      for (int i = grp; i < nloc; i += 2) {
        if (!mbar_wait(wfull0 + 8 * w_slot, w_parity, ok)) ok = false;
        HQ_TR(1)
        uint32_t w[6];
        uint16_t sc_bits, z_bits;
        {
          const uint32_t src = my_words + w_slot * kWordSlot;
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[0]) : "r"(src));
          asm volatile("ld.shared.u32 %0, [%1+512];" : "=r"(w[1]) : "r"(src));
          asm volatile("ld.shared.u32 %0, [%1+1024];" : "=r"(w[2]) : "r"(src));
          asm volatile("ld.shared.u32 %0, [%1+1536];" : "=r"(w[3]) : "r"(src));
          asm volatile("ld.shared.u32 %0, [%1+2048];" : "=r"(w[4]) : "r"(src));
          asm volatile("ld.shared.u32 %0, [%1+2560];" : "=r"(w[5]) : "r"(src));
          const uint32_t par = my_param + w_slot * kWordSlot;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sc_bits) : "r"(par));
          asm volatile("ld.shared.u16 %0, [%1+256];" : "=h"(z_bits) : "r"(par));
        }
        const __half2 sc2 = __half2half2(__ushort_as_half(sc_bits));
        const __half2 nz2 = __half2half2(__hneg(__ushort_as_half(z_bits)));
        uint32_t o[32];
  #pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          const uint32_t w0 = w[3 * hf], w1 = w[3 * hf + 1], w2 = w[3 * hf + 2];
          // sixteen 6-bit pair values of the 96-bit stream, as byte offsets (v << 7) | lane*4
          uint32_t po[16];
          po[0] = ((w0 << 7) & 0x1f80u) | lane4;
          po[1] = ((w0 << 1) & 0x1f80u) | lane4;
  #pragma unroll
          for (int q = 2; q < 5; q++) po[q] = ((w0 >> (6 * q - 7)) & 0x1f80u) | lane4;
          po[5] = (__funnelshift_r(w0, w1, 23) & 0x1f80u) | lane4;
          po[6] = ((w1 << 3) & 0x1f80u) | lane4;
  #pragma unroll
          for (int q = 1; q < 4; q++) po[6 + q] = ((w1 >> (6 * q - 3)) & 0x1f80u) | lane4;
          po[10] = (__funnelshift_r(w1, w2, 21) & 0x1f80u) | lane4;
          po[11] = ((w2 << 5) & 0x1f80u) | lane4;
  #pragma unroll
          for (int q = 1; q < 5; q++) po[11 + q] = ((w2 >> (6 * q - 5)) & 0x1f80u) | lane4;
  #pragma unroll
          for (int e = 0; e < 16; e++) {
            const uint32_t q2 = *reinterpret_cast<const uint32_t*>(lut + po[e]);
            o[16 * hf + e] = half2_as_u32(__hfma2(u32_as_half2(q2), sc2, nz2));
          }
        }
        // the ring slot is released only now: the lookups above consumed the words,
        // so the loads have certainly returned
        __syncwarp();
        if (lane == 0) mbar_arrive(wempty0 + 8 * w_slot);
        w_slot += 2;
        if (w_slot >= kWordAhead) { w_slot -= kWordAhead; w_parity ^= 1u; }
        HQ_TR(2)
        // the A tile of this stage must have been released by the tensor core
        if (a_use != 0 && !mbar_wait(empty0 + 8 * a_stage, (a_use - 1u) & 1u, ok)) ok = false;
        HQ_TR(3)
        tc_fence_after();  // orders the stores after the tensor core's reads of the stage
        tmem_store_32(a_lane + a_stage * (uint32_t)kAColumns, o);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * x_stage);
        HQ_TR(4)
        a_stage += 2;
        if (a_stage >= kStages) { a_stage -= kStages; a_use++; }
        x_stage += 2;
        if (x_stage >= kXStages) x_stage -= kXStages;
      }
    } else {
      // NF4: the thread's 64 codes of a block are 32 consecutive bytes of its row;
      // the block's absmax comes straight from global memory, one block ahead
      const uint32_t my_bytes = word_ring + (uint32_t)(row * 32);
      const float* am_row = p.absmax + ((size_t)(n0 + row) * p.K) / p.group_size;
      const int am_shift = 31 - __clz(p.group_size / kBlockK);  // blocks per absmax = 2^am_shift
      const bool am_pow2 = ((p.group_size / kBlockK) & (p.group_size / kBlockK - 1)) == 0;
      auto am_index = [&](int kb) {
        return am_pow2 ? (kb >> am_shift) : (kb * kBlockK) / p.group_size;
      };
      float am_next = grp < nloc ? __ldg(am_row + am_index(kb0 + grp)) : 0.f;
      for (int i = grp; i < nloc; i += 2) {
        const float am = am_next;
        if (i + 2 < nloc) am_next = __ldg(am_row + am_index(kb0 + i + 2));
        if (!mbar_wait(wfull0 + 8 * w_slot, w_parity, ok)) ok = false;
        uint32_t w[8];
        {
          const uint32_t src = my_bytes + w_slot * kWordSlot;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                       : "r"(src));
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+16];"
                       : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                       : "r"(src));
        }
        uint32_t o[32];
#pragma unroll
        for (int q = 0; q < 8; q++) {
#pragma unroll
          for (int t = 0; t < 4; t++) {
            // byte t of word q -> table row offset (byte << 7) | copy
            const uint32_t off =
                ((t == 0 ? (w[q] << 7) : (w[q] >> (8 * t - 7))) & 0x7f80u) | lane8;
            const float2 lv = *reinterpret_cast<const float2*>(lut + off);
            o[4 * q + t] = half2_as_u32(__floats2half2_rn(lv.x * am, lv.y * am));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(wempty0 + 8 * w_slot);
        w_slot += 2;
        if (w_slot >= kWordAhead) { w_slot -= kWordAhead; w_parity ^= 1u; }
        if (a_use != 0 && !mbar_wait(empty0 + 8 * a_stage, (a_use - 1u) & 1u, ok)) ok = false;
        tc_fence_after();  // orders the stores after the tensor core's reads of the stage
        tmem_store_32(a_lane + a_stage * (uint32_t)kAColumns, o);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * x_stage);
        a_stage += 2;
        if (a_stage >= kStages) { a_stage -= kStages; a_use++; }
        x_stage += 2;
        if (x_stage >= kXStages) x_stage -= kXStages;
      }
    }
  } else if ((warp == 8 || warp == 11) && lane == 0) {
    // ------------------------------ MMA issuers ------------------------------
    // Issuer j takes blocks j, j + 2, ... (the blocks of unpack group j) and
    // accumulates into its own tensor-memory columns, so that one issuer's
    // barrier polls overlap the other's instructions; the epilogue adds the two.
    // instruction descriptor: D fp32, A/B fp16, both K-major, N = tokens_padded, M = 128
    const uint32_t idesc = (1u << 4) | ((uint32_t)(p.tokens_padded >> 3) << 17) |
                           ((uint32_t)(kTileN >> 4) << 24);
    const int j = warp == 8 ? 0 : 1;
    const uint32_t acc = tmem_d + (uint32_t)(j * p.tokens_padded);
    uint32_t st = (uint32_t)j, xs = (uint32_t)j, xuse = 0;
    uint32_t accumulate = 0;
    HQ_TR(0)
    for (int i = j; i < nloc; i += 2) {
      if (!mbar_wait(full0 + 8 * xs, xuse & 1u, ok)) ok = false;
      HQ_TR(1)
      tc_fence_after();
      const uint32_t a_tmem = tmem_d + a_col0 + st * (uint32_t)kAColumns;
      const uint64_t bdesc = smem_desc(b_tiles + xs * kBTile);
#pragma unroll
      for (int k = 0; k < kBlockK / 16; k++) {
        umma_f16_ts(acc, a_tmem + 8 * k, bdesc + 2 * k, idesc, accumulate);
        accumulate = 1u;
      }
      umma_commit(empty0 + 8 * st);
      umma_commit(xempty0 + 8 * xs);
      HQ_TR(2)
      st += 2;
      if (st >= kStages) st -= kStages;
      xs += 2;
      if (xs >= kXStages) { xs -= kXStages; xuse++; }
    }
    umma_commit(accum_bar);
  } else if ((warp == 9 || warp == 10) && lane < 3) {
    // ------------------------------ packed-word TMA ------------------------------
    // One warp per pipeline j: lane 0 waits for the slot and posts the byte
    // count, then lanes 0-2 issue the loads side by side (3-bit: lane 0 the word
    // box, lanes 1 and 2 the scales and zeros; NF4: lane 0 alone).
    const int j = warp - 9;
    uint32_t slot = (uint32_t)j, use = 0;
    for (int i = j; i < nloc; i += 2) {
      if (lane == 0) {
        if (use != 0 && !mbar_wait(wempty0 + 8 * slot, (use - 1u) & 1u, ok)) ok = false;
        mbar_expect_tx(wfull0 + 8 * slot, kWordSlot);
      }
      __syncwarp(0x7u);
      const uint32_t dst = word_ring + slot * kWordSlot;
      if constexpr (FMT == kFmtQ3) {
        const int g = ((kb0 + i) * kBlockK) / p.group_size;
        if (lane == 0) tma_load_2d(dst, &map_w, n0, 6 * (kb0 + i), wfull0 + 8 * slot);
        else if (lane == 1) tma_load_2d(dst + 6 * 512, &map_s, n0, g, wfull0 + 8 * slot);
        else tma_load_2d(dst + 6 * 512 + 256, &map_z, n0, g, wfull0 + 8 * slot);
      } else {
        if (lane == 0) tma_load_2d(dst, &map_w, 32 * (kb0 + i), n0, wfull0 + 8 * slot);
      }
      slot += 2;
      if (slot >= kWordAhead) { slot -= kWordAhead; use++; }
    }
  } else if ((warp == 12 || warp == 13) && lane == 0) {
    // ------------------------------ X TMA ------------------------------
    const int j = warp - 12;
    uint32_t xs = (uint32_t)j, use = 0;
    for (int i = j; i < nloc; i += 2) {
      if (use != 0 && !mbar_wait(xempty0 + 8 * xs, (use - 1u) & 1u, ok)) ok = false;
      const uint32_t bar = full0 + 8 * xs;
      mbar_expect_tx(bar, (uint32_t)kBTile);
      tma_load_2d(b_tiles + xs * (uint32_t)kBTile, &map_x, (kb0 + i) * kBlockK, 0, bar);
      xs += 2;
      if (xs >= kXStages) { xs -= kXStages; use++; }
    }
  }

#ifdef HQ_QGEMM_TRACE
  if (p.trace != nullptr) {
    int role = -1;
    if (tid == 0) role = 0;            // unpack group 0
    else if (tid == 128) role = 1;     // unpack group 1
    else if (warp == 8 && lane == 0) role = 2;   // MMA issuer 0
    else if (warp == 11 && lane == 0) role = 3;  // MMA issuer 1
    if (role >= 0) {
      HQ_TR(5)
      for (int k = 0; k < 8; k++)
        p.trace[((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 4 + role) * 8 + k] = tr[k];
    }
  }
#endif
  if (warp < 8) {
    // ------------------------------ epilogue ------------------------------
    if (!mbar_wait(accum_bar, 0, ok)) ok = false;
    tc_fence_after();
    const int n = n0 + (warp & 3) * 32 + lane;  // TMEM lane = D row = output feature
    const uint32_t taddr = tmem_d + ((uint32_t)((warp & 3) * 32) << 16);
    // warps 0-3 take the even 16-token chunks, warps 4-7 the odd ones
    for (int j0 = (warp >> 2) * 16; j0 < p.tokens_padded; j0 += 32) {
      uint32_t r[16];
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
          "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
            "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
            "=r"(r[14]), "=r"(r[15])
          : "r"(taddr + (uint32_t)j0));
      if (nloc > 1) {
        // second issuer's partial sums (its columns are untouched when the CTA has one block)
        uint32_t q[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]),
              "=r"(q[7]), "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]),
              "=r"(q[14]), "=r"(q[15])
            : "r"(taddr + (uint32_t)(p.tokens_padded + j0)));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; j++)
          r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
      } else {
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      if (p.ksplit == 1 && !PEERS) {
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (j0 + j < p.Mb)
            p.Y[(size_t)(j0 + j) * p.N + n] = __float2half_rn(__uint_as_float(r[j]));
      } else if (p.ksplit == 1) {
        // sharded form: the tile is collected in shared memory as fp16 [token][128
        // features] (the X stages are free: every MMA has completed) and leaves in
        // whole 256-byte rows below
        __half* tile = reinterpret_cast<__half*>(sm);
#pragma unroll
        for (int j = 0; j < 16; j++)
          tile[(j0 + j) * kTileN + (warp & 3) * 32 + lane] = __float2half_rn(__uint_as_float(r[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (j0 + j < p.Mb)
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p.ws + (size_t)(j0 + j) * p.N + n),
                         "f"(__uint_as_float(r[j]))
                         : "memory");
      }
    }
  }
  if (PEERS && warp < 8 && p.ksplit == 1) {
    // 16 threads x 16 bytes = one token row of the tile; every row goes to the
    // output slice of every GPU of the node as one 256-byte run (over NVLink for
    // the peers)
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const __half* tile = reinterpret_cast<const __half*>(sm);
    const int e = tid, c8 = (e & 15) * 8;
    for (int g = 0; g < p.world; g++) {
      __half* Yg = peer_slice(p, g);
      const bool vec = (reinterpret_cast<uintptr_t>(Yg) & 15u) == 0;
      for (int t = e >> 4; t < p.Mb; t += 16) {
        const uint4 v = *reinterpret_cast<const uint4*>(tile + t * kTileN + c8);
        __half* dst = Yg + (size_t)t * p.N + n0 + c8;
        if (vec) {
          *reinterpret_cast<uint4*>(dst) = v;
        } else {
          const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
          for (int k = 0; k < 8; k++) dst[k] = h[k];
        }
      }
    }
  }
  if (!ok && p.status != nullptr) atomicExch(p.status, 1);
  tc_fence_before();
  if (p.ksplit > 1) __threadfence();
  __syncthreads();
  if (warp == 8) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                 "r"(tmem_cols)
                 : "memory");
  }
  if (p.ksplit > 1) {
    // the last CTA of this tile converts the scratch tile to fp16 and re-zeroes it
    if (tid == 0) {
      const unsigned prev = atomicAdd(p.counters + blockIdx.x, 1u);
      s_last = (prev == (unsigned)p.ksplit - 1u) ? 1u : 0u;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      // Mb x 32 groups of four features; five groups per thread and turn, all loads
      // of a turn issued before the first is used (one L2 round trip per turn
      // instead of one per element)
      constexpr int kTurn = 5;
      const int groups = p.Mb * (kTileN / 4);
      for (int g0 = tid; g0 < groups; g0 += kThreads * kTurn) {
        float4 v[kTurn];
#pragma unroll
        for (int u = 0; u < kTurn; u++) {
          const int gi = g0 + u * kThreads;
          if (gi < groups) {
            const int j = gi / (kTileN / 4), c = (gi - j * (kTileN / 4)) * 4;
            v[u] = __ldcg(reinterpret_cast<const float4*>(p.ws + (size_t)j * p.N + n0 + c));
          }
        }
#pragma unroll
        for (int u = 0; u < kTurn; u++) {
          const int gi = g0 + u * kThreads;
          if (gi < groups) {
            const int j = gi / (kTileN / 4), c = (gi - j * (kTileN / 4)) * 4;
            const size_t at = (size_t)j * p.N + n0 + c;
            const __half2 lo = __floats2half2_rn(v[u].x, v[u].y), hi = __floats2half2_rn(v[u].z, v[u].w);
            const uint2 packed = make_uint2(half2_as_u32(lo), half2_as_u32(hi));
            for (int g = 0; g < (PEERS ? p.world : 1); g++) {
              __half* Yg = PEERS ? peer_slice(p, g) : p.Y;
              if ((reinterpret_cast<uintptr_t>(Yg + at) & 7u) == 0) {
                *reinterpret_cast<uint2*>(Yg + at) = packed;
              } else {
                Yg[at] = __low2half(lo); Yg[at + 1] = __high2half(lo);
                Yg[at + 2] = __low2half(hi); Yg[at + 3] = __high2half(hi);
              }
            }
            *reinterpret_cast<float4*>(p.ws + at) = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      }
      if (tid == 0) p.counters[blockIdx.x] = 0u;
    }
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no libcuda link)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return (EncodeTiledFn) nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}


// X[Mb][K] fp16: box = 64 inputs x tokens_padded rows, 128-byte swizzle; rows
// beyond Mb are out of bounds and arrive as zeros
int encode_x_map(EncodeTiledFn encode, CUtensorMap* map_x, const void* X_half, int Mb, int K) {
  const int tokens_padded = (Mb + 15) / 16 * 16;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)Mb};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)tokens_padded};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(X_half), dims, strides,
             box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return HQ_ERR_UNSUPPORTED;
  return HQ_OK;
}

size_t qgemm_ws_bytes(int Mb, int N) {
  return ((size_t)Mb * N * 4 + 255) / 256 * 256 + ((size_t)(N / kTileN + 1) * 4 + 255) / 256 * 256;
}

// K split: only with a workspace, and only when the tiles alone cannot fill
// the CTA slots of the machine (two per SM)
QgemmParams make_params(void* Y_half, int Mb, int N, int K, int group_size, void* workspace,
                        size_t workspace_bytes, int* status_word) {
  QgemmParams prm;
  const int tiles = N / kTileN;
  const int slots = 2 * sm_count();
  int ksplit = 1;
  if (workspace != nullptr && workspace_bytes >= qgemm_ws_bytes(Mb, N) && aligned16(workspace)) {
    ksplit = slots / tiles;
    const int nkb = K / kBlockK;
    if (ksplit > nkb / 8) ksplit = nkb / 8;
    if (ksplit < 1) ksplit = 1;
  }
  prm.Y = reinterpret_cast<__half*>(Y_half);
  prm.peer_Y = nullptr;
  prm.y_offset = 0;
  prm.world = 1;
  prm.ws = reinterpret_cast<float*>(workspace);
  prm.counters = workspace ? reinterpret_cast<unsigned*>(reinterpret_cast<char*>(workspace) +
                                                         ((size_t)Mb * N * 4 + 255) / 256 * 256)
                           : nullptr;
  prm.status = status_word;
  prm.Mb = Mb;
  prm.N = N;
  prm.K = K;
  prm.group_size = group_size;
  prm.tokens_padded = (Mb + 15) / 16 * 16;
  prm.ksplit = ksplit;
  prm.absmax = nullptr;
  prm.lut16 = nullptr;
  prm.low_first = 0;
#ifdef HQ_QGEMM_TRACE
  {
    const char* tp = getenv("HQ_QGEMM_TRACE_PTR");
    prm.trace = tp ? reinterpret_cast<long long*>(strtoull(tp, nullptr, 0)) : nullptr;
  }
#endif
  return prm;
}

template <int FMT>
int launch_qgemm(const CUtensorMap& map_x, const CUtensorMap& map_w, const CUtensorMap& map_s,
                 const CUtensorMap& map_z, const QgemmParams& prm, hq_stream_t stream) {
  const size_t smem = qgemm_smem_bytes<FMT>(prm.tokens_padded);
  const dim3 grid(prm.N / kTileN, prm.ksplit);
  if (prm.peer_Y != nullptr) {
    constexpr auto kern = qgemm_kernel<FMT, true>;
    cudaError_t e = ensure_dynamic_smem<kern>(smem);
    if (e != cudaSuccess) return cuda_status(e);
    kern<<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_x, map_w, map_s, map_z, prm);
  } else {
    constexpr auto kern = qgemm_kernel<FMT, false>;
    cudaError_t e = ensure_dynamic_smem<kern>(smem);
    if (e != cudaSuccess) return cuda_status(e);
    kern<<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_x, map_w, map_s, map_z, prm);
  }
  return launch_status();
}
}  // namespace
}  // namespace hq

// Where a sharded launch stores its tiles (all null / 1 without sharding).
struct PeerOut {
  void* const* peer_Y = nullptr;
  long long y_offset = 0;
  int world = 1;
};

static int qgemm_q3_impl(const void* X_half, const int32_t* mat, const void* scales_half,
                         const void* zeros_half, void* Y_half, const PeerOut& po, int Mb, int N,
                         int K, int group_size, void* workspace, size_t workspace_bytes,
                         int* status_word, hq_stream_t stream) {
  using namespace hq;
  if (!X_half || !mat || !scales_half || !zeros_half || (!Y_half && !po.peer_Y))
    return HQ_ERR_NULL_POINTER;
  if (po.peer_Y && (po.world < 1 || po.world > 32 || po.y_offset < 0)) return HQ_ERR_BAD_SHAPE;
  if (Mb <= 0 || Mb > kMaxTokens || N <= 0 || K <= 0 || N % kTileN != 0 || K % kBlockK != 0)
    return HQ_ERR_BAD_SHAPE;
  if (group_size <= 0 || group_size % kBlockK != 0 || K % group_size != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(X_half) || !aligned16(mat) || !aligned16(scales_half) || !aligned16(zeros_half))
    return HQ_ERR_MISALIGNED;
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return HQ_ERR_UNSUPPORTED;
  CUtensorMap map_x, map_w, map_s, map_z;
  int st = encode_x_map(encode, &map_x, X_half, Mb, K);
  if (st != HQ_OK) return st;
  {
    // mat int32[K*3/32][N]: box = 128 columns x 6 rows (one block of 64 inputs)
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 32 * 3)};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 4};
    const cuuint32_t box[2] = {(cuuint32_t)kTileN, 6};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&map_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t*>(mat), dims, strides,
               box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HQ_ERR_UNSUPPORTED;
  }
  for (int which = 0; which < 2; which++) {
    // scales / zeros fp16 [K/group_size][N]: box = 128 columns x 1 group
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / group_size)};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTileN, 1};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(which ? &map_z : &map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
               const_cast<void*>(which ? zeros_half : scales_half), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HQ_ERR_UNSUPPORTED;
  }
  QgemmParams prm = make_params(Y_half, Mb, N, K, group_size, workspace, workspace_bytes, status_word);
  prm.peer_Y = reinterpret_cast<__half* const*>(po.peer_Y);
  prm.y_offset = po.y_offset;
  prm.world = po.world;
  return launch_qgemm<kFmtQ3>(map_x, map_w, map_s, map_z, prm, stream);
}

static int qgemm_nf4_impl(const void* X_half, const uint8_t* B, const float* absmax,
                          const float* lut16, void* Y_half, const PeerOut& po, int Mb, int N, int K,
                          int blocksize, int flags, void* workspace, size_t workspace_bytes,
                          int* status_word, hq_stream_t stream) {
  using namespace hq;
  if (!X_half || !B || !absmax || !lut16 || (!Y_half && !po.peer_Y)) return HQ_ERR_NULL_POINTER;
  if (po.peer_Y && (po.world < 1 || po.world > 32 || po.y_offset < 0)) return HQ_ERR_BAD_SHAPE;
  if (Mb <= 0 || Mb > kMaxTokens || N <= 0 || K <= 0 || N % kTileN != 0 || K % kBlockK != 0)
    return HQ_ERR_BAD_SHAPE;
  // one absmax per (row, K block): blocks of 64 k inputs that never straddle a row
  if (blocksize <= 0 || blocksize % kBlockK != 0 || K % blocksize != 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned16(X_half) || !aligned16(B) || ((uintptr_t)absmax & 3u) != 0)
    return HQ_ERR_MISALIGNED;
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return HQ_ERR_UNSUPPORTED;
  CUtensorMap map_x, map_w;
  int st = encode_x_map(encode, &map_x, X_half, Mb, K);
  if (st != HQ_OK) return st;
  {
    // B uint8[N][K/2]: box = 32 bytes (64 codes) x 128 rows
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    const cuuint32_t box[2] = {32, (cuuint32_t)kTileN};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(B), dims, strides, box,
               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HQ_ERR_UNSUPPORTED;
  }
  QgemmParams prm = make_params(Y_half, Mb, N, K, blocksize, workspace, workspace_bytes, status_word);
  prm.absmax = absmax;
  prm.lut16 = lut16;
  prm.low_first = (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0;
  prm.peer_Y = reinterpret_cast<__half* const*>(po.peer_Y);
  prm.y_offset = po.y_offset;
  prm.world = po.world;
  return launch_qgemm<kFmtNf4>(map_x, map_w, map_w, map_w, prm, stream);
}

extern "C" {

size_t hq_qgemm_workspace_bytes(int Mb, int N) {
  if (Mb <= 0 || N <= 0) return 0;
  return hq::qgemm_ws_bytes(Mb, N);
}

int hq_qgemm_q3_f16(const void* X_half, const int32_t* mat, const void* scales_half,
                    const void* zeros_half, void* Y_half, int Mb, int N, int K, int group_size,
                    void* workspace, size_t workspace_bytes, int* status_word,
                    hq_stream_t stream) {
  if (!Y_half) return HQ_ERR_NULL_POINTER;
  return qgemm_q3_impl(X_half, mat, scales_half, zeros_half, Y_half, PeerOut(), Mb, N, K,
                       group_size, workspace, workspace_bytes, status_word, stream);
}

int hq_qgemm_q3_f16_peers(const void* X_half, const int32_t* mat, const void* scales_half,
                          const void* zeros_half, void* const* peer_Y_half, long long y_offset,
                          int world, int Mb, int N, int K, int group_size, void* workspace,
                          size_t workspace_bytes, int* status_word, hq_stream_t stream) {
  if (!peer_Y_half) return HQ_ERR_NULL_POINTER;
  PeerOut po;
  po.peer_Y = peer_Y_half;
  po.y_offset = y_offset;
  po.world = world;
  return qgemm_q3_impl(X_half, mat, scales_half, zeros_half, nullptr, po, Mb, N, K, group_size,
                       workspace, workspace_bytes, status_word, stream);
}

int hq_qgemm_nf4_f16(const void* X_half, const uint8_t* B, const float* absmax, const float* lut16,
                     void* Y_half, int Mb, int N, int K, int blocksize, int flags, void* workspace,
                     size_t workspace_bytes, int* status_word, hq_stream_t stream) {
  if (!Y_half) return HQ_ERR_NULL_POINTER;
  return qgemm_nf4_impl(X_half, B, absmax, lut16, Y_half, PeerOut(), Mb, N, K, blocksize, flags,
                        workspace, workspace_bytes, status_word, stream);
}

int hq_qgemm_nf4_f16_peers(const void* X_half, const uint8_t* B, const float* absmax,
                           const float* lut16, void* const* peer_Y_half, long long y_offset,
                           int world, int Mb, int N, int K, int blocksize, int flags,
                           void* workspace, size_t workspace_bytes, int* status_word,
                           hq_stream_t stream) {
  if (!peer_Y_half) return HQ_ERR_NULL_POINTER;
  PeerOut po;
  po.peer_Y = peer_Y_half;
  po.y_offset = y_offset;
  po.world = world;
  return qgemm_nf4_impl(X_half, B, absmax, lut16, nullptr, po, Mb, N, K, blocksize, flags,
                        workspace, workspace_bytes, status_word, stream);
}

}  // extern "C"
