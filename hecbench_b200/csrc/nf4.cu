// NF4 blockwise 4-bit dequantize and batch-1 GEMV for sm_100a.
//
// Format: element e of the flattened [N][K] matrix has its 4-bit code in byte
// e/2 (even element = high nibble by default, low nibble with
// HQ_NF4_LOW_NIBBLE_FIRST); one fp32 absmax per `blocksize` consecutive
// elements; the 16 levels are a runtime fp32 table.
//   dequant : out[e] = half_rn(lut16[code] * absmax[e/blocksize])   (bit exact)
//   gemv    : out[n] = half_rn(sum_k A[k] * lut16[code[n][k]] * absmax[...])
//
// GEMV design (HBM-bound, 0.5 B of codes + 1/16 B of absmax per weight):
//  * one persistent CTA of 1024 threads per SM; rows are dealt round-robin to
//    CTAs and, inside a CTA, to groups of S warps; warp q of a group owns the
//    K slice [q*1024*C, (q+1)*1024*C) of every row of its group, a lane reads
//    16 bytes (32 codes) per chunk, so a warp streams 512 contiguous bytes;
//  * packed codes and their absmax are staged through shared memory with
//    per-lane asynchronous copies (cp.async), kStages rows deep: 128 KiB of
//    weights are in flight per SM without holding a single register, which is
//    what it takes to cover HBM latency at full bandwidth; each lane reads back
//    only the slots it filled itself, so no barrier guards the ring; the first
//    kStages rows are requested before the lookup table is built;
//  * the lane's slice of the input vector never changes, so it lives in
//    registers for the whole kernel;
//  * one byte = two codes = one shared-memory lookup into a 256-entry half2
//    table (lut[first code], lut[second code]); the table is stored once per
//    bank with a 256-byte row per byte value (row b: 32 lane copies in its
//    first 128 bytes), so the 32 random lookups of a warp never conflict and
//    the table offset (b << 8) | lane*4 is ONE byte-permute of the packed word
//    and the lane offset - no shift, no mask;
//  * products are summed in half2 over the 32 weights of a chunk (two
//    accumulators of 8 fused multiply-adds), then scaled by the chunk's fp32
//    absmax in fp32;
//  * per-lane partial sums of a row go to shared memory (into the unused second
//    128 bytes of the table rows); after kRound rows the
//    S warps of the group meet at a named barrier and each finishes some of
//    the rows (sum over the slices, warp-shuffle tree, one fp16 store).
#include <algorithm>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;        // dequant kernel
constexpr int kGemvThreads = 1024;   // GEMV: one persistent CTA per SM
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kStageChunks = 8;      // 16-byte chunks in flight per lane (shared-memory ring)
constexpr int kRound = 4;            // rows between two group barriers

constexpr int kLutBytes = 256 * 256;  // table rows interleaved with the partial-sum slots
// The table sits at the fixed shared-window address kLutImm, so that a lookup
// address is the byte-permute {0, 0, byte value, lane*4} plus an immediate.
constexpr int kLutImm = 2048;

template <int IMM>
__device__ __forceinline__ uint32_t lds_u32_imm(uint32_t addr) {
  // not volatile: the table is constant after the prologue barrier
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
  return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool pred) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %2, 0;\n"
      " @p cp.async.cg.shared.global [%0], [%1], 16;\n}\n" ::"r"(dst), "l"(src), "r"((int)pred)
      : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, bool pred) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %2, 0;\n"
      " @p cp.async.ca.shared.global [%0], [%1], 4;\n}\n" ::"r"(dst), "l"(src), "r"((int)pred)
      : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// sum of the 32 products of one 16-byte chunk against 16 half2 inputs
__device__ __forceinline__ float chunk_dot(const uint4& codes, const uint4 (&xp)[4],
                                           uint32_t lane4) {
  const uint32_t w[4] = {codes.x, codes.y, codes.z, codes.w};
  __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t xw[4] = {xp[i].x, xp[i].y, xp[i].z, xp[i].w};
    // byte k of the word -> (byte << 8) | lane*4: bytes {lane4.0, w.k, 0, 0}
    const uint32_t o0 = __byte_perm(w[i], lane4, 0x7604);
    const uint32_t o1 = __byte_perm(w[i], lane4, 0x7614);
    const uint32_t o2 = __byte_perm(w[i], lane4, 0x7624);
    const uint32_t o3 = __byte_perm(w[i], lane4, 0x7634);
    const uint32_t l0 = lds_u32_imm<kLutImm>(o0);
    const uint32_t l1 = lds_u32_imm<kLutImm>(o1);
    const uint32_t l2 = lds_u32_imm<kLutImm>(o2);
    const uint32_t l3 = lds_u32_imm<kLutImm>(o3);
    a0 = __hfma2(u32_as_half2(l0), u32_as_half2(xw[0]), a0);
    a1 = __hfma2(u32_as_half2(l1), u32_as_half2(xw[1]), a1);
    a0 = __hfma2(u32_as_half2(l2), u32_as_half2(xw[2]), a0);
    a1 = __hfma2(u32_as_half2(l3), u32_as_half2(xw[3]), a1);
  }
  const float2 f = __half22float2(__hadd2(a0, a1));
  return f.x + f.y;
}

__device__ __forceinline__ void group_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

struct GemvParams {
  const __half* A;
  const uint8_t* B;
  const float* absmax;
  const float* lut16;
  __half* out;
  int nchunks;          // K / 32
  int S, G;             // warps per row, row groups per CTA
  int rows_base, rows_rem;  // N / (grid*G), N % (grid*G)
  int cpb_shift;        // log2(chunks per absmax block), or -1
  int cpb;              // chunks per absmax block
  int low_first;
  unsigned long long w_step;   // bytes between two rows of one group
  unsigned int a_step;         // absmax entries between two rows of one group (ALIGNED only)
  // fused gather (null when unused): every result is also stored into the
  // gathered vector of each GPU of the node at element gather_offset + n
  __half* const* peer_out;
  uint32_t* const* peer_flags;  // flags array of each rank; this rank writes word `rank`
  unsigned* sync_words;         // local: [0] CTAs finished, [1] launches completed
  int world, rank;
  long long gather_offset;
  // optional: before the input vector is read, wait (bounded) until every rank's
  // flag has reached this rank's launch count, i.e. until the previous fused
  // gather - which produced the input of this layer - has landed everywhere
  const uint32_t* wait_flags;
  int early_fetch;  // weights may be fetched before the preceding kernel in the stream has finished
  int* status;
};

// store one result locally and, for the fused gather, into every peer's vector
__device__ __forceinline__ void store_result(const GemvParams& p, __half* local, long long n,
                                             float v) {
  const __half h = __float2half_rn(v);
  if (p.peer_out == nullptr) *local = h;
  else p.peer_out[p.rank][p.gather_offset + n] = h;  // own copy first; peers get it in bulk
}

// C = chunks (32 codes) per lane per row; S warps share a row (ST > 0: compile
// time, ST == 0: run time), G groups per CTA.  ALIGNED: every row starts on an
// absmax block boundary and blocks are a power of two, so the absmax pointer
// of a lane advances by a constant.  Every instruction of this kernel is
// executed by 32 warps per SM, so per-thread setup is kept to a minimum:
// nothing is divided on the device.
template <int C, int ST, bool ALIGNED>
__global__ void __launch_bounds__(kGemvThreads, 1)
nf4_gemv_kernel(const GemvParams p) {
  constexpr int kStages = kStageChunks / C;  // rows in flight per lane
  extern __shared__ __align__(16) unsigned char dsm_raw[];
  // [pad up to shared address kLutImm] table rows (256 x 256 B: lane copies |
  // partial-sum slot) | [kStages][C][1024] uint4 | [kStages][C][1024] float
  if (smem_u32(dsm_raw) > (uint32_t)kLutImm) return;  // never on sm_100 (1 KiB reserved)
  // Programmatic dependent launch: let the next kernel of the stream start its
  // own prologue as soon as this grid is resident, and do not touch global
  // memory that earlier work may still be writing before the wait below.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!p.early_fetch) asm volatile("griddepcontrol.wait;" ::: "memory");
  unsigned char* dsm = dsm_raw + (kLutImm - smem_u32(dsm_raw));
  const int S = ST > 0 ? ST : p.S;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = warp / S, q = warp - g * S;
  const int G = p.G;

  // rows of this group: n = blockIdx.x + gridDim.x * (g + G * j), j < my_rows
  const int row_first = blockIdx.x + gridDim.x * g;
  const int row_stride = gridDim.x * G;
  const int my_rows = g < G ? p.rows_base + (row_first < p.rows_rem ? 1 : 0) : 0;

  // this lane's chunk columns; a lane beyond the row end copies nothing and
  // sees zero scales in its (zero-filled) ring slots
  const uint32_t ring_w0 = smem_u32(dsm + kLutBytes) + tid * 16;
  const uint32_t ring_s0 = smem_u32(dsm + kLutBytes + kStageChunks * kGemvThreads * 16) + tid * 4;
  const unsigned char* wp[C];
  const float* ap[C];
  bool live[C];
  uint32_t ci[C];
#pragma unroll
  for (int i = 0; i < C; i++) {
    const int c = (q * C + i) * 32 + lane;
    live[i] = c < p.nchunks;
    const int cc = live[i] ? c : 0;
    wp[i] = p.B + (size_t)row_first * ((size_t)p.nchunks * 16) + (size_t)cc * 16;
    ci[i] = (uint32_t)row_first * (uint32_t)p.nchunks + (uint32_t)cc;
    ap[i] = p.absmax + (ALIGNED ? (ci[i] >> p.cpb_shift) : 0u);
    if (!live[i]) {
#pragma unroll
      for (int st = 0; st < kStages; st++) {
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(
                         ring_w0 + (uint32_t)((st * C + i) * kGemvThreads * 16)), "r"(0));
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(
                         ring_s0 + (uint32_t)((st * C + i) * kGemvThreads * 4)), "r"(0));
      }
    }
  }
  int to_issue = my_rows;  // rows not yet requested

#define HQ_NF4_ISSUE(STAGE)                                                                     \
  {                                                                                             \
    const bool ok = to_issue > 0;                                                               \
    _Pragma("unroll") for (int i = 0; i < C; i++) {                                             \
      const float* a = ap[i];                                                                   \
      if (!ALIGNED)                                                                             \
        a = p.absmax + (p.cpb_shift >= 0 ? (ci[i] >> p.cpb_shift) : (ci[i] / (uint32_t)p.cpb)); \
      cp_async_16(ring_w0 + (uint32_t)(((STAGE)*C + i) * kGemvThreads * 16), wp[i],             \
                  ok && live[i]);                                                               \
      cp_async_4(ring_s0 + (uint32_t)(((STAGE)*C + i) * kGemvThreads * 4), a, ok && live[i]);   \
      wp[i] += p.w_step;                                                                        \
      if (ALIGNED) ap[i] += p.a_step;                                                           \
      else ci[i] += (uint32_t)row_stride * (uint32_t)p.nchunks;                                 \
    }                                                                                           \
    cp_async_commit();                                                                          \
    to_issue--;                                                                                 \
  }
#pragma unroll
  for (int st = 0; st < kStages; st++) HQ_NF4_ISSUE(st)

  // ---- prologue (overlaps the copies above): byte table, input slice ----
  {
    const int entry = tid >> 2, quarter = tid & 3;  // four threads per 128-byte table row
    const int hi = entry >> 4, lo = entry & 15;
    const int first = p.low_first ? lo : hi, second = p.low_first ? hi : lo;
    const uint32_t u = half2_as_u32(__floats2half2_rn(p.lut16[first], p.lut16[second]));
    const uint4 u4 = make_uint4(u, u, u, u);
    uint4* row = reinterpret_cast<uint4*>(dsm + (size_t)entry * 256 + quarter * 32);
    row[entry & 1] = u4;
    row[(entry & 1) ^ 1] = u4;
  }
  // the input vector (and, without early_fetch, everything) is read only after
  // the preceding kernel has completed
  if (p.early_fetch) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (p.wait_flags != nullptr) {
    if (tid < p.world) {
      const unsigned want = *reinterpret_cast<volatile unsigned*>(p.sync_words + 1);
      const volatile uint32_t* f = p.wait_flags + tid;
      bool landed = false;
      for (unsigned spin = 0; spin < (1u << 20); spin++) {
        if ((int)(*f - want) >= 0) { landed = true; break; }
        __nanosleep(32);
      }
      if (landed) __threadfence_system();
      else if (p.status != nullptr) atomicExch(p.status, 1);
    }
    __syncthreads();
  }
  uint4 xr[C][4];
#pragma unroll
  for (int i = 0; i < C; i++) {
    const int c = (q * C + i) * 32 + lane;
    const uint4* xp = reinterpret_cast<const uint4*>(p.A) + 4 * (live[i] ? c : 0);
#pragma unroll
    for (int t = 0; t < 4; t++) xr[i][t] = p.wait_flags ? __ldcg(xp + t) : __ldg(xp + t);
  }
  __syncthreads();

  const uint32_t lane4 = lane * 4;
  __half* outp = p.out + row_first;  // row j of this group is outp[j * row_stride]
  // partial-sum slot s (32 floats) lives in the second half of table row s
  float* const part_lane = reinterpret_cast<float*>(dsm + 128) + lane;  // slot s: part_lane[s*64]
  const uint4* ring_w = reinterpret_cast<const uint4*>(dsm + kLutBytes) + tid;
  const float* ring_s =
      reinterpret_cast<const float*>(dsm + kLutBytes + kStageChunks * kGemvThreads * 16) + tid;

  int rows_left = my_rows;
  const int slot_g = g * kRound * S;        // slots of this group: [parity][g][d][t]
  const int slot_flip = G * kRound * S;
  int parity = 0;                           // used only when a super-round is one round
  constexpr int kRoundsPerPass = kStages / kRound;

  // one round = kRound rows out of compile-time stages RR*kRound .. +kRound-1
#define HQ_NF4_ROUND(RR)                                                                       \
  {                                                                                            \
    const int rows_in_round = min(kRound, rows_left);                                          \
    const int slot0 = slot_g + ((kRoundsPerPass > 1 ? ((RR)&1) : parity) ? slot_flip : 0);      \
    _Pragma("unroll") for (int d = 0; d < kRound; d++) {                                       \
      cp_async_wait<kStages - 1>();                                                            \
      if (d < rows_in_round) {                                                                 \
        float acc = 0.f;                                                                       \
        _Pragma("unroll") for (int i = 0; i < C; i++) acc =                                    \
            fmaf(chunk_dot(ring_w[(((RR)*kRound + d) * C + i) * kGemvThreads], xr[i], lane4),       \
                 ring_s[(((RR)*kRound + d) * C + i) * kGemvThreads], acc);                      \
        if (S > 1) {                                                                           \
          part_lane[(slot0 + d * S + q) * 64] = acc;                                           \
        } else {                                                                               \
          acc = warp_sum(acc);                                                                 \
          if (lane == 0) store_result(p, outp, outp - p.out, acc);                             \
          outp += row_stride;                                                                  \
        }                                                                                      \
      }                                                                                        \
      HQ_NF4_ISSUE((RR)*kRound + d)                                                            \
    }                                                                                          \
    if (S > 1) {                                                                               \
      group_barrier(1 + g, S * 32);                                                            \
      for (int d = q; d < rows_in_round; d += S) {                                             \
        float v = 0.f;                                                                         \
        if (ST > 0) {                                                                          \
          _Pragma("unroll") for (int t = 0; t < (ST > 0 ? ST : 1); t++) v +=                   \
              part_lane[(slot0 + d * S + t) * 64];                                             \
        } else {                                                                               \
          for (int t = 0; t < S; t++) v += part_lane[(slot0 + d * S + t) * 64];                \
        }                                                                                      \
        v = warp_sum(v);                                                                       \
        if (lane == 0)                                                                         \
          store_result(p, outp + (size_t)d * row_stride, (outp - p.out) + (long long)d * row_stride, v); \
      }                                                                                        \
      outp += (size_t)kRound * row_stride;                                                     \
    }                                                                                          \
    parity ^= 1;                                                                               \
    rows_left -= kRound;                                                                       \
  }

  while (rows_left > 0) {
    HQ_NF4_ROUND(0)
    if (kRoundsPerPass > 1) {
      if (rows_left <= 0) break;
      HQ_NF4_ROUND(1)
    }
  }
#undef HQ_NF4_ROUND
  cp_async_wait<0>();
  if (p.peer_out != nullptr) {
    // Fused gather epilogue: every CTA has stored its results into this GPU's own
    // copy of the gathered vector; the last CTA of the grid to finish copies the
    // whole slice to every peer with 16-byte stores over NVLink, makes them
    // visible system-wide and then tells every peer, by one flag word per
    // (receiver, sender), that this launch's slice has landed.
    __shared__ unsigned s_last_cta;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned prev = atomicAdd(p.sync_words, 1u);
      s_last_cta = (prev == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (s_last_cta) {
      __threadfence();
      const int n_slice = p.rows_base * (int)(gridDim.x * p.G) + p.rows_rem;  // rows of this rank
      const __half* mine = p.peer_out[p.rank] + p.gather_offset;
      const bool vec_ok = ((p.gather_offset | (long long)n_slice) & 7) == 0;
      for (int r = 0; r < p.world; r++) {
        if (r == p.rank) continue;
        __half* dst = p.peer_out[r] + p.gather_offset;
        if (vec_ok) {
          for (int i = tid; i < n_slice / 8; i += kGemvThreads)
            reinterpret_cast<uint4*>(dst)[i] = __ldcg(reinterpret_cast<const uint4*>(mine) + i);
        } else {
          for (int i = tid; i < n_slice; i += kGemvThreads)
            reinterpret_cast<unsigned short*>(dst)[i] =
                __ldcg(reinterpret_cast<const unsigned short*>(mine) + i);
        }
      }
      __threadfence_system();
      __syncthreads();
      if (tid == 0) {
        p.sync_words[0] = 0u;
        const unsigned epoch = p.sync_words[1] + 1u;
        p.sync_words[1] = epoch;
        __threadfence_system();
        for (int r = 0; r < p.world; r++)
          *reinterpret_cast<volatile uint32_t*>(p.peer_flags[r] + p.rank) = epoch;
      }
    }
  }
#undef HQ_NF4_ISSUE
}

// One thread: 4 bytes of codes (8 elements) -> 16 bytes of fp16.
__global__ void __launch_bounds__(kThreads)
nf4_dequant_kernel(const uint8_t* __restrict__ B, const float* __restrict__ absmax,
                   const float* __restrict__ lut16, __half* __restrict__ out, size_t nwords,
                   int words_per_block, int low_first) {
  __shared__ float lut[16 * 32];  // [code][lane]
  const int tid = threadIdx.x, lane = tid & 31;
  for (int i = tid; i < 16 * 32; i += kThreads) lut[i] = lut16[i >> 5];
  __syncthreads();
  const float* lut_lane = lut + lane;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t w = (size_t)blockIdx.x * kThreads + tid; w < nwords; w += stride) {
    const uint32_t codes = ldg_stream_u32(reinterpret_cast<const uint32_t*>(B) + w);
    const float s = __ldg(absmax + w / (size_t)words_per_block);
    uint32_t o[4];
#pragma unroll
    for (int b = 0; b < 4; b++) {
      const uint32_t byte = (codes >> (8 * b)) & 0xffu;
      const uint32_t hi = byte >> 4, lo = byte & 15u;
      const uint32_t first = low_first ? lo : hi, second = low_first ? hi : lo;
      const float v0 = __fmul_rn(lut_lane[first * 32], s);
      const float v1 = __fmul_rn(lut_lane[second * 32], s);
      o[b] = half2_as_u32(__floats2half2_rn(v0, v1));
    }
    reinterpret_cast<uint4*>(out)[w] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// One warp: lane r waits (bounded) until rank r's flag has reached this rank's
// own launch count, i.e. until rank r's slice of the latest gather has landed.
__global__ void gather_wait_kernel(const uint32_t* flags, const unsigned* sync_words, int world,
                                   int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const unsigned want = sync_words[1];
  const volatile uint32_t* f = flags + r;
  bool ok = false;
  for (unsigned spin = 0; spin < (1u << 22); spin++) {
    // flags only grow; "reached" is tested modulo 2^32
    if ((int)(*f - want) >= 0) { ok = true; break; }
    __nanosleep(64);
  }
  if (ok) __threadfence_system();
  else if (status != nullptr) atomicExch(status, 1);
}

// One CTA per rank r of the node: CTA r copies this rank's finished slice
// (already in its own gathered vector) into rank r's vector with 16-byte stores
// over NVLink, makes the stores visible system-wide, raises this rank's flag on
// GPU r, then waits (bounded) until rank r's flag on THIS GPU has reached the
// same launch count.  The last CTA to finish advances the launch count.
constexpr int kPublishThreads = 1024;
__global__ void __launch_bounds__(kPublishThreads, 1)
gather_publish_kernel(__half* const* peer_out, long long offset, int n_slice,
                      uint32_t* const* peer_flags, unsigned* sync_words, int world, int rank,
                      int* status) {
  const int tid = threadIdx.x;
  const int r = blockIdx.x;
  // Programmatic dependent launch: these CTAs may become resident while the kernel
  // that produces the slice is still draining, and the next kernel of the stream
  // may start its own prologue while they wait for the other ranks; the slice is
  // read only after the producing kernel has completed.
  pdl_launch_dependents();
  pdl_wait();
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(sync_words + 1) + 1u;
  if (r != rank) {
    const __half* mine = peer_out[rank] + offset;
    __half* dst = peer_out[r] + offset;
    const bool vec_ok = ((offset | (long long)n_slice) & 7) == 0;
    if (vec_ok) {
      for (int i = tid; i < n_slice / 8; i += kPublishThreads)
        reinterpret_cast<uint4*>(dst)[i] = __ldcg(reinterpret_cast<const uint4*>(mine) + i);
    } else {
      for (int i = tid; i < n_slice; i += kPublishThreads)
        reinterpret_cast<unsigned short*>(dst)[i] =
            __ldcg(reinterpret_cast<const unsigned short*>(mine) + i);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (tid == 0) {
    *reinterpret_cast<volatile uint32_t*>(peer_flags[r] + rank) = epoch;
    const volatile uint32_t* f = peer_flags[rank] + r;
    bool landed = false;
    for (unsigned spin = 0; spin < (1u << 22); spin++) {
      if ((int)(*f - epoch) >= 0) { landed = true; break; }
      __nanosleep(32);
    }
    if (landed) __threadfence_system();
    else if (status != nullptr) atomicExch(status, 1);
    // every CTA has read the old launch count before it gets here
    __threadfence();
    const unsigned prev = atomicAdd(sync_words, 1u);
    if (prev == (unsigned)world - 1u) {
      sync_words[1] = epoch;
      sync_words[0] = 0u;
    }
  }
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_gather_publish(void* const* peer_out_half, long long offset, int n_slice,
                      uint32_t* const* peer_flags, unsigned* sync_words, int world, int rank,
                      int* status, hq_stream_t stream) {
  using namespace hq;
  if (!peer_out_half || !peer_flags || !sync_words) return HQ_ERR_NULL_POINTER;
  if (world < 1 || world > 32 || rank < 0 || rank >= world || n_slice <= 0) return HQ_ERR_BAD_SHAPE;
  return cuda_status(launch_pdl(gather_publish_kernel, dim3(world), dim3(kPublishThreads), 0,
                                (cudaStream_t)stream,
                                reinterpret_cast<__half* const*>(peer_out_half), offset, n_slice,
                                peer_flags, sync_words, world, rank, status));
}

int hq_gather_wait(const uint32_t* local_flags, const unsigned* sync_words, int world, int* status,
                   hq_stream_t stream) {
  using namespace hq;
  if (!local_flags || !sync_words) return HQ_ERR_NULL_POINTER;
  if (world < 1 || world > 32) return HQ_ERR_BAD_SHAPE;
  gather_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(local_flags, sync_words, world, status);
  return launch_status();
}

int hq_nf4_dequant_f16(const uint8_t* B, const float* absmax, const float* lut16, void* out_half,
                       size_t n, int blocksize, int flags, hq_stream_t stream) {
  using namespace hq;
  if (!lut16 || (n && (!B || !absmax || !out_half))) return HQ_ERR_NULL_POINTER;
  if (blocksize <= 0 || blocksize % 32 != 0 || n % 32 != 0) return HQ_ERR_BAD_SHAPE;
  if (n == 0) return HQ_OK;
  if (!aligned4(B) || !aligned16(out_half)) return HQ_ERR_MISALIGNED;
  const size_t nwords = n / 8;
  const size_t want = (nwords + kThreads - 1) / kThreads;
  const size_t cap = (size_t)sm_count() * 16;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  nf4_dequant_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
      B, absmax, lut16, reinterpret_cast<__half*>(out_half), nwords, blocksize / 8,
      (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0);
  return launch_status();
}

static int nf4_gemv_impl(const void* A_half, const uint8_t* B, const float* absmax,
                         const float* lut16, void* out_half, int N, int K, int blocksize, int flags,
                         void* const* peer_out, uint32_t* const* peer_flags, unsigned* sync_words,
                         int world, int rank, long long gather_offset, const uint32_t* wait_flags,
                         int* status, hq_stream_t stream) {
  using namespace hq;
  if (!A_half || !B || !absmax || !lut16 || (!out_half && !peer_out)) return HQ_ERR_NULL_POINTER;
  if (N <= 0 || K <= 0 || K % 32 != 0 || blocksize <= 0 || blocksize % 32 != 0 ||
      false)
    return HQ_ERR_BAD_SHAPE;
  if (!aligned16(B) || !aligned16(A_half)) return HQ_ERR_MISALIGNED;
  if ((uint64_t)N * (uint64_t)(K / 32) > 0xffffffffull) return HQ_ERR_TOO_LARGE;
  const int nchunks = K / 32;
  // warps per row S and chunks per lane C: C = 1 unless that needs more than 15
  // named barriers (S = 2) or more warps than a CTA has.
  const int cols = (nchunks + 31) / 32;  // 1024-input slices per row
  int C = 1;
  if (cols == 2 || cols > kGemvWarps) C = 2;
  const int S = (cols + C - 1) / C;
  if (S > kGemvWarps) return HQ_ERR_TOO_LARGE;  // K > 65536
  int G = kGemvWarps / S;
  if (S > 1 && G > 15) G = 15;
  // room for the pad that brings the table to shared address kLutImm wherever the
  // dynamic region starts (at or below kLutImm)
  const size_t smem = (size_t)kLutImm + kLutBytes + (size_t)kStageChunks * kGemvThreads * 20;
  const int sms = sm_count();
  const int grid = std::min(sms, (N + G - 1) / G);
  const int cpb = blocksize / 32;
  int shift = -1;
  if ((cpb & (cpb - 1)) == 0) {
    shift = 0;
    while ((1 << shift) < cpb) shift++;
  }
  const bool aligned = shift >= 0 && nchunks % cpb == 0;
  GemvParams prm;
  prm.A = reinterpret_cast<const __half*>(A_half);
  prm.B = B;
  prm.absmax = absmax;
  prm.lut16 = lut16;
  prm.out = reinterpret_cast<__half*>(out_half);
  prm.nchunks = nchunks;
  prm.S = S;
  prm.G = G;
  prm.rows_base = N / (grid * G);
  prm.rows_rem = N % (grid * G);
  prm.cpb_shift = shift;
  prm.cpb = cpb;
  prm.low_first = (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0;
  prm.w_step = (unsigned long long)grid * G * nchunks * 16ull;
  prm.a_step = aligned ? (unsigned)(((unsigned long long)grid * G * nchunks) >> shift) : 0u;
  prm.peer_out = reinterpret_cast<__half* const*>(peer_out);
  prm.peer_flags = peer_flags;
  prm.sync_words = sync_words;
  prm.world = world;
  prm.rank = rank;
  prm.gather_offset = gather_offset;
  prm.wait_flags = wait_flags;
  prm.status = status;
  prm.early_fetch = (flags & HQ_NF4_WEIGHTS_RESIDENT) ? 1 : 0;
  cudaStream_t st = (cudaStream_t)stream;
#define HQ_NF4_LAUNCH(CC, SS, AL)                                                               \
  {                                                                                             \
    auto kern = nf4_gemv_kernel<CC, SS, AL>;                                                    \
    cudaError_t e =                                                                             \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    if (e != cudaSuccess) return cuda_status(e);                                                \
    cudaLaunchConfig_t cfg = {};                                                                \
    cfg.gridDim = dim3(grid);                                                                   \
    cfg.blockDim = dim3(kGemvThreads);                                                          \
    cfg.dynamicSmemBytes = smem;                                                                \
    cfg.stream = st;                                                                            \
    cudaLaunchAttribute attr[1];                                                                \
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                            \
    attr[0].val.programmaticStreamSerializationAllowed = 1;                                     \
    cfg.attrs = attr;                                                                           \
    cfg.numAttrs = 1;                                                                           \
    e = cudaLaunchKernelEx(&cfg, kern, prm);                                                    \
    if (e != cudaSuccess) return cuda_status(e);                                                \
  }
  if (C == 1 && S == 4 && aligned) HQ_NF4_LAUNCH(1, 4, true)
  else if (C == 1 && S == 8 && aligned) HQ_NF4_LAUNCH(1, 8, true)
  else if (C == 1 && S == 1 && aligned) HQ_NF4_LAUNCH(1, 1, true)
  else if (C == 1 && aligned) HQ_NF4_LAUNCH(1, 0, true)
  else if (C == 1) HQ_NF4_LAUNCH(1, 0, false)
  else if (S == 2 && aligned) HQ_NF4_LAUNCH(2, 2, true)
  else if (aligned) HQ_NF4_LAUNCH(2, 0, true)
  else HQ_NF4_LAUNCH(2, 0, false)
#undef HQ_NF4_LAUNCH
  return launch_status();
}

int hq_nf4_gemv_f16(const void* A_half, const uint8_t* B, const float* absmax, const float* lut16,
                    void* out_half, int N, int K, int blocksize, int flags, hq_stream_t stream) {
  return nf4_gemv_impl(A_half, B, absmax, lut16, out_half, N, K, blocksize, flags, nullptr, nullptr,
                       nullptr, 1, 0, 0, nullptr, nullptr, stream);
}

int hq_nf4_gemv_f16_gather(const void* A_half, const uint8_t* B, const float* absmax,
                           const float* lut16, int N, int K, int blocksize, int flags,
                           void* const* peer_out_half, long long gather_offset,
                           uint32_t* const* peer_flags, unsigned* sync_words, int world, int rank,
                           const uint32_t* wait_flags, int* status, hq_stream_t stream) {
  if (!peer_out_half || !peer_flags || !sync_words) return HQ_ERR_NULL_POINTER;
  if (world < 1 || world > 32 || rank < 0 || rank >= world) return HQ_ERR_BAD_SHAPE;
  return nf4_gemv_impl(A_half, B, absmax, lut16, nullptr, N, K, blocksize, flags, peer_out_half,
                       peer_flags, sync_words, world, rank, gather_offset, wait_flags, status,
                       stream);
}

}  // extern "C"
