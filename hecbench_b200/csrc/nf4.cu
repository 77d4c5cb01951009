// NF4 blockwise 4-bit dequantize and batch-1 GEMV for sm_100a.
//
// Format: element e of the flattened [N][K] matrix has its 4-bit code in byte
// e/2 (even element = high nibble by default, low nibble with
// HQ_NF4_LOW_NIBBLE_FIRST); one fp32 absmax per `blocksize` consecutive
// elements; the 16 levels are a runtime fp32 table.
//   dequant : out[e] = half_rn(lut16[code] * absmax[e/blocksize])   (bit exact)
//   gemv    : out[n] = half_rn(sum_k A[k] * lut16[code[n][k]] * absmax[...])
//
// GEMV design (HBM-bound, 0.5 B of codes + 1/16 B of absmax per weight; the
// second wall is instruction issue, so the kernel is built around the number
// of instructions per weight):
//  * one persistent CTA per SM; rows are dealt round-robin to CTAs and, inside
//    a CTA, to groups of S warps; warp q of a group owns the K slice
//    [q*1024*C, (q+1)*1024*C) of every row of its group; a lane reads C
//    16-byte chunks (32 codes each) per row, and the 32 lanes of a warp read
//    512 contiguous bytes per load instruction;
//  * packed codes and absmax go from global memory straight into registers
//    (128-bit streaming loads that bypass L1), D rows ahead of their use: the
//    D*C outstanding 16-byte loads per thread are what covers the HBM
//    latency, and nothing is staged through shared memory, whose bandwidth the
//    table lookups need (asking the L2 for rows further ahead with bulk
//    prefetches was measured and made the kernel slower);
//  * the lane's slice of the input vector never changes, so it lives in
//    registers for the whole kernel;
//  * one byte = two codes = one shared-memory lookup into a 256-entry half2
//    table (lut[first code], lut[second code]); the table is stored once per
//    bank with a 256-byte row per byte value (row b: 32 lane copies in its
//    first 128 bytes), so the 32 random lookups of a warp never conflict and
//    the table offset (b << 8) | lane*4 is ONE byte-permute of the packed word
//    and the lane offset - no shift, no mask;
//  * products are summed in half2 over the 32 weights of a chunk (four
//    accumulators of 4 fused multiply-adds), then scaled by the chunk's fp32
//    absmax in fp32;
//  * per-lane partial sums of a row go to shared memory; after D rows the S
//    warps of the group meet at a named barrier and each finishes some of the
//    rows (sum over the slices, warp-shuffle tree, one fp16 store).  With
//    S == 1 a warp finishes its rows alone and there is no barrier.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "hq_common.cuh"

namespace hq {
namespace {

constexpr int kThreads = 256;        // dequant kernel
constexpr unsigned kDefaultPolls = 1u << 21;  // about a second of polling with back-off

constexpr int kLutBytes = 256 * 256;  // 256 table rows of 256 bytes (first 128: lane copies)
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

// Loads that keep their place in the program order among the other ordered
// loads (asm volatile): the prologue depends on WHICH request reaches the memory
// system first.
__device__ __forceinline__ float ldg_ordered_f32(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// 16-byte asynchronous copy global -> shared (no register holds the data)
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// sum of the 32 products of one 16-byte chunk against 16 half2 inputs
__device__ __forceinline__ float chunk_dot(const uint4& codes, const uint4 (&xp)[4],
                                           uint32_t lane4) {
  const uint32_t w[4] = {codes.x, codes.y, codes.z, codes.w};
  __half2 a0 = __float2half2_rn(0.f), a1 = a0, a2 = a0, a3 = a0;
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
    a2 = __hfma2(u32_as_half2(l2), u32_as_half2(xw[2]), a2);
    a3 = __hfma2(u32_as_half2(l3), u32_as_half2(xw[3]), a3);
  }
  const float2 f = __half22float2(__hadd2(__hadd2(a0, a1), __hadd2(a2, a3)));
  return f.x + f.y;
}

__device__ __forceinline__ void group_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// GemvParams::act value (internal): rows are walked in adjacent pairs like value /
// gate rows, but both results are kept and go out as two neighbouring packets in
// ONE 16-byte store per GPU (half as many stores over NVLink as one per row)
constexpr int kPairPackets = 100;

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
  // Low-latency gather (null when unused).  Output: every result is stored as
  // one 8-byte packet {fp16 value, epoch} into element gather_offset + n of the
  // packet vector of EVERY GPU of the node (peer_ll[r], peer-mapped memory).
  // Input: the vector may itself be given as packets (A_ll, element k at
  // A_ll[k * a_stride]); a packet counts once its epoch equals the epoch of the
  // latest completed gather, which sync_words[1] holds.
  uint2* const* peer_ll;
  const uint2* A_ll;
  long long a_stride;
  unsigned* sync_words;         // local: [0] CTAs finished, [1] epoch of the latest completed gather
  int world, rank;
  int multicast;                // peer_ll[0] is a multicast address: one multimem.st per result
  long long gather_offset;
  unsigned max_polls;           // limit of every wait for a packet, in polls
  // buffer extents in bytes, used only by the index-checked build
  unsigned long long b_bytes, absmax_bytes, a_bytes, out_bytes;
  int early_fetch;  // weights may be fetched before the preceding kernel in the stream has finished
  int* status;
  // Fused forms (FUSE kernels only).  gamma != null: the input vector is RMS-
  // normalised and scaled by gamma first.  act != 0: the rows come in pairs
  // (value row 2m, gate row 2m + 1), a group walks pairs instead of rows and
  // output m = value * gate_act(gate).  w_step / a_step then are the distance
  // from a value row to its gate row, the _odd ones from a gate row to the next
  // pair's value row.
  const __half* gamma;
  float eps;
  int act;
  unsigned long long w_step_odd;
  unsigned int a_step_odd;
#ifdef HQ_NF4_TRACE
  unsigned long long* trace;  // development: [CTA][16] globaltimer stamps
#endif
};

#ifdef HQ_NF4_TRACE
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define HQ_STAMP(i) \
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 16 + (i)] = gtime();
#else
#define HQ_STAMP(i)
#endif

__device__ __forceinline__ uint2 ld_packet(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
// one store that the NVSwitch delivers to every GPU of the multicast group
__device__ __forceinline__ void st_packet_multicast(uint2* p, uint32_t value, uint32_t epoch) {
  const unsigned long long v = ((unsigned long long)epoch << 32) | value;
  asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_packet(uint2* p, uint32_t value, uint32_t epoch) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(value), "r"(epoch)
               : "memory");
}
// Waits (bounded) until the packet carries `epoch`; returns its value.  On
// expiry *status becomes 1 and the stale value is returned: the kernel still
// terminates, the host sees the status.
__device__ __forceinline__ uint32_t wait_packet(const uint2* p, uint32_t epoch, unsigned max_polls,
                                                int* status) {
  uint2 v = ld_packet(p);
  if (v.y == epoch) return v.x;
  for (unsigned spin = 0; spin < max_polls; spin++) {
    __nanosleep(20);
    v = ld_packet(p);
    if (v.y == epoch) return v.x;
  }
  if (status != nullptr) atomicExch(status, 1);
  return v.x;
}

// The input vector given as packets -> plain fp16 in shared memory.  The loads of
// a batch are all issued before the first is examined (examined one at a time, a
// thread's packets cost one L2 round trip each: 8 x 0.5 us at K = 4096); only a
// packet that does not carry the epoch yet is polled.
template <int THREADS>
__device__ __forceinline__ void stage_packets(__half* xs, const uint2* ll, long long stride, int n,
                                              uint32_t epoch, unsigned max_polls, int* status,
                                              int tid) {
  constexpr int kBatch = 8;
  for (int k0 = tid; k0 < n; k0 += THREADS * kBatch) {
    uint2 v[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; b++) {
      const int k = k0 + b * THREADS;
      v[b] = k < n ? ld_packet(ll + (size_t)k * stride) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int b = 0; b < kBatch; b++) {
      const int k = k0 + b * THREADS;
      if (k < n) {
        const uint32_t val =
            v[b].y == epoch ? v[b].x : wait_packet(ll + (size_t)k * stride, epoch, max_polls, status);
        xs[k] = __ushort_as_half((unsigned short)val);
      }
    }
  }
}

// C = chunks (32 codes) per lane per row; D = rows in flight per lane; S warps
// share a row (ST > 0: compile time, ST == 0: run time), G groups per CTA;
// ALIGNED: every row
// starts on an absmax block boundary and blocks are a power of two, so the
// absmax pointer of a lane advances by a constant.  Nothing is divided on the
// device in the ALIGNED kernels.
//
// FUSE: RMSNorm of the input vector before the product and / or a gated
// activation of row pairs after it (rmsnorm-cuda/reference.h:4-25,
// geglu-cuda/reference.h:8-16), see GemvParams; plain fp16 input and output only.
// LL: packet input and / or packet output (hq_nf4_gemv_f16_ll); the plain
// instantiations carry none of that code.
template <int C, int D, int ST, bool ALIGNED, int THREADS, bool FUSE, bool LL>
__global__ void __launch_bounds__(THREADS, 1)
nf4_gemv_kernel(const GemvParams p) {
  constexpr int W = THREADS / 32;
  static_assert(D % 2 == 0, "a value row and its gate row sit in adjacent stages");
  __shared__ float s_sq[W];  // FUSE: sum of squares of each warp's inputs
  extern __shared__ __align__(16) unsigned char dsm_raw[];
  // [pad up to shared address kLutImm] table rows (256 x 256 B) |
  // partial sums [2][W * D][32] float
  // Programmatic dependent launch: let the next kernel of the stream start its
  // own prologue as soon as this grid is resident, and do not touch global
  // memory that earlier work may still be writing before the wait below.
  HQ_STAMP(0)
  pdl_launch_dependents();
  if (!p.early_fetch) pdl_wait();
  unsigned char* dsm = dsm_raw + (kLutImm - smem_u32(dsm_raw));
  const int S = ST > 0 ? ST : p.S;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = warp / S, q = warp - g * S;
  const int G = p.G;

  // rows of this group: n = blockIdx.x + gridDim.x * (g + G * j), j < my_rows
  // (paired: the same walk over pairs; matrix rows 2n and 2n + 1 of each)
  const bool paired = FUSE && p.act != 0;
  const int unit_first = blockIdx.x + gridDim.x * g;
  const int row_stride = gridDim.x * G;
  const int my_units = g < G ? p.rows_base + (unit_first < p.rows_rem ? 1 : 0) : 0;
  const int row_first = paired ? 2 * unit_first : unit_first;
  const int my_rows = paired ? 2 * my_units : my_units;

  // The 16 levels first: the table build must not queue behind the weight loads
  // below.  (The levels count as weights: read before the wait with early_fetch.)
  // (ordered loads: the compiler must not sink them below the weight loads)
  constexpr int kTabTurns = (256 * 4 + THREADS - 1) / THREADS;
  float lv_first[kTabTurns], lv_second[kTabTurns];
#pragma unroll
  for (int t = 0; t < kTabTurns; t++) {
    const int entry = ((tid + t * THREADS) >> 2) & 255;
    const int hi = entry >> 4, lo = entry & 15;
    lv_first[t] = ldg_ordered_f32(p.lut16 + (p.low_first ? lo : hi));
    lv_second[t] = ldg_ordered_f32(p.lut16 + (p.low_first ? hi : lo));
  }
  // this lane's chunk columns; a lane beyond the row end loads nothing and
  // keeps zero codes, scales and inputs
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
  }
  uint4 cw[D][C];
  float cs[D][C];

  // request row (loaded rows so far) into stage STAGE
#define HQ_NF4_LOAD(STAGE)                                                                      \
  {                                                                                             \
    _Pragma("unroll") for (int i = 0; i < C; i++) {                                             \
      const float* a = ap[i];                                                                   \
      if (!ALIGNED)                                                                             \
        a = p.absmax + (p.cpb_shift >= 0 ? (ci[i] >> p.cpb_shift) : (ci[i] / (uint32_t)p.cpb)); \
      if (live[i] && HQ_IN_BOUNDS(wp[i], 16, p.B, p.b_bytes, 101) &&                            \
          HQ_IN_BOUNDS(a, 4, p.absmax, p.absmax_bytes, 102)) {                                  \
        cw[STAGE][i] = ldg_stream_u4(wp[i]);                                                    \
        cs[STAGE][i] = __ldg(a);                                                                \
      }                                                                                         \
      const bool odd = FUSE && (((STAGE) & 1) != 0);                                            \
      wp[i] += odd ? p.w_step_odd : p.w_step;                                                   \
      if (ALIGNED) ap[i] += odd ? p.a_step_odd : p.a_step;                                      \
      else ci[i] += (uint32_t)(!paired ? row_stride : (odd ? 2 * row_stride - 1 : 1)) *         \
                    (uint32_t)p.nchunks;                                                        \
    }                                                                                           \
  }
  // Order of the prologue.  With early_fetch: the first kEarly rows of weights,
  // then the wait for the preceding kernel, then the INPUT VECTOR, then the other
  // rows, then the table.  The vector is requested before the bulk of the weights
  // on purpose: behind D rows per lane (9.5 MB over the whole GPU) its 8 KB took
  // 1.5 us to come back, and nothing can be computed without it.
  constexpr int kEarly = D / 2;
#pragma unroll
  for (int d = 0; d < D; d++) {
#pragma unroll
    for (int i = 0; i < C; i++) {
      cw[d][i] = make_uint4(0, 0, 0, 0);
      cs[d][i] = 0.f;
    }
    if (p.early_fetch && d < kEarly && d < my_rows) HQ_NF4_LOAD(d)
  }
  HQ_STAMP(1)
  // the input vector (and, without early_fetch, everything) is read only after
  // the preceding kernel has completed
  if (p.early_fetch) pdl_wait();
  HQ_STAMP(2)
  // epoch of the latest completed gather: the input packets carry it, the
  // output packets of this launch carry the next one
  const uint32_t epoch_in =
      LL && p.sync_words != nullptr ? *reinterpret_cast<volatile unsigned*>(p.sync_words + 1) : 0u;
  uint2* my_peer = nullptr;  // lane r stores the packets that go to rank r
  const bool packets_out = LL && p.peer_ll != nullptr, packets_in = LL && p.A_ll != nullptr;
  if (packets_out && lane < (p.multicast ? 1 : p.world)) my_peer = p.peer_ll[lane] + p.gather_offset;
  uint4 xr[C][4];
  if (!packets_in) {
#pragma unroll
    for (int i = 0; i < C; i++) {
      const int c = (q * C + i) * 32 + lane;
      const uint4* xp = reinterpret_cast<const uint4*>(p.A) + 4 * (live[i] ? c : 0);
#pragma unroll
      for (int t = 0; t < 4; t++) {
        if (live[i] && HQ_IN_BOUNDS(xp + t, 16, p.A, p.a_bytes, 103)) xr[i][t] = ld_dependent_u4(xp + t);
        else xr[i][t] = make_uint4(0, 0, 0, 0);
      }
    }
  }
  // FUSE: gamma goes to shared memory by asynchronous copies (no registers are
  // held for it while the weights are requested)
  __half* const gs = reinterpret_cast<__half*>(dsm + kLutBytes + (size_t)2 * W * D * 32 * sizeof(float));
  if (FUSE && p.gamma != nullptr) {
    for (int i = tid; i < p.nchunks * 4; i += THREADS)
      if (HQ_IN_BOUNDS(reinterpret_cast<const uint4*>(p.gamma) + i, 16, p.gamma, p.a_bytes, 105))
        cp_async_16(reinterpret_cast<uint4*>(gs) + i, reinterpret_cast<const uint4*>(p.gamma) + i);
    cp_async_commit();
  }
#pragma unroll
  for (int d = 0; d < D; d++)
    if (!(p.early_fetch && d < kEarly) && d < my_rows) HQ_NF4_LOAD(d)
  // ---- byte table ----
#pragma unroll
  for (int t = 0; t < kTabTurns; t++) {
    const int e4 = tid + t * THREADS;
    if (e4 < 256 * 4) {
      const int entry = e4 >> 2, quarter = e4 & 3;  // four threads per 128-byte table row
      const uint32_t u = half2_as_u32(__floats2half2_rn(lv_first[t], lv_second[t]));
      const uint4 u4 = make_uint4(u, u, u, u);
      uint4* row = reinterpret_cast<uint4*>(dsm + (size_t)entry * 256 + quarter * 32);
      row[entry & 1] = u4;
      row[(entry & 1) ^ 1] = u4;
    }
  }
  HQ_STAMP(3)
  if (packets_in) {
    // the whole input arrives as packets: every thread waits for its share and
    // leaves plain fp16 in shared memory
    __half* xs = reinterpret_cast<__half*>(dsm + kLutBytes + (size_t)2 * W * D * 32 * sizeof(float));
    stage_packets<THREADS>(xs, p.A_ll, p.a_stride, p.nchunks * 32, epoch_in, p.max_polls, p.status,
                           tid);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < C; i++) {
      const int c = (q * C + i) * 32 + lane;
      const uint4* xp = reinterpret_cast<const uint4*>(xs) + 4 * (live[i] ? c : 0);
#pragma unroll
      for (int t = 0; t < 4; t++) xr[i][t] = live[i] ? xp[t] : make_uint4(0, 0, 0, 0);
    }
  }
  if (FUSE && p.gamma != nullptr) {
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < C; i++)
#pragma unroll
      for (int t = 0; t < 4; t++) {
        const uint32_t h[4] = {xr[i][t].x, xr[i][t].y, xr[i][t].z, xr[i][t].w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const float2 f = __half22float2(u32_as_half2(h[k]));
          sq = fmaf(f.x, f.x, fmaf(f.y, f.y, sq));
        }
      }
    sq = warp_sum(sq);
    if (lane == 0) s_sq[warp] = sq;
    cp_async_wait_all();
  }
  __syncthreads();
  if (FUSE && p.gamma != nullptr) {
    // the S warps of a group hold the whole vector between them
    float tot = 0.f;
    for (int t = 0; t < S; t++) tot += s_sq[g * S + t];
    const float norm = rsqrtf(tot / (float)(p.nchunks * 32) + p.eps);
#pragma unroll
    for (int i = 0; i < C; i++) {
      const int c = (q * C + i) * 32 + lane;
      const uint4* gp = reinterpret_cast<const uint4*>(gs) + 4 * (live[i] ? c : 0);
#pragma unroll
      for (int t = 0; t < 4; t++) {
        const uint4 gv = gp[t];
        uint32_t h[4] = {xr[i][t].x, xr[i][t].y, xr[i][t].z, xr[i][t].w};
        const uint32_t gh[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const float2 f = __half22float2(u32_as_half2(h[k]));
          const float2 w = __half22float2(u32_as_half2(gh[k]));
          h[k] = half2_as_u32(__floats2half2_rn(f.x * norm * w.x, f.y * norm * w.y));
        }
        if (live[i]) xr[i][t] = make_uint4(h[0], h[1], h[2], h[3]);
      }
    }
  }

  HQ_STAMP(4)
  const uint32_t lane4 = lane * 4;
  // row j of this group is output element n_out + j * row_stride: stored as fp16
  // (lane 0) or as one packet per GPU of the node (lane r -> rank r)
  long long n_out = unit_first;
  float held = 0.f;  // paired, one warp per row: the value row's sum until its gate row is done
  auto store_result = [&](long long n, float v) {
    const __half h = __float2half_rn(v);
    if (!packets_out) {
      if (lane == 0 && HQ_IN_BOUNDS(p.out + n, 2, p.out, p.out_bytes, 104)) p.out[n] = h;
    } else if (my_peer != nullptr) {
      if (p.multicast) st_packet_multicast(my_peer + n, (uint32_t)__half_as_ushort(h), epoch_in + 1u);
      else st_packet(my_peer + n, (uint32_t)__half_as_ushort(h), epoch_in + 1u);
    }
  };
  // results of rows 2 m and 2 m + 1 (kPairPackets), or value and gate of output m
  auto store_pair = [&](long long m, float v0, float v1) {
    if (p.act != kPairPackets) {
      store_result(m, v0 * gate_act(v1, p.act));
      return;
    }
    const uint32_t h0 = __half_as_ushort(__float2half_rn(v0)), h1 = __half_as_ushort(__float2half_rn(v1));
    if (!packets_out) {
      if (lane == 0 && HQ_IN_BOUNDS(p.out + 2 * m, 4, p.out, p.out_bytes, 106))
        *reinterpret_cast<uint32_t*>(p.out + 2 * m) = h0 | (h1 << 16);
    } else if (my_peer != nullptr) {
      uint2* at = my_peer + 2 * m;
      if (p.multicast) {
        st_packet_multicast(at, h0, epoch_in + 1u);
        st_packet_multicast(at + 1, h1, epoch_in + 1u);
      } else if ((reinterpret_cast<uintptr_t>(at) & 15u) == 0) {
        // each 8-byte half carries its own epoch: the halves may land in any order
        asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(at), "r"(h0),
                     "r"(epoch_in + 1u), "r"(h1), "r"(epoch_in + 1u)
                     : "memory");
      } else {
        st_packet(at, h0, epoch_in + 1u);
        st_packet(at + 1, h1, epoch_in + 1u);
      }
    }
  };
  // partial sums: [parity][g][d][t][lane]
  float* const part = reinterpret_cast<float*>(dsm + kLutBytes) + (g * S * D) * 32 + lane;
  int parity = 0;

  for (int j0 = 0; j0 < my_rows; j0 += D) {
    const int rows_in_round = min(D, my_rows - j0);
    float* const part_r = part + (parity ? W * D * 32 : 0);
#pragma unroll
    for (int d = 0; d < D; d++) {
      if (d < rows_in_round) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < C; i++) acc = fmaf(chunk_dot(cw[d][i], xr[i], lane4), cs[d][i], acc);
        if (j0 + d + D < my_rows) HQ_NF4_LOAD(d)
        if (S > 1) {
          part_r[(d * S + q) * 32] = acc;
        } else if (paired) {
          const float total = warp_sum(acc);
          if (d & 1) {
            store_pair(n_out, held, total);
            n_out += row_stride;
          } else {
            held = total;
          }
        } else {
          store_result(n_out, warp_sum(acc));
          n_out += row_stride;
        }
      }
    }
    if (S > 1 && paired) {
      group_barrier(1 + g, S * 32);
      for (int pr = q; 2 * pr < rows_in_round; pr += S) {
        float v = 0.f, gt = 0.f;
        for (int t = 0; t < S; t++) {
          v += part_r[(2 * pr * S + t) * 32];
          gt += part_r[((2 * pr + 1) * S + t) * 32];
        }
        store_pair(n_out + (long long)pr * row_stride, warp_sum(v), warp_sum(gt));
      }
      n_out += (long long)(D / 2) * row_stride;
      parity ^= 1;
    } else if (S > 1) {
      group_barrier(1 + g, S * 32);
      for (int d = q; d < rows_in_round; d += S) {
        float v = 0.f;
        if (ST > 0) {
#pragma unroll
          for (int t = 0; t < (ST > 0 ? ST : 1); t++) v += part_r[(d * S + t) * 32];
        } else {
          for (int t = 0; t < S; t++) v += part_r[(d * S + t) * 32];
        }
        store_result(n_out + (long long)d * row_stride, warp_sum(v));
      }
      n_out += (long long)D * row_stride;
      parity ^= 1;
    }
    HQ_STAMP(5 + min(j0 / D, 9))
  }
  HQ_STAMP(15)
#undef HQ_NF4_LOAD
  if (packets_out) {
    // the last CTA to finish records that this gather round is complete on the
    // sending side (the packets validate themselves on the receiving side)
    __syncthreads();
    if (tid == 0) {
      const unsigned prev = atomicAdd(p.sync_words, 1u);
      if (prev == gridDim.x - 1) {
        p.sync_words[0] = 0u;
        *reinterpret_cast<volatile unsigned*>(p.sync_words + 1) = epoch_in + 1u;
      }
    }
  }
}

// ---- bulk-copy form (rows of up to 4096 inputs) -------------------------------
// A CTA owns a CONTIGUOUS range of rows and moves it through shared memory in
// chunks of 16 rows (one row per compute warp): one bulk copy (cp.async.bulk,
// global -> shared, completing on the chunk's mbarrier) for the chunk's packed
// codes and one for its absmax run, into one of four chunk slots.  A seventeenth
// warp does nothing but issue these copies.  It keeps at most kCopiesInFlight
// chunks outstanding and issues the next one when the oldest has LANDED (not
// when a slot has been consumed): requested all at once, the copies of a CTA
// are served side by side and the first chunk arrives with the last; paced by
// arrival they land in order at the full rate, and by the time the input vector
// is there most of the CTA's share of an 11008 x 4096 layer sits in shared
// memory.  No load instruction, address update or register is spent on weights
// in the compute warps.  One warp owns a whole row (C = K / 1024 chunks per
// lane), so a row ends with a shuffle tree and one store: no partial sums, no
// barrier between warps.  A slot is refilled once all 16 compute warps have
// released it.  Every mbarrier wait is bounded.
constexpr int kTmaWarps = 16;                      // compute warps = rows per chunk
constexpr int kTmaCompute = kTmaWarps * 32;        // compute threads
constexpr int kTmaThreads = kTmaCompute + 32;      // + the copy warp
constexpr int kChunkSlots = 4;
constexpr int kCopiesInFlight = 2;
constexpr uint32_t kMbarSpins = 1u << 22;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait for the phase with the given parity; false when the limit was hit
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
// bulk copy global -> this CTA's shared memory; bytes a multiple of 16, both
// addresses 16-byte aligned; completes on the mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// C = chunks (32 codes) per lane = K / 1024.
template <int C>
__global__ void __launch_bounds__(kTmaThreads, 1)
nf4_gemv_bulk_kernel(const GemvParams p, int rows_total) {
  extern __shared__ __align__(16) unsigned char dsm_raw[];
  // [pad up to shared address kLutImm] table rows (256 x 256 B) |
  // chunk slots [kChunkSlots][16 rows of codes | 16 absmax runs] |
  // mbarriers full[kChunkSlots], empty[kChunkSlots] | unpacked input (packet input only)
  HQ_STAMP(0)
  pdl_launch_dependents();
  if (!p.early_fetch) pdl_wait();
  unsigned char* dsm = dsm_raw + (kLutImm - smem_u32(dsm_raw));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t row_bytes = (uint32_t)p.nchunks * 16u;
  const uint32_t am_bytes = ((uint32_t)p.nchunks >> p.cpb_shift) * 4u;
  const uint32_t slot_bytes = (row_bytes + am_bytes) * kTmaWarps;
  const uint32_t slots0 = smem_u32(dsm) + kLutBytes;
  const uint32_t full0 = slots0 + kChunkSlots * slot_bytes;
  const uint32_t empty0 = full0 + 8 * kChunkSlots;

  // rows of this CTA: a contiguous, balanced range
  const long long r0 = ((long long)rows_total * blockIdx.x) / gridDim.x;
  const long long r1 = ((long long)rows_total * (blockIdx.x + 1)) / gridDim.x;
  const int nrows = (int)(r1 - r0);
  const int nchunk = (nrows + kTmaWarps - 1) / kTmaWarps;
  // chunk c (rows r0 + 16c ..) into slot c % kChunkSlots; issued by one thread
  auto request = [&](int c) {
    const long long n = r0 + (long long)c * kTmaWarps;
    const uint32_t rows = (uint32_t)min((long long)kTmaWarps, r1 - n);
    const int s = c % kChunkSlots;
    const uint32_t dst = slots0 + (uint32_t)s * slot_bytes, bar = full0 + 8u * s;
    const unsigned char* src = p.B + (size_t)n * row_bytes;
    const float* am = p.absmax + (((size_t)n * p.nchunks) >> p.cpb_shift);
    if (HQ_IN_BOUNDS(src, rows * row_bytes, p.B, p.b_bytes, 121) &&
        HQ_IN_BOUNDS(am, rows * am_bytes, p.absmax, p.absmax_bytes, 122)) {
      mbar_expect_tx(bar, rows * (row_bytes + am_bytes));
      bulk_load(dst, src, rows * row_bytes, bar);
      bulk_load(dst + kTmaWarps * row_bytes, am, rows * am_bytes, bar);
    } else {
      mbar_expect_tx(bar, 0);  // checked build: the chunk is skipped, the waiters still pass
    }
  };
  const bool copy_thread = tid == kTmaCompute;
  int issued = 0;
  if (copy_thread) {
    for (int s = 0; s < kChunkSlots; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kTmaWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (; issued < nchunk && issued < kCopiesInFlight; issued++) request(issued);
  }
  HQ_STAMP(1)
  __syncthreads();  // the barriers are initialised for everybody

  if (warp == kTmaWarps) {
    // ---- the copy warp: one thread paces the remaining chunks ----
    if (copy_thread) {
      bool ok = true;
      int landed = 0;
      while (ok && issued < nchunk) {
        // the oldest outstanding chunk has landed ...
        if (!mbar_wait(full0 + 8u * (landed % kChunkSlots), (uint32_t)(landed / kChunkSlots) & 1u)) {
          ok = false;
          break;
        }
        landed++;
        // ... and the slot of the next one is free (its previous chunk consumed)
        const int s = issued % kChunkSlots;
        if (issued >= kChunkSlots) {
          if (!mbar_wait(empty0 + 8u * s, (uint32_t)(issued / kChunkSlots - 1) & 1u)) {
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        request(issued);
        issued++;
      }
      if (!ok && p.status != nullptr) atomicExch(p.status, 1);
    }
  } else {
    // ---- byte table (overlaps the copies) ----
    constexpr int kTabTurns = (256 * 4 + kTmaCompute - 1) / kTmaCompute;
#pragma unroll
    for (int t = 0; t < kTabTurns; t++) {
      const int e4 = tid + t * kTmaCompute;
      if (e4 < 256 * 4) {
        const int entry = e4 >> 2, quarter = e4 & 3;  // four threads per 128-byte table row
        const int hi = entry >> 4, lo = entry & 15;
        const int first = p.low_first ? lo : hi, second = p.low_first ? hi : lo;
        const uint32_t u = half2_as_u32(__floats2half2_rn(p.lut16[first], p.lut16[second]));
        const uint4 u4 = make_uint4(u, u, u, u);
        uint4* row = reinterpret_cast<uint4*>(dsm + (size_t)entry * 256 + quarter * 32);
        row[entry & 1] = u4;
        row[(entry & 1) ^ 1] = u4;
      }
    }
    if (p.early_fetch && p.A != nullptr)
      for (int line = tid; line * 128 < p.nchunks * 64; line += kTmaCompute)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.A) + line * 128));
    HQ_STAMP(2)
    if (p.early_fetch) pdl_wait();
    HQ_STAMP(3)
    const uint32_t epoch_in =
        p.sync_words != nullptr ? *reinterpret_cast<volatile unsigned*>(p.sync_words + 1) : 0u;
    uint2* my_peer = nullptr;  // lane r stores the packets that go to rank r
    if (p.peer_ll != nullptr && lane < p.world) my_peer = p.peer_ll[lane] + p.gather_offset;
    const uint4* xsrc = reinterpret_cast<const uint4*>(p.A);
    if (p.A_ll != nullptr) {
      __half* xs = reinterpret_cast<__half*>(dsm + kLutBytes + (size_t)kChunkSlots * slot_bytes +
                                             (size_t)16 * kChunkSlots);
      stage_packets<kTmaCompute>(xs, p.A_ll, p.a_stride, p.nchunks * 32, epoch_in, p.max_polls,
                                 p.status, tid);
      group_barrier(1, kTmaCompute);
      xsrc = reinterpret_cast<const uint4*>(xs);
    }
    uint4 xr[C][4];
#pragma unroll
    for (int i = 0; i < C; i++) {
      const uint4* xp = xsrc + 4 * (i * 32 + lane);
#pragma unroll
      for (int t = 0; t < 4; t++) {
        if (p.A_ll != nullptr) xr[i][t] = xp[t];
        else if (HQ_IN_BOUNDS(xp + t, 16, p.A, p.a_bytes, 123)) xr[i][t] = ld_dependent_u4(xp + t);
        else xr[i][t] = make_uint4(0, 0, 0, 0);
      }
    }
    group_barrier(1, kTmaCompute);  // the table is complete
    HQ_STAMP(4)

    const uint32_t lane4 = lane * 4;
    bool ok = true;
    for (int c = 0; c < nchunk; c++) {
      const int s = c % kChunkSlots;
      const uint32_t use = (uint32_t)(c / kChunkSlots);
      const long long n = r0 + (long long)c * kTmaWarps + warp;
      if (ok && !mbar_wait(full0 + 8u * s, use & 1u)) ok = false;
      if (n < r1) {
        const uint32_t codes = slots0 + (uint32_t)s * slot_bytes + (uint32_t)warp * row_bytes;
        const uint32_t scales =
            slots0 + (uint32_t)s * slot_bytes + kTmaWarps * row_bytes + (uint32_t)warp * am_bytes;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < C; i++) {
          const int ch = i * 32 + lane;
          uint4 cw;
          float cs;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(cw.x), "=r"(cw.y), "=r"(cw.z), "=r"(cw.w)
                       : "r"(codes + (uint32_t)ch * 16u));
          asm volatile("ld.shared.f32 %0, [%1];"
                       : "=f"(cs)
                       : "r"(scales + ((uint32_t)ch >> p.cpb_shift) * 4u));
          acc = fmaf(chunk_dot(cw, xr[i], lane4), cs, acc);
        }
        acc = warp_sum(acc);  // every lane's sum has arrived: the warp has read its row
        const __half h = __float2half_rn(acc);
        if (p.peer_ll == nullptr) {
          if (lane == 0 && HQ_IN_BOUNDS(p.out + n, 2, p.out, p.out_bytes, 124)) p.out[n] = h;
        } else if (my_peer != nullptr) {
          st_packet(my_peer + n, (uint32_t)__half_as_ushort(h), epoch_in + 1u);
        }
      }
      // release the slot: the copy warp refills it once all 16 warps have released it
      if (c + kChunkSlots < nchunk && lane == 0) mbar_arrive(empty0 + 8u * s);
      HQ_STAMP(5 + min(c, 9))
    }
    if (!ok && p.status != nullptr && lane == 0) atomicExch(p.status, 1);
    HQ_STAMP(15)
    if (p.peer_ll != nullptr) {
      group_barrier(1, kTmaCompute);
      if (tid == 0) {
        const unsigned prev = atomicAdd(p.sync_words, 1u);
        if (prev == gridDim.x - 1) {
          p.sync_words[0] = 0u;
          *reinterpret_cast<volatile unsigned*>(p.sync_words + 1) = epoch_in + 1u;
        }
      }
    }
  }
}

// Plain fp16 copy of a packet vector: thread i waits (bounded) until packet i
// carries the epoch of the latest completed gather (sync_words[1]; no check
// when sync_words is null) and stores its value.
__global__ void __launch_bounds__(256)
ll_unpack_kernel(const uint2* __restrict__ ll, long long n, __half* __restrict__ out,
                 const unsigned* sync_words, unsigned max_polls, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const bool check = sync_words != nullptr;
  const uint32_t epoch = check ? *reinterpret_cast<const volatile unsigned*>(sync_words + 1) : 0u;
  // four packets per thread and turn, loaded before the first is examined
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n; i0 += 4 * step) {
    uint2 v[4];
#pragma unroll
    for (int b = 0; b < 4; b++) {
      const long long i = i0 + b * step;
      v[b] = i < n ? ld_packet(ll + i) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int b = 0; b < 4; b++) {
      const long long i = i0 + b * step;
      if (i < n) {
        const uint32_t val =
            (!check || v[b].y == epoch) ? v[b].x : wait_packet(ll + i, epoch, max_polls, status);
        out[i] = __ushort_as_half((unsigned short)val);
      }
    }
  }
}

// One thread and turn: 4 bytes of codes (8 elements) -> 16 bytes of fp16, two
// turns in flight per thread.  SHIFT >= 0: words per absmax block is a power of
// two (a shift instead of a division); the output is written with streaming
// stores (it is 3.5x the size of everything that is read and not read again
// here).
__device__ __forceinline__ void st_stream_u4(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
template <bool POW2>
__global__ void __launch_bounds__(kThreads)
nf4_dequant_kernel(const uint8_t* __restrict__ B, const float* __restrict__ absmax,
                   const float* __restrict__ lut16, __half* __restrict__ out, size_t nwords,
                   int words_per_block, int shift, int low_first) {
  __shared__ float lut[16 * 32];  // [code][lane]
  const int tid = threadIdx.x, lane = tid & 31;
  for (int i = tid; i < 16 * 32; i += kThreads) lut[i] = lut16[i >> 5];
  __syncthreads();
  const float* lut_lane = lut + lane;
  const size_t stride = (size_t)gridDim.x * kThreads;
  auto block_of = [&](size_t w) -> size_t {
    if (POW2) return w >> shift;
    return nwords <= 0xffffffffull ? (size_t)((uint32_t)w / (uint32_t)words_per_block)
                                   : w / (size_t)words_per_block;
  };
  auto convert = [&](uint32_t codes, float s) {
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
    return make_uint4(o[0], o[1], o[2], o[3]);
  };
  const size_t nblocks = (nwords + words_per_block - 1) / words_per_block;
  (void)nblocks;
  for (size_t w = (size_t)blockIdx.x * kThreads + tid; w < nwords; w += 2 * stride) {
    const size_t w2 = w + stride;
    const bool two = w2 < nwords;
    if (!HQ_IN_BOUNDS(reinterpret_cast<const uint32_t*>(B) + w, 4, B, nwords * 4, 111) ||
        !HQ_IN_BOUNDS(absmax + block_of(w), 4, absmax, nblocks * 4, 112) ||
        !HQ_IN_BOUNDS(reinterpret_cast<uint4*>(out) + w, 16, out, nwords * 16, 113))
      continue;
    const uint32_t c0 = ldg_stream_u32(reinterpret_cast<const uint32_t*>(B) + w);
    const uint32_t c1 = two ? ldg_stream_u32(reinterpret_cast<const uint32_t*>(B) + w2) : 0u;
    const float s0 = __ldg(absmax + block_of(w));
    const float s1 = two ? __ldg(absmax + block_of(w2)) : 0.f;
    st_stream_u4(reinterpret_cast<uint4*>(out) + w, convert(c0, s0));
    if (two) st_stream_u4(reinterpret_cast<uint4*>(out) + w2, convert(c1, s1));
  }
}

// One warp: lane r waits (bounded) until rank r's flag has reached this rank's
// own launch count, i.e. until rank r's slice of the latest gather has landed.
__global__ void gather_wait_kernel(const uint32_t* flags, const unsigned* sync_words, int world,
                                   unsigned max_polls, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const unsigned want = sync_words[1];
  const volatile uint32_t* f = flags + r;
  bool ok = false;
  for (unsigned spin = 0; spin < max_polls; spin++) {
    // flags only grow; "reached" is tested modulo 2^32
    if ((int)(*f - want) >= 0) { ok = true; break; }
    __nanosleep(64);
  }
  if (ok) __threadfence_system();
  else if (status != nullptr) atomicExch(status, 1);
}

// Copies this rank's finished slice (already in its own gathered vector) into
// every peer's vector with 16-byte stores over NVLink, the (peer, piece) pairs
// spread over the CTAs of the grid; the CTA that finishes last raises this
// rank's flag on every GPU, waits (bounded) until every rank's flag on THIS GPU
// has reached the same launch count and advances the launch count.  With an
// empty slice (the producing kernel stored to the peers itself) only the
// signalling remains.
constexpr int kPublishThreads = 1024;
constexpr int kPublishPiece = kPublishThreads * 16;  // bytes one CTA moves per sweep
__global__ void __launch_bounds__(kPublishThreads, 1)
gather_publish_kernel(__half* const* peer_out, long long offset, int n_slice,
                      uint32_t* const* peer_flags, unsigned* sync_words, int world, int rank,
                      unsigned max_polls, int* status) {
  __shared__ unsigned s_last;
  const int tid = threadIdx.x;
  // Programmatic dependent launch: these CTAs may become resident while the kernel
  // that produces the slice is still draining, and the next kernel of the stream
  // may start its own prologue while they wait for the other ranks; the slice is
  // read only after the producing kernel has completed.
  pdl_launch_dependents();
  pdl_wait();
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(sync_words + 1) + 1u;
  // work items = (peer, 16 KB piece of the slice), dealt round-robin to the CTAs;
  // consecutive items go to different peers so that all links carry data at once
  const long long bytes = (long long)n_slice * 2;
  const int pieces = (int)((bytes + kPublishPiece - 1) / kPublishPiece);
  const int peers = world - 1;
  const bool vec_ok = ((offset | (long long)n_slice) & 7) == 0;
  const __half* mine = peer_out[rank] + offset;
  for (int item = blockIdx.x; item < pieces * peers; item += gridDim.x) {
    const int piece = item / peers, pr = item - piece * peers;
    const int r = pr + (pr >= rank ? 1 : 0);
    __half* dst = peer_out[r] + offset;
    if (vec_ok) {
      const int i = piece * kPublishThreads + tid;
      if (i < n_slice / 8)
        reinterpret_cast<uint4*>(dst)[i] = __ldcg(reinterpret_cast<const uint4*>(mine) + i);
    } else {
      const int i0 = piece * (kPublishPiece / 2);
      for (int i = i0 + tid; i < min(i0 + kPublishPiece / 2, n_slice); i += kPublishThreads)
        reinterpret_cast<unsigned short*>(dst)[i] =
            __ldcg(reinterpret_cast<const unsigned short*>(mine) + i);
    }
  }
  // every CTA makes its own stores visible system-wide before it is counted; the
  // CTA that is counted last raises the flags, so a flag is ordered after the
  // stores of ALL CTAs (fence - atomic - fence)
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(sync_words, 1u);
    s_last = prev == gridDim.x - 1u ? 1u : 0u;
  }
  __syncthreads();
  if (s_last == 0u) return;
  __threadfence_system();
  bool landed = true;
  if (tid < world) {
    // thread r: this rank's flag on GPU r, then rank r's flag here
    *reinterpret_cast<volatile uint32_t*>(peer_flags[tid] + rank) = epoch;
    const volatile uint32_t* f = peer_flags[rank] + tid;
    landed = false;
    for (unsigned spin = 0; spin < max_polls; spin++) {
      if ((int)(*f - epoch) >= 0) { landed = true; break; }
      __nanosleep(32);
    }
    if (landed) __threadfence_system();
    else if (status != nullptr) atomicExch(status, 1);
  }
  __syncthreads();
  if (tid == 0) {
    sync_words[0] = 0u;
    *reinterpret_cast<volatile unsigned*>(sync_words + 1) = epoch;
  }
}

// Small slices (a mat-vec's output): one CTA per rank r of the node copies the
// whole slice to GPU r, makes it visible, raises this rank's flag there and
// waits for rank r's flag here - no counter between the copy and the flag, which
// is what the latency of a 20 KB gather is made of.  The last CTA to finish
// advances the launch count.
__global__ void __launch_bounds__(kPublishThreads, 1)
gather_publish_small_kernel(__half* const* peer_out, long long offset, int n_slice,
                            uint32_t* const* peer_flags, unsigned* sync_words, int world,
                            int rank, unsigned max_polls, int* status) {
  const int tid = threadIdx.x;
  const int r = blockIdx.x;
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
    for (unsigned spin = 0; spin < max_polls; spin++) {
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

namespace hq {
namespace {

// N: rows of the matrix, or (FUSE with a gated activation) pairs of rows
template <int C, int D, int ST, bool AL, int THREADS, bool FUSE, bool LL>
int launch_gemv(GemvParams& prm, int N, cudaStream_t st) {
  constexpr int W = THREADS / 32;
  const int S = prm.S;
  int G = W / S;
  if (S > 1 && G > 15) G = 15;  // named barriers 1..15
  const int grid = std::min(sm_count(), (N + G - 1) / G);
  prm.G = G;
  prm.rows_base = N / (grid * G);
  prm.rows_rem = N % (grid * G);
  // rows from one row of a group to its next one, even and odd stages
  unsigned long long step = (unsigned long long)grid * G, step_odd = step;
  if (FUSE && prm.act != 0) {
    step = 1;
    step_odd = 2ull * grid * G - 1;
  }
  prm.w_step = step * prm.nchunks * 16ull;
  prm.w_step_odd = step_odd * prm.nchunks * 16ull;
  prm.a_step = AL ? (unsigned)((step * prm.nchunks) >> prm.cpb_shift) : 0u;
  prm.a_step_odd = AL ? (unsigned)((step_odd * prm.nchunks) >> prm.cpb_shift) : 0u;
  // room for the pad that brings the table to shared address kLutImm wherever the
  // dynamic region starts (at or below kLutImm)
  size_t smem = (size_t)kLutImm + kLutBytes + (size_t)2 * W * D * 32 * sizeof(float);
  // unpacked input (packets) or gamma (FUSE)
  if (prm.A_ll != nullptr || (FUSE && prm.gamma != nullptr))
    smem += (size_t)prm.nchunks * 32 * sizeof(__half);
  if (smem > 227 * 1024) return HQ_ERR_TOO_LARGE;
  constexpr auto kern = nf4_gemv_kernel<C, D, ST, AL, THREADS, FUSE, LL>;
  cudaError_t e = ensure_dynamic_smem<kern>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  return cuda_status(launch_pdl(kern, dim3(grid), dim3(THREADS), smem, st, prm));
}

}  // namespace
}  // namespace hq

// What the low-latency gather adds to a GEMV call (all null / zero without it).
struct LlArgs {
  const void* A_ll = nullptr;
  long long a_stride = 1;
  void* const* peer_ll = nullptr;
  long long gather_offset = 0;
  unsigned* sync_words = nullptr;
  int world = 1, rank = 0;
  unsigned max_polls = 0;
  int* status = nullptr;
};

namespace hq {
namespace {
template <int C>
int launch_gemv_bulk(GemvParams& prm, int N, cudaStream_t st) {
  const uint32_t slot_bytes =
      ((uint32_t)prm.nchunks * 16u + ((uint32_t)prm.nchunks >> prm.cpb_shift) * 4u) * kTmaWarps;
  const size_t smem = (size_t)kLutImm + kLutBytes + (size_t)kChunkSlots * slot_bytes +
                      (size_t)16 * kChunkSlots +
                      (prm.A_ll != nullptr ? (size_t)prm.nchunks * 32 * sizeof(__half) : 0);
  if (smem > 227 * 1024) return HQ_ERR_UNSUPPORTED;
  const int grid = std::min(sm_count(), (N + kTmaWarps - 1) / kTmaWarps);
  constexpr auto kern = nf4_gemv_bulk_kernel<C>;
  cudaError_t e = ensure_dynamic_smem<kern>(smem);
  if (e != cudaSuccess) return cuda_status(e);
  return cuda_status(launch_pdl(kern, dim3(grid), dim3(kTmaThreads), smem, st, prm, N));
}
}  // namespace
}  // namespace hq

// What the fused forms add (see GemvParams): N stays the number of matrix rows.
struct FuseArgs {
  const void* gamma = nullptr;
  float eps = 0.f;
  int act = HQ_ACT_NONE;
};

static int nf4_gemv_impl(const void* A_half, const uint8_t* B, const float* absmax,
                         const float* lut16, void* out_half, int N, int K, int blocksize, int flags,
                         const LlArgs& ll, hq_stream_t stream, const FuseArgs* fuse = nullptr) {
  using namespace hq;
  if ((!A_half && !ll.A_ll) || !B || !absmax || !lut16 || (!out_half && !ll.peer_ll))
    return HQ_ERR_NULL_POINTER;
  if (N <= 0 || K <= 0 || K % 32 != 0 || blocksize <= 0 || blocksize % 32 != 0)
    return HQ_ERR_BAD_SHAPE;
  if (!aligned16(B) || (A_half && !aligned16(A_half)) || (ll.A_ll && !aligned8(ll.A_ll)))
    return HQ_ERR_MISALIGNED;
  if ((uint64_t)N * (uint64_t)(K / 32) > 0xffffffffull) return HQ_ERR_TOO_LARGE;
  // the kernels address their table at a fixed shared-memory address, which the
  // system-reserved part of the window (1 KiB on sm_100) must not overlap
  if (reserved_smem_per_block() > kLutImm) return HQ_ERR_UNSUPPORTED;
  const int nchunks = K / 32;
  const int cols = (nchunks + 31) / 32;  // 1024-input slices per row
  if (cols > 64) return HQ_ERR_TOO_LARGE;  // K > 65536
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
  prm.cpb_shift = shift;
  prm.cpb = cpb;
  prm.low_first = (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0;
  prm.peer_ll = reinterpret_cast<uint2* const*>(ll.peer_ll);
  prm.A_ll = reinterpret_cast<const uint2*>(ll.A_ll);
  prm.a_stride = ll.a_stride;
  prm.sync_words = ll.sync_words;
  prm.world = ll.world;
  prm.multicast = (ll.peer_ll != nullptr && (flags & HQ_NF4_LL_MULTICAST)) ? 1 : 0;
  prm.rank = ll.rank;
  prm.gather_offset = ll.gather_offset;
  prm.max_polls = ll.max_polls ? ll.max_polls : kDefaultPolls;
  prm.status = ll.status;
  prm.early_fetch = (flags & HQ_NF4_WEIGHTS_RESIDENT) ? 1 : 0;
  prm.b_bytes = (unsigned long long)N * (K / 2);
  prm.absmax_bytes = ((unsigned long long)N * K + blocksize - 1) / blocksize * 4ull;
  prm.a_bytes = (unsigned long long)K * 2;
  prm.out_bytes = (unsigned long long)N * 2;
  prm.gamma = nullptr;
  prm.eps = 0.f;
  prm.act = HQ_ACT_NONE;
  int units = N;  // what a group of warps walks: rows, or value / gate pairs
  if (fuse != nullptr) {
    if (fuse->act != HQ_ACT_NONE && fuse->act != HQ_ACT_SWIGLU && fuse->act != HQ_ACT_GEGLU)
      return HQ_ERR_BAD_SHAPE;
    if (fuse->gamma && !aligned16(fuse->gamma)) return HQ_ERR_MISALIGNED;
    if (fuse->act != HQ_ACT_NONE) {
      if (N % 2 != 0) return HQ_ERR_BAD_SHAPE;
      units = N / 2;
      prm.out_bytes = (unsigned long long)units * 2;
    }
    prm.gamma = reinterpret_cast<const __half*>(fuse->gamma);
    prm.eps = fuse->eps;
    prm.act = fuse->act;
  }
  // Packet output, opt-in (environment HQ_LL_PAIRS=1): walk the rows in adjacent
  // pairs and send both results in one 16-byte store per GPU - half as many
  // stores over NVLink.  On 2 GPUs it measured 12.0 us per layer against 10.2 us
  // with one 8-byte store per row, so it is off by default.
  bool pair_packets = false;
  if (fuse == nullptr && ll.peer_ll != nullptr && N % 2 == 0 && ll.gather_offset % 2 == 0 &&
      env_flag("HQ_LL_PAIRS")) {
    pair_packets = true;
    prm.act = kPairPackets;
    units = N / 2;
  }
#ifdef HQ_NF4_TRACE
  {
    const char* tp = getenv("HQ_NF4_TRACE_PTR");
    prm.trace = tp ? reinterpret_cast<unsigned long long*>(strtoull(tp, nullptr, 0)) : nullptr;
  }
#endif
  cudaStream_t st = (cudaStream_t)stream;
  // The bulk-copy form is opt-in (environment HQ_NF4_BULK=1): on B200 it measured
  // 10.1 us against 7.8 us for the register pipeline on an 11008 x 4096 layer.
  // It takes rows of 1024 .. 4096 inputs whose codes and absmax runs start on
  // 16-byte boundaries (one warp per row).
  if (fuse == nullptr && !prm.multicast && env_flag("HQ_NF4_BULK") && aligned && nchunks % 32 == 0 && cols <= 4 && aligned16(absmax) &&
      ((nchunks >> shift) * 4) % 16 == 0) {
    int rc;
    switch (cols) {
      case 1: rc = launch_gemv_bulk<1>(prm, N, st); break;
      case 2: rc = launch_gemv_bulk<2>(prm, N, st); break;
      case 3: rc = launch_gemv_bulk<3>(prm, N, st); break;
      default: rc = launch_gemv_bulk<4>(prm, N, st); break;
    }
    if (rc != HQ_ERR_UNSUPPORTED) return rc;
  }
  // Chunks per lane C and warps per row S = cols / C.  512 threads with up to
  // 128 registers each hold C = 2 chunks of the input vector and D = 4 rows of
  // packed weights in flight per lane.
  const bool with_packets = ll.A_ll != nullptr || ll.peer_ll != nullptr;
#define HQ_NF4_GO(C_, D_, ST_, AL_)                                                         \
  (with_packets                                                                              \
       ? (pair_packets ? launch_gemv<C_, D_, ST_, AL_, 512, true, true>(prm, units, st)      \
                       : launch_gemv<C_, D_, ST_, AL_, 512, false, true>(prm, units, st))    \
       : (fuse != nullptr ? launch_gemv<C_, D_, ST_, AL_, 512, true, false>(prm, units, st)  \
                          : launch_gemv<C_, D_, ST_, AL_, 512, false, false>(prm, units, st)))
  if (aligned && cols == 4) { prm.S = 2; return HQ_NF4_GO(2, 4, 2, true); }
  int C = cols <= 1 ? 1 : (cols <= 32 ? 2 : 4);
  prm.S = (cols + C - 1) / C;
  if (C == 1) return aligned ? HQ_NF4_GO(1, 4, 1, true) : HQ_NF4_GO(1, 4, 1, false);
  if (C == 2) return aligned ? HQ_NF4_GO(2, 4, 0, true) : HQ_NF4_GO(2, 4, 0, false);
  return aligned ? HQ_NF4_GO(4, 2, 0, true) : HQ_NF4_GO(4, 2, 0, false);
#undef HQ_NF4_GO
}

extern "C" {

int hq_gather_publish(void* const* peer_out_half, long long offset, int n_slice,
                      uint32_t* const* peer_flags, unsigned* sync_words, int world, int rank,
                      unsigned max_polls, int* status, hq_stream_t stream) {
  using namespace hq;
  if (!peer_out_half || !peer_flags || !sync_words) return HQ_ERR_NULL_POINTER;
  if (world < 1 || world > 32 || rank < 0 || rank >= world || n_slice < 0) return HQ_ERR_BAD_SHAPE;
  // n_slice == 0: the producing kernel has stored the slice to the peers itself,
  // only signal and wait.  Larger slices: one CTA per (peer, 16 KB piece) up to the
  // number of SMs.
  const long long pieces = ((long long)n_slice * 2 + kPublishPiece - 1) / kPublishPiece;
  if (pieces <= 4)  // up to 64 KB per peer: one CTA per peer, flag straight after the copy
    return cuda_status(launch_pdl(gather_publish_small_kernel, dim3(world), dim3(kPublishThreads),
                                  0, (cudaStream_t)stream,
                                  reinterpret_cast<__half* const*>(peer_out_half), offset, n_slice,
                                  peer_flags, sync_words, world, rank,
                                  max_polls ? max_polls : kDefaultPolls, status));
  const int grid = (int)std::max<long long>(1, std::min<long long>(pieces * (world - 1), sm_count()));
  return cuda_status(launch_pdl(gather_publish_kernel, dim3(grid), dim3(kPublishThreads), 0,
                                (cudaStream_t)stream,
                                reinterpret_cast<__half* const*>(peer_out_half), offset, n_slice,
                                peer_flags, sync_words, world, rank,
                                max_polls ? max_polls : kDefaultPolls, status));
}

int hq_gather_wait(const uint32_t* local_flags, const unsigned* sync_words, int world,
                   unsigned max_polls, int* status, hq_stream_t stream) {
  using namespace hq;
  if (!local_flags || !sync_words) return HQ_ERR_NULL_POINTER;
  if (world < 1 || world > 32) return HQ_ERR_BAD_SHAPE;
  gather_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
      local_flags, sync_words, world, max_polls ? max_polls : kDefaultPolls, status);
  return launch_status();
}

int hq_ll_unpack(const hq_ll_packet* ll, long long n, void* out_half, const unsigned* sync_words,
                 unsigned max_polls, int* status, hq_stream_t stream) {
  using namespace hq;
  if (!ll || !out_half) return HQ_ERR_NULL_POINTER;
  if (n <= 0) return HQ_ERR_BAD_SHAPE;
  if (!aligned8(ll)) return HQ_ERR_MISALIGNED;
  const long long want = (n + 255) / 256;
  const int grid = (int)std::min<long long>(want, 4LL * sm_count());
  return cuda_status(launch_pdl(ll_unpack_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                                reinterpret_cast<const uint2*>(ll), n,
                                reinterpret_cast<__half*>(out_half), sync_words,
                                max_polls ? max_polls : kDefaultPolls, status));
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
  const int wpb = blocksize / 8;
  int shift = -1;
  if ((wpb & (wpb - 1)) == 0) {
    shift = 0;
    while ((1 << shift) < wpb) shift++;
  }
  const int low = (flags & HQ_NF4_LOW_NIBBLE_FIRST) ? 1 : 0;
  if (shift >= 0)
    nf4_dequant_kernel<true><<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        B, absmax, lut16, reinterpret_cast<__half*>(out_half), nwords, wpb, shift, low);
  else
    nf4_dequant_kernel<false><<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        B, absmax, lut16, reinterpret_cast<__half*>(out_half), nwords, wpb, 0, low);
  return launch_status();
}

int hq_nf4_gemv_f16(const void* A_half, const uint8_t* B, const float* absmax, const float* lut16,
                    void* out_half, int N, int K, int blocksize, int flags, hq_stream_t stream) {
  return nf4_gemv_impl(A_half, B, absmax, lut16, out_half, N, K, blocksize, flags, LlArgs(),
                       stream);
}

int hq_gemv_fused_nf4_f16(const void* x_half, const void* gamma_half, float eps, const uint8_t* B,
                          const float* absmax, const float* lut16, void* out_half, int rows_out,
                          int n, int blocksize, int flags, int act, hq_stream_t stream) {
  if (rows_out <= 0 || rows_out > (1 << 30)) return HQ_ERR_BAD_SHAPE;
  FuseArgs fuse;
  fuse.gamma = gamma_half;
  fuse.eps = eps;
  fuse.act = act;
  const int rows = act != HQ_ACT_NONE ? 2 * rows_out : rows_out;
  return nf4_gemv_impl(x_half, B, absmax, lut16, out_half, rows, n, blocksize, flags, LlArgs(),
                       stream, &fuse);
}

int hq_nf4_gemv_f16_ll(const void* A_half, const hq_ll_packet* A_ll, long long a_stride,
                       const uint8_t* B, const float* absmax, const float* lut16, void* out_half,
                       int N, int K, int blocksize, int flags, hq_ll_packet* const* peer_ll,
                       long long gather_offset, unsigned* sync_words, int world, int rank,
                       unsigned max_polls, int* status, hq_stream_t stream) {
  if ((A_half != nullptr) == (A_ll != nullptr)) return HQ_ERR_NULL_POINTER;  // exactly one input
  if ((out_half != nullptr) == (peer_ll != nullptr)) return HQ_ERR_NULL_POINTER;  // one output form
  if (!sync_words) return HQ_ERR_NULL_POINTER;
  if (world < 1 || world > 32 || rank < 0 || rank >= world || a_stride < 1)
    return HQ_ERR_BAD_SHAPE;
  LlArgs ll;
  ll.A_ll = A_ll;
  ll.a_stride = a_stride;
  ll.peer_ll = reinterpret_cast<void* const*>(peer_ll);
  ll.gather_offset = gather_offset;
  ll.sync_words = sync_words;
  ll.world = world;
  ll.rank = rank;
  ll.max_polls = max_polls;
  ll.status = status;
  return nf4_gemv_impl(A_half, B, absmax, lut16, out_half, N, K, blocksize, flags, ll, stream);
}

}  // extern "C"
