/*
 * hq.h - C ABI of libhq.so: B200 (sm_100a) kernels for HeCBench's weight-only
 * quantized matrix-vector family.
 *
 * Every entry point takes plain device pointers and sizes, is asynchronous on
 * the given CUDA stream (pass NULL for the default stream), returns 0 on
 * success or a negative HQ_ERR_* code, never throws, never exits, and never
 * falls back to the CPU.  Packed-weight pointers must be 16-byte aligned.
 * "half" buffers are IEEE binary16 (the layout of CUDA's __half), declared
 * void* so that this header needs no CUDA include.
 *
 * File:line citations give the HeCBench interface each entry replaces
 * (paths relative to the HeCBench source tree).
 */
#ifndef HQ_H_
#define HQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* hq_stream_t; /* == cudaStream_t */

enum {
  HQ_OK = 0,
  HQ_ERR_BAD_SHAPE = -1,   /* a size violates the documented divisibility rule */
  HQ_ERR_NULL_POINTER = -2,
  HQ_ERR_MISALIGNED = -3,  /* a pointer is not aligned as documented */
  HQ_ERR_CUDA = -4,        /* a CUDA runtime call failed (see hq_last_cuda_error) */
  HQ_ERR_WORKSPACE = -5,   /* workspace missing or too small */
  HQ_ERR_UNSUPPORTED = -6, /* valid arguments the kernels do not cover */
  HQ_ERR_TOO_LARGE = -7,   /* size beyond a documented fixed maximum */
  HQ_ERR_NCCL = -8         /* an NCCL call failed (the communicators were aborted) */
};

int hq_version(void);
const char* hq_status_string(int status);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
int hq_last_cuda_error(void);

/* Index-checked build.  A library compiled with -DHQ_BOUNDS_CHECK tests every
 * global access of its instrumented kernels (NF4 GEMV and dequantize, LUT-GEMM,
 * kQuantize, the int8 activation quantization) against the extent of the
 * buffer the caller described; a violation is recorded and the access skipped,
 * nothing traps.  This call synchronises the current device and returns the
 * number of violations seen since the last reset, with the first one's site
 * (100 * file + access number), byte offset and buffer extent.  An ordinary
 * build returns HQ_ERR_UNSUPPORTED.  No counterpart in the reference (its own
 * guards are commented out, quant3MatMul-cuda/kernels.h:25,41). */
int hq_bounds_check_report(unsigned* violations, unsigned* site, unsigned long long* offset,
                           unsigned long long* extent, int reset);

/* ---------------- GPTQ 3-bit GEMV (quant3MatMul) ---------------- */

/* Replaces vecquant3matmul<float> (quant3MatMul-cuda/kernels.h:171-190).
 * mul[c] += sum_k (scales[c]*q[k][c] - zeros[c]) * vec[k]; mat is
 * int32[height][width], 32 codes per 3 consecutive rows; height % 3 == 0,
 * width % 4 == 0.  Accumulates into mul (the caller zeroes it), like the
 * reference. */
int hq_q3_gemv_f32(const float* vec, const int32_t* mat, float* mul, const float* scales,
                   const float* zeros, int height, int width, hq_stream_t stream);

/* Replaces vecquant3matmul_faster (quant3MatMul-cuda/kernels.h:193-217):
 * fp16 input vector, fp32 parameters and output, fp16 dequant rule. */
int hq_q3_gemv_f16in(const void* vec_half, const int32_t* mat, float* mul,
                     const float* scales, const float* zeros, int height, int width,
                     hq_stream_t stream);

/* Dequantised weights W[K][width], K = height*32/3, by the fp32 rule of
 * kernels.h:43 (fma(scale, q, -zero)) resp. the fp16 rule of
 * kernels.h:121-122,137 (hfma(half(q), half(scale), half(-zero))).
 * No counterpart launcher in the reference; exists for bit-exact checks. */
int hq_q3_dequant_f32(const int32_t* mat, const float* scales, const float* zeros, float* W,
                      int height, int width, hq_stream_t stream);
int hq_q3_dequant_f16(const int32_t* mat, const float* scales, const float* zeros,
                      void* W_half, int height, int width, hq_stream_t stream);

/* ---------------- bitsandbytes blockwise (quantBnB) ---------------- */

/* Replaces the launch kQuantize<256,256><<<grid,block>>>(code, A, out, n)
 * (quantBnB-cuda/main.cu:90-130,176): out[i] = index of the code-table entry
 * that dQuantize<0> (main.cu:13-66) selects for A[i].  Bit exact. */
int hq_bnb_quantize_u8(const float* code256, const float* A, uint8_t* out, size_t n,
                       hq_stream_t stream);

/* flags for the NF4 entry points */
#define HQ_NF4_HIGH_NIBBLE_FIRST 0 /* even element = high nibble (default) */
#define HQ_NF4_LOW_NIBBLE_FIRST 1  /* even element = low nibble */
/* hq_nf4_gemv_f16 only: B, absmax and lut16 are not written by earlier work in
 * the stream (resident model weights), so the kernel may fetch them while the
 * preceding kernel of the stream is still finishing (programmatic dependent
 * launch); the input vector is always read after that kernel has completed. */
#define HQ_NF4_WEIGHTS_RESIDENT 2
/* hq_nf4_gemv_f16_ll with packet output only: peer_ll[0] is the MULTICAST address
 * of the packet vector (an NVSwitch multicast mapping that covers the vector on
 * every GPU of the group, this one included - e.g. the multicast pointer of a
 * symmetric-memory allocation); every result is then written with ONE
 * multimem.st that the switch delivers to all GPUs, instead of one store per
 * GPU.  The other entries of peer_ll are not read. */
#define HQ_NF4_LL_MULTICAST 4

/* NF4 blockwise dequantize (no counterpart in the reference tree):
 * out[e] = half_rn(lut16[code_e] * absmax[e / blocksize]), n elements, two
 * codes per byte, n % 32 == 0, blocksize a multiple of 32. */
int hq_nf4_dequant_f16(const uint8_t* B, const float* absmax, const float* lut16,
                       void* out_half, size_t n, int blocksize, int flags,
                       hq_stream_t stream);

/* NF4 4-bit GEMV (no counterpart in the reference tree):
 * out[n] = half_rn(sum_k A[k] * lut16[code[n][k]] * absmax[(n*K+k)/blocksize]),
 * B is [N][K/2] bytes row-major; K % 32 == 0, blocksize a multiple of 32 that
 * divides K. */
int hq_nf4_gemv_f16(const void* A_half, const uint8_t* B, const float* absmax,
                    const float* lut16, void* out_half, int N, int K, int blocksize,
                    int flags, hq_stream_t stream);

/* ---------------- output-feature sharding over the GPUs of a node ----------------
 *
 * No counterpart in the reference tree (its only collective code is the NCCL
 * all-reduce sample ccl-cuda/main.cu:83-117).  Every output feature of the
 * family is independent, so a layer is split by output features: each GPU runs
 * the ordinary kernel on its slice and the slices are gathered into a vector
 * every GPU holds.  Two gathers are provided, both on peer-mapped device memory
 * with plain peer stores (no NCCL, no multicast); every wait in them is bounded
 * by a poll limit (max_polls, 0 = default of about a second) after which the
 * kernel sets *status (device int, nullable) to 1 and returns.
 *
 * (1) Low-latency packets, for the batch-1 path where the gather is tens of
 * kilobytes and latency is everything.  The gathered vector is an array of
 * hq_ll_packet, one per element: the fp16 value and the number ("epoch") of the
 * gather round that wrote it, written and read with single 8-byte accesses, so
 * a reader that sees the expected epoch also sees the value - no fence, no flag
 * round trip, no follow-up kernel.  The GEMV stores every result as a packet
 * into the packet vector of EVERY GPU as soon as the row is finished, and the
 * next layer's GEMV takes its input straight from the packets, waiting for
 * each until it carries the epoch of the latest completed round.
 * sync_words: two device words per GPU, zero before the first call: [0] a CTA
 * counter, [1] the epoch of the latest round this GPU has completed sending.
 * A call reads E = sync_words[1] when it starts, expects E in its input
 * packets, writes E + 1 into its output packets and leaves sync_words[1] =
 * E + 1.  All GPUs must issue the same sequence of calls.  Packet vectors must
 * start zeroed.  A vector may be rewritten as soon as the NEXT round's packets
 * are complete on this GPU, so a chain of layers must alternate between at
 * least two packet vectors. */
typedef struct hq_ll_packet {
  uint32_t value; /* low 16 bits: the fp16 element */
  uint32_t epoch; /* gather round that wrote it */
} hq_ll_packet;

/* hq_nf4_gemv_f16 with packet input and/or packet output.
 * Input: exactly one of A_half (plain fp16[K]) and A_ll (packets; element k is
 * A_ll[k * a_stride], a_stride >= 1; K <= 32768 in this form) is non-null.
 * Output: exactly one of out_half (plain fp16[N]) and peer_ll is non-null;
 * peer_ll is a device-resident array of `world` pointers, peer_ll[r] = packet
 * vector of GPU r (peer-mapped), and result n goes to element gather_offset + n
 * of each (normally gather_offset = rank * N). */
int hq_nf4_gemv_f16_ll(const void* A_half, const hq_ll_packet* A_ll, long long a_stride,
                       const uint8_t* B, const float* absmax, const float* lut16, void* out_half,
                       int N, int K, int blocksize, int flags, hq_ll_packet* const* peer_ll,
                       long long gather_offset, unsigned* sync_words, int world, int rank,
                       unsigned max_polls, int* status, hq_stream_t stream);

/* Plain fp16 copy of n packets: waits (bounded) for each until it carries
 * sync_words[1], the epoch of the latest round completed on this GPU; with
 * sync_words == NULL the values are copied unchecked. */
int hq_ll_unpack(const hq_ll_packet* ll, long long n, void* out_half, const unsigned* sync_words,
                 unsigned max_polls, int* status, hq_stream_t stream);

/* (2) Copy + flag, for larger slices (the batched path) and for any kernel of
 * the family: an ordinary launch writes its slice into this GPU's own gathered
 * vector (elements offset .. offset + n_slice of peer_out_half[rank]);
 * hq_gather_publish then copies the slice to every peer with 16-byte stores
 * over NVLink (the copy is spread over as many CTAs as the slice has 16 KB
 * pieces per peer), makes it visible system-wide, raises this rank's flag word
 * on every GPU (peer_flags[r], `world` words each, zero before the first call)
 * and waits until all ranks' slices of the same round have landed here.
 * n_slice = 0: the producing kernel stored the slice to the peers itself
 * (hq_qgemm_*_peers); only the flags and the wait remain.
 * sync_words as above ([1] counts rounds).  hq_gather_wait is that wait alone.
 * As with packets, a chain of rounds must alternate between at least two
 * gathered vectors: a rank that has seen round L complete may start storing
 * round L + 1 while a slower rank still reads round L - 1's vector. */
int hq_gather_publish(void* const* peer_out_half, long long offset, int n_slice,
                      uint32_t* const* peer_flags, unsigned* sync_words, int world, int rank,
                      unsigned max_polls, int* status, hq_stream_t stream);
int hq_gather_wait(const uint32_t* local_flags, const unsigned* sync_words, int world,
                   unsigned max_polls, int* status, hq_stream_t stream);

/* (3) A context for hosts that drive all GPUs of the node from ONE process
 * (C or C++ drivers; the Python layer runs one process per GPU instead and
 * keeps its buffers in torch symmetric memory).  hq_shard_create enables peer
 * access between the listed devices and allocates, per rank, a stream, `slots`
 * gathered buffers in both forms above (packet vectors for rows == 1; fp16
 * buffers [world][rows][n_local] with their flag words), the device-resident
 * pointer tables, the sync words and a status word; with HQ_SHARD_NCCL it also
 * loads libnccl.so.2 and creates one communicator per device (the sequence of
 * ccl-cuda/main.cu:83-91).  n_local = output features per rank, rows = 1 for a
 * mat-vec or the token batch for the batched product, slots >= 2.  The
 * per-rank calls are asynchronous on that rank's stream (hq_shard_stream) and
 * may be issued for rank 0 .. world-1 in turn from one host thread: a rank
 * that waits for another's data polls with a bound of about a second.
 *   hq_shard_nf4_gemv      NF4 GEMV of the rank's n_local rows with packet
 *                          output into buffer `slot` of every rank; input
 *                          A_half, or (A_half == NULL) elements 0, a_stride,
 *                          2*a_stride, ... of the rank's own packet vector a_slot
 *   hq_shard_unpack        plain fp16 copy of the rank's packet vector `slot`
 *   hq_shard_local_slice   where an ordinary kernel on that rank's stream
 *                          writes its slice [rows][n_local] of buffer `slot`
 *   hq_shard_publish       copy + flag gather of that slice
 *   hq_shard_allgather_nccl  the same gather by ncclAllGather, one grouped call
 *                          for all ranks (ccl-cuda/main.cu:112-117); on failure
 *                          the communicators are aborted (ncclCommAbort) and
 *                          HQ_ERR_NCCL is returned
 *   hq_shard_gathered      the rank's copy of gathered buffer `slot`
 *   hq_shard_status        synchronises the rank's stream and returns its
 *                          status word (1 = a bounded wait ran out)
 * hq_shard_layout is the index arithmetic alone (no CUDA call): first packet
 * of a rank's results and first fp16 element of its slice, counted from the
 * start of the rank's packet resp. fp16 region, and elements per buffer. */
#define HQ_SHARD_NCCL 1
typedef struct hq_shard_ctx hq_shard_ctx;
int hq_shard_layout(int world, int rows, long long n_local, int slots, int rank, int slot,
                    long long* packet_index, long long* slice_index, long long* slot_elems);
int hq_shard_create(hq_shard_ctx** ctx, const int* devices, int world, long long n_local, int rows,
                    int slots, int flags);
void hq_shard_destroy(hq_shard_ctx* ctx);
hq_stream_t hq_shard_stream(hq_shard_ctx* ctx, int rank);
int hq_shard_nf4_gemv(hq_shard_ctx* ctx, int rank, int slot, const void* A_half, int a_slot,
                      long long a_stride, const uint8_t* B, const float* absmax,
                      const float* lut16, int K, int blocksize, int flags);
int hq_shard_unpack(hq_shard_ctx* ctx, int rank, int slot, void* out_half);
void* hq_shard_local_slice(hq_shard_ctx* ctx, int rank, int slot);
int hq_shard_publish(hq_shard_ctx* ctx, int rank, int slot);
int hq_shard_allgather_nccl(hq_shard_ctx* ctx, int slot);
const void* hq_shard_gathered(hq_shard_ctx* ctx, int rank, int slot);
int hq_shard_status(hq_shard_ctx* ctx, int rank, int* status_out);

/* ---------------- LUT-GEMM binary-coding mat-vec (lut-gemm) ---------------- */

/* Bytes of zero-initialised device scratch hq_lutgemm_nqmv needs for M
 * outputs.  The scratch must be zero before the first call; every call leaves
 * it zero again, so one buffer can serve a sequence of calls on one stream. */
size_t hq_lutgemm_workspace_bytes(int M);

/* Replaces matmul(output, input, nqW, m) -> nqmv / nqmv_bias
 * (lut-gemm-cuda/kernels.cu:22-31, mv_fp16.h:101-131,228-259) for one input
 * row.  bW uint32[K/32][nb][M], alpha half[K/group][nb][M], q_bias
 * half[K/group][M] or NULL, x half[K], out half[M] (overwritten).
 * K % 32 == 0, group_size % 32 == 0 (32, or an even multiple of 32), M % 4 == 0,
 * 1 <= nb <= 8; bW 16-byte aligned, alpha, q_bias and out 8-byte aligned. */
int hq_lutgemm_nqmv(void* out_half, const void* x_half, const uint32_t* bW,
                    const void* alpha_half, const void* q_bias_half, int M, int K, int nb,
                    int group_size, void* workspace, size_t workspace_bytes,
                    hq_stream_t stream);

/* Largest M hq_lutgemm_nqmv_noalloc accepts. */
#define HQ_LUTGEMM_NOALLOC_MAX_M 65536

/* hq_lutgemm_nqmv for callers that must not allocate device memory.  It has no
 * counterpart in the reference.  Some hosts of this library cannot call
 * cudaMalloc at the point where they need the mat-vec: a plugin that runs
 * inside another framework's memory pool and owns no allocator of its own, a
 * real-time or serving loop in which a cudaMalloc (which synchronises the
 * device) is forbidden, or code whose memory budget was fixed at start-up.
 * For them the fp32 scratch row the kernel needs is a fixed array inside the
 * library's device image instead of a caller-provided workspace, so the call
 * takes only inputs and outputs and performs no cudaMalloc / cudaFree and uses
 * no allocating library routine.
 *   - M must not exceed HQ_LUTGEMM_NOALLOC_MAX_M; larger sizes return
 *     HQ_ERR_TOO_LARGE and nothing is launched.  All other argument rules are
 *     those of hq_lutgemm_nqmv.
 *   - The array (257 KiB) is held by every GPU that loads the library, until
 *     the process exits.
 *   - The first call on each device looks up the array's device address (with
 *     that device current).  Make that first call outside any stream capture.
 *   - Every call on a device uses the same array and begins by clearing the
 *     part it needs on the given stream.  Calls whose execution overlaps on
 *     the GPU (different streams, or several host threads on one device) race
 *     on it and give wrong results: serialise them. */
int hq_lutgemm_nqmv_noalloc(void* out_half, const void* x_half, const uint32_t* bW,
                            const void* alpha_half, const void* q_bias_half, int M, int K, int nb,
                            int group_size, hq_stream_t stream);

/* ---------------- AQLM additive codebooks (quantAQLM) ---------------- */

/* Replaces code1x16_matvec (quantAQLM-cuda/main.cu:113-141).  codes
 * uint16[prob_m][prob_k/8], x half[prob_k], out half[prob_m] (overwritten),
 * codebook half[.][65536][8] with up to three stacked codebooks selected by
 * the cumulative row ranges cb_sizes[0..3] (main.cu:43-51), cb_stride_int4 =
 * 16-byte units between codebooks.  scales (half[prob_m], nullable) is an
 * extension: the row sum is multiplied by it before rounding.
 * prob_k % 64 == 0. */
int hq_aqlm_1x16_matvec(const void* codes, const void* x_half, void* out_half,
                        const void* codebook, int prob_m, int prob_k, const int cb_sizes[4],
                        int cb_stride_int4, const void* scales_half, hq_stream_t stream);

/* AQLM 2x8 (no counterpart in the reference tree): codes
 * uint8[prob_m][prob_k/8][2], codebooks half[2][256][8], scales nullable.
 * prob_k % 64 == 0. */
int hq_aqlm_2x8_matvec(const void* codes, const void* x_half, void* out_half,
                       const void* codebooks, int prob_m, int prob_k, const void* scales_half,
                       hq_stream_t stream);

/* ---------------- per-token int8 activation quantization (quantVLLM) ---------------- */

/* input element types of the hq_vllm_* entries */
#define HQ_DTYPE_F16 0
#define HQ_DTYPE_BF16 1
#define HQ_DTYPE_F32 2

/* Replaces static_scaled_int8_quant<scalar_t>(output, input, hidden_size,
 * num_tokens, scale, azp) (quantVLLM-cuda/main.cu:137-153) and its kernels
 * (main.cu:12-46): out[t][i] = sat8(rint(x[t][i] / scale)) when azp == 0, else
 * sat8(sat32(rint(x / scale)) + azp).  input is [num_tokens][hidden_size] of
 * the given element type, out int8 of the same shape.  Byte exact against the
 * reference's host functions (reference.h:1-31). */
int hq_vllm_static_scaled_int8_quant(int8_t* out, const void* input, int dtype, int hidden_size,
                                     int num_tokens, float scale, int32_t azp,
                                     hq_stream_t stream);

/* Replaces dynamic_scaled_int8_quant<scalar_t>(output, input, hidden_size,
 * num_tokens, scales, azp) (quantVLLM-cuda/main.cu:155-172) and its kernels
 * (main.cu:48-134): per token row, scales[t] = absmax / 127 and out =
 * sat8(rint(x * (127 / absmax))) when azp == NULL; else scales[t] = (max -
 * min) / 255, azp[t] = rint(-128 - min / scales[t]) and out = sat8(sat32(rint(x
 * / scales[t])) + azp[t]), the running maximum starting at FLT_MIN as in the
 * reference.  Byte exact against reference.h:33-93. */
int hq_vllm_dynamic_scaled_int8_quant(int8_t* out, const void* input, int dtype, int hidden_size,
                                      int num_tokens, float* scales, int32_t* azp,
                                      hq_stream_t stream);

/* ---------------- gemv: uniform int8 / int4 weight-only mat-vec ---------------- */

/* gemv_quantized_int8 / gemv_quantized_int4 / gemv_fp16 of src/gemv-cuda
 * (kernels.h:127-200, :205-307, :64-123; launchers gemv.cu:15-36, :38-59,
 * :61-81).  mat is row-major [rows][n]: int8 values, or for int4 n/2 bytes
 * per row with element 2j in the LOW nibble of byte j and 2j+1 in the high
 * nibble (uint4_2::getX / getY, kernels.h:17-23), or fp16.  One scale and one
 * zero point per tensor, rounded to fp16 as the reference launchers do
 * (gemv.cu:21-22, :44-45):
 *   res[row] = half( half(scale) * sum_j vec[j] * (w[row][j] - half(zero_point)) )
 * with fp32 accumulation across 32- or 64-weight partial sums formed in fp16.
 * The reference drivers use square matrices (rows == n == size); here rows and
 * n are independent.  n must be a multiple of 8 (fp16), 16 (int8) or 32 (int4);
 * mat and vec 16-byte aligned; n <= 115712, else HQ_ERR_TOO_LARGE (the inputs are
 * staged in 226 KB of shared memory; beyond half of that length only one CTA fits
 * an SM).  The grid and block shapes of the reference launchers
 * (block_dim_x, block_dim_y, num_per_thread) are tuning knobs of its kernels
 * and have no counterpart here. */
int hq_gemv_f16(const void* mat_half, const void* vec_half, void* res_half, int rows, int n,
                hq_stream_t stream);
int hq_gemv_int8_f16(const int8_t* mat, const void* vec_half, void* res_half, int rows, int n,
                     float scale, float zero_point, hq_stream_t stream);
int hq_gemv_int4_f16(const uint8_t* mat, const void* vec_half, void* res_half, int rows, int n,
                     float scale, float zero_point, hq_stream_t stream);

/* ---------------- RMSNorm -> mat-vec -> gated activation, fused ---------------- */

/* The entry of a decode-time MLP in one launch: RMSNorm of the input vector
 * (src/rmsnorm-cuda/reference.h:4-25: xn[k] = x[k] * rsqrt(mean(x^2) + eps) *
 * gamma[k], computed in fp32 and rounded to fp16; gamma_half == NULL skips it),
 * the weight-only mat-vec in one of the four formats above, and the gated
 * activation of row pairs.  With act != HQ_ACT_NONE the matrix has 2 * rows_out
 * rows: row 2m is the value row and row 2m + 1 the gate row of output m (the
 * x / gate order of src/geglu-cuda/reference.h:8-16, per output feature) and
 *   out[m] = v * g / (1 + exp(-g))                  HQ_ACT_SWIGLU (src/swish-cuda/reference.h:4)
 *   out[m] = v * 0.5 * g * (1 + erf(g / sqrt(2)))   HQ_ACT_GEGLU  (src/geglu-cuda/reference.h:1-5)
 * in fp32, rounded to fp16 once; with HQ_ACT_NONE the matrix has rows_out rows
 * and the call is the plain mat-vec of the normalised vector.  Layouts, scale /
 * zero point / absmax / level-table rules, alignment and length limits are those
 * of hq_gemv_f16, hq_gemv_int8_f16, hq_gemv_int4_f16 and hq_nf4_gemv_f16 (NF4:
 * B is the row-major matrix of 2 * rows_out (or rows_out) rows of n codes, n
 * takes the place of K, flags are HQ_NF4_LOW_NIBBLE_FIRST and
 * HQ_NF4_WEIGHTS_RESIDENT).
 * No counterpart in the reference tree, which has the three steps as separate
 * benchmarks. */
#define HQ_ACT_NONE 0
#define HQ_ACT_SWIGLU 1
#define HQ_ACT_GEGLU 2
int hq_gemv_fused_f16(const void* x_half, const void* gamma_half, float eps, const void* mat_half,
                      void* out_half, int rows_out, int n, int act, hq_stream_t stream);
int hq_gemv_fused_int8_f16(const void* x_half, const void* gamma_half, float eps, const int8_t* mat,
                           void* out_half, int rows_out, int n, float scale, float zero_point,
                           int act, hq_stream_t stream);
int hq_gemv_fused_int4_f16(const void* x_half, const void* gamma_half, float eps,
                           const uint8_t* mat, void* out_half, int rows_out, int n, float scale,
                           float zero_point, int act, hq_stream_t stream);
int hq_gemv_fused_nf4_f16(const void* x_half, const void* gamma_half, float eps, const uint8_t* B,
                          const float* absmax, const float* lut16, void* out_half, int rows_out,
                          int n, int blocksize, int flags, int act, hq_stream_t stream);

/* ---------------- quantization parameters and packers ---------------- */

/* Scale and zero point of an affine integer quantization from per-channel minima
 * and maxima: replaces the kernel zero_point of src/zeropoint-cuda/main.cu:10-80
 * (same argument order; host check src/zeropoint-cuda/reference.h:1-71).  Bit for
 * bit the reference's results, including its mixed fp32 / fp64 arithmetic: with
 * preserve_sparsity and min < 0 < max the range is made symmetric first and the
 * zero point is (qmin + qmax) / 2; the range is widened to contain 0; scale =
 * (max - min) / (qmax - qmin), or 0.1 where that is 0 or its reciprocal
 * overflows; the zero point is clamped to [qmin, qmax] and rounded to nearest,
 * ties to even.  size >= 0, qmax > qmin. */
int hq_zero_point(const float* x_min, const float* x_max, int32_t qmin, int32_t qmax, int size,
                  int preserve_sparsity, float* scale, int32_t* zero_point, hq_stream_t stream);

/* Round-to-nearest 3-bit quantizer and packer: produces what hq_q3_gemv_f32 /
 * hq_q3_gemv_f16in consume (the layout of src/quant3MatMul-cuda/kernels.h:41-87;
 * the reference tree holds only that consumer).  W: K x N weights, row-major, of
 * type dtype (HQ_DTYPE_F16, _BF16, _F32).  Per column c, in fp32: lo = min(column,
 * 0), hi = max(column, 0) (-1 and 1 if both are 0); scale = (hi - lo) / 7; z =
 * rint(-lo / scale); code = clamp(rint(w / scale) + z, 0, 7), roundings to
 * nearest, ties to even - GPTQ's min / max quantizer without its error search;
 * scales[c] = scale, zeros[c] = scale * z.  mat: int32[K * 3 / 32][N].  workspace:
 * hq_q3_quantize_workspace_bytes(N) bytes of device scratch (contents
 * irrelevant).  K % 32 == 0, N % 8 == 0, W / mat / scales / zeros 16-byte
 * aligned. */
size_t hq_q3_quantize_workspace_bytes(int N);
int hq_q3_quantize(const void* W, int dtype, int K, int N, int32_t* mat, float* scales,
                   float* zeros, void* workspace, size_t workspace_bytes, hq_stream_t stream);

/* Greedy binary-coding quantizer: produces what hq_lutgemm_nqmv consumes (the
 * layouts of src/lut-gemm-cuda/main.cu:27-30,118-134; the reference tree holds only
 * that consumer).  W: K x M weights, row-major (input k, output m), of type dtype.
 * Per output m and group of group_size consecutive inputs, in fp32 (a sum over a
 * group = one sum per 32 consecutive inputs, ascending, those partial sums added
 * in ascending order): q_bias = half(mean) (q_bias_half == NULL: no offsets, the
 * mean stays in the residual); r = w - q_bias; for each of the nb planes alpha =
 * half(mean |r|), bit = (r >= 0), r -= +-alpha (the rounded value).  bW:
 * uint32[K / 32][nb][M], bit t of a word = input 32 * row + t; alpha_half:
 * half[K / group_size][nb][M]; q_bias_half: half[K / group_size][M].
 * 1 <= nb <= 8, group_size % 32 == 0 and at most 512, K % group_size == 0,
 * M % 8 == 0, W and bW 16-byte aligned. */
int hq_lutgemm_quantize(const void* W, int dtype, int K, int M, int nb, int group_size,
                        uint32_t* bW, void* alpha_half, void* q_bias_half, hq_stream_t stream);

/* Blockwise 4-bit quantizer: produces what hq_nf4_dequant_f16 / hq_nf4_gemv_f16 /
 * hq_qgemm_nf4_f16 consume.  W: n weights of type dtype (HQ_DTYPE_F16, _BF16 or
 * _F32); absmax[b] = max |w| over block b of blocksize weights; x = fp32(w) * (1 /
 * absmax[b]) (0 where absmax is zero, denormal or infinite); code = how many of the 15 midpoints
 * (lut16[j] + lut16[j+1]) / 2, formed in fp32 from the 16 ascending levels, are
 * < x: the nearest level, a tie going to the lower one.  B gets two codes per
 * byte in the nibble order of flags (HQ_NF4_*_NIBBLE_FIRST).  blocksize a power
 * of two in 32 .. 4096, n % blocksize == 0, W 16-byte aligned, B 4-byte aligned.
 * No counterpart in the reference tree (src/quantBnB-cuda/main.cu:13-85 is the
 * 8-bit whole-tensor quantizer, hq_bnb_quantize_u8 here). */
int hq_nf4_quantize(const void* W, int dtype, size_t n, int blocksize, const float* lut16,
                    int flags, uint8_t* B, float* absmax, hq_stream_t stream);

/* MXFP4 (32 consecutive elements share a power-of-two scale, each element is a
 * 4-bit e2m1 float with values 0, .5, 1, 1.5, 2, 3, 4, 6 and a sign).
 * hq_mxfp4_qdq replaces qdq_mxfp4_kernel of src/mxfp4-cuda/main.cu:112-150 (out =
 * the quantized values in the input type; dtype HQ_DTYPE_F16 or HQ_DTYPE_BF16):
 * per group k = floor(log2(max |x|, rounded up to the next power of two from
 * 1.75 * 2^e)) - 2, clamped to [-127, 127]; x / 2^k is rounded to the nearest grid
 * value, ties to the even mantissa, magnitudes above 6 saturate; out = that *
 * 2^k.  Same bits as the reference kernel for every group whose maximum is
 * finite and, after that rounding, a normal number of the type; a group with a
 * smaller maximum (the reference takes the logarithm of zero there) uses the
 * smallest k the reference can produce, so a group of zeros gives zeros.
 * hq_mxfp4_quantize writes the packed form instead - codes: one byte per two
 * elements, element 2j in the low nibble, nibble = sign << 3 | index into the
 * grid; scales_e8m0: one byte k + 127 per group - and hq_mxfp4_dequantize turns
 * it back into values (= what hq_mxfp4_qdq gives).  numel % 32 == 0; in / out
 * 16-byte aligned, codes 4-byte aligned.  No packed form exists in the reference. */
int hq_mxfp4_qdq(const void* in, void* out, size_t numel, int dtype, hq_stream_t stream);
int hq_mxfp4_quantize(const void* in, uint8_t* codes, uint8_t* scales_e8m0, size_t numel, int dtype,
                      hq_stream_t stream);
int hq_mxfp4_dequantize(const uint8_t* codes, const uint8_t* scales_e8m0, void* out, size_t numel,
                        int dtype, hq_stream_t stream);

/* ---------------- batched dequant-GEMM (tensor cores) ---------------- */

/* Y[Mb][N] = X[Mb][K] * W[K][N] with W the GPTQ 3-bit layout of quant3MatMul
 * (mat int32[K*3/32][N]) and per-group fp16 parameters scales/zeros
 * half[K/group_size][N]: W[k][n] = hfma(half(q), scale, -zero), fp32
 * accumulation on the sm_100a tensor cores (tcgen05 / tensor memory), fp16
 * output.  No counterpart in the reference tree.  1 <= Mb <= 128,
 * N % 128 == 0, K % group_size == 0, group_size % 64 == 0.  workspace
 * (nullable) is zero-initialised device scratch of hq_qgemm_workspace_bytes
 * bytes that lets the kernel split K over several CTAs when N alone gives too
 * few tiles to fill the GPU; every call that ends with status 0 leaves it
 * zero.  Two rules follow: (1) one workspace serves one stream - calls that may
 * overlap on the GPU (different streams, several host threads) need a
 * workspace each, or they race on the partial sums and tile counters and give
 * wrong results without any error; (2) after a call that set the status word
 * the workspace may hold partial sums and counters: clear it (cudaMemsetAsync
 * on the same stream) before it is used again.  status_word (device int,
 * nullable) is set to 1 if a bounded in-kernel wait ran out. */
size_t hq_qgemm_workspace_bytes(int Mb, int N);
int hq_qgemm_q3_f16(const void* X_half, const int32_t* mat, const void* scales_half,
                    const void* zeros_half, void* Y_half, int Mb, int N, int K, int group_size,
                    void* workspace, size_t workspace_bytes, int* status_word,
                    hq_stream_t stream);

/* The same product with NF4 weights in the layout of hq_nf4_gemv_f16:
 * B uint8[N][K/2] (output-feature-major, two codes per byte; flags as there),
 * absmax float[N*K/blocksize], lut16 float[16];
 * W[k][n] = half(lut16[code] * absmax[(n*K + k) / blocksize]) exactly as
 * hq_nf4_dequant_f16 produces it.  No counterpart in the reference tree.
 * 1 <= Mb <= 128, N % 128 == 0, blocksize % 64 == 0, K % blocksize == 0.
 * workspace and status_word as for hq_qgemm_q3_f16. */
int hq_qgemm_nf4_f16(const void* X_half, const uint8_t* B, const float* absmax, const float* lut16,
                     void* Y_half, int Mb, int N, int K, int blocksize, int flags, void* workspace,
                     size_t workspace_bytes, int* status_word, hq_stream_t stream);

/* Sharded layers: the same two products with the gather fused into the
 * epilogue.  Every finished 128-feature tile is stored straight into the output
 * slice of EVERY GPU of the node: element (t, n) goes to peer_Y_half[r][y_offset
 * + t * N + n] for r = 0 .. world - 1 (peer-mapped buffers, this GPU's own
 * among them; peer_Y_half is a device-resident pointer table as for
 * hq_gather_publish), so the transfer over NVLink runs tile by tile beside the
 * remaining tiles' math and no copy kernel follows.  The stores are complete
 * when the launch is; hq_gather_publish with n_slice = 0 on the same stream
 * then raises the flags and waits for the other ranks. */
int hq_qgemm_q3_f16_peers(const void* X_half, const int32_t* mat, const void* scales_half,
                          const void* zeros_half, void* const* peer_Y_half, long long y_offset,
                          int world, int Mb, int N, int K, int group_size, void* workspace,
                          size_t workspace_bytes, int* status_word, hq_stream_t stream);
int hq_qgemm_nf4_f16_peers(const void* X_half, const uint8_t* B, const float* absmax,
                           const float* lut16, void* const* peer_Y_half, long long y_offset,
                           int world, int Mb, int N, int K, int blocksize, int flags,
                           void* workspace, size_t workspace_bytes, int* status_word,
                           hq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HQ_H_ */
