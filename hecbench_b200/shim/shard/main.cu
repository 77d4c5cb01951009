// C++ host for the single-process sharding context of libhq.so (hq_shard_*):
// one NF4 layer split by output features over G GPUs of the node, driven from
// one process and one host thread.
//
//   shard_demo <gpus> [layers] [n_local] [K]
//
// 1. a chain of `layers` NF4 GEMVs with the low-latency packet gather: layer 0
//    takes a plain input vector, every later layer reads its input from the
//    previous layer's gathered packets (every stride-th element); each rank's
//    copy of every gathered vector is compared with a host fp64 reference;
// 2. the same layer through the ordinary kernel + copy/flag gather
//    (hq_shard_publish), and - when libnccl.so.2 can be loaded - through
//    ncclAllGather (hq_shard_allgather_nccl).
// Prints one line per check and PASS or FAIL; exit code 0 only on PASS.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "hq.h"

#define CK(x)                                                                            \
  do {                                                                                   \
    cudaError_t e_ = (x);                                                                \
    if (e_ != cudaSuccess) {                                                             \
      printf("%s:%d %s: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_));          \
      return 2;                                                                          \
    }                                                                                    \
  } while (0)
#define HQ(x)                                                                            \
  do {                                                                                   \
    int s_ = (x);                                                                        \
    if (s_ != HQ_OK) {                                                                   \
      printf("%s:%d %s: %s (cuda %d)\n", __FILE__, __LINE__, #x, hq_status_string(s_),   \
             hq_last_cuda_error());                                                      \
      return 2;                                                                          \
    }                                                                                    \
  } while (0)

static uint64_t g_state = 0x243f6a8885a308d3ull;
static uint32_t rnd() {
  g_state = g_state * 6364136223846793005ull + 1442695040888963407ull;
  return (uint32_t)(g_state >> 33);
}
static float uni() { return (rnd() & 0xffffff) * (1.0f / 16777216.0f); }

// fp64 reference of rows [n0, n0 + rows) of y = W x for the NF4 format of hq.h
static void host_gemv(const std::vector<__half>& x, const uint8_t* B, const float* absmax,
                      const float* lut, int rows, int K, int bs, std::vector<double>& y) {
  y.assign(rows, 0.0);
  for (int n = 0; n < rows; n++) {
    double acc = 0.0;
    for (int k = 0; k < K; k++) {
      const size_t e = (size_t)n * K + k;
      const uint8_t byte = B[e / 2];
      const int code = (e & 1) ? (byte & 15) : (byte >> 4);  // even element = high nibble
      acc += (double)__half2float(x[k]) * (double)lut[code] * (double)absmax[e / bs];
    }
    y[n] = acc;
  }
}
static double rel_err(const std::vector<__half>& got, size_t off, const std::vector<double>& ref) {
  double rms = 0;
  for (double v : ref) rms += v * v;
  rms = std::sqrt(rms / ref.size());
  double worst = 0;
  for (size_t i = 0; i < ref.size(); i++) {
    const double den = std::fmax(std::fabs(ref[i]), rms > 0 ? rms : 1.0);
    worst = std::fmax(worst, std::fabs((double)__half2float(got[off + i]) - ref[i]) / den);
  }
  return worst;
}

int main(int argc, char** argv) {
  const int G = argc > 1 ? atoi(argv[1]) : 2;
  const int layers = argc > 2 ? atoi(argv[2]) : 4;
  const int n_local = argc > 3 ? atoi(argv[3]) : 1376;
  const int K = argc > 4 ? atoi(argv[4]) : 1024;
  const int bs = 64, slots = 3;
  int ndev = 0;
  CK(cudaGetDeviceCount(&ndev));
  if (G < 1 || G > ndev) {
    printf("need %d GPUs, have %d\n", G, ndev);
    return 2;
  }
  const int N = n_local * G;
  const long long stride = N / K;
  if (stride < 1) {
    printf("n_local * gpus must be at least K\n");
    return 2;
  }
  // one layer (the same weights serve every layer of the chain), rank r owns rows r*n_local..
  std::vector<uint8_t> B((size_t)N * K / 2);
  std::vector<float> absmax((size_t)N * K / bs), lut(16);
  std::vector<__half> x0(K);
  for (auto& b : B) b = (uint8_t)rnd();
  for (auto& a : absmax) a = 0.01f + 0.09f * uni();
  for (int i = 0; i < 16; i++) lut[i] = -1.0f + 2.0f * i / 15.0f;
  for (auto& v : x0) v = __float2half(2.0f * uni() - 1.0f);

  std::vector<int> devs(G);
  for (int r = 0; r < G; r++) devs[r] = r;
  hq_shard_ctx* ctx = nullptr;
  bool nccl = true;
  if (hq_shard_create(&ctx, devs.data(), G, n_local, 1, slots, HQ_SHARD_NCCL) != HQ_OK) {
    nccl = false;
    HQ(hq_shard_create(&ctx, devs.data(), G, n_local, 1, slots, 0));
  }
  std::vector<uint8_t*> dB(G);
  std::vector<float*> dabs(G), dlut(G);
  std::vector<__half*> dx(G), dplain(G);
  for (int r = 0; r < G; r++) {
    CK(cudaSetDevice(r));
    const size_t wb = (size_t)n_local * K / 2, ab = (size_t)n_local * K / bs;
    CK(cudaMalloc(&dB[r], wb));
    CK(cudaMalloc(&dabs[r], ab * 4));
    CK(cudaMalloc(&dlut[r], 64));
    CK(cudaMalloc(&dx[r], K * 2));
    CK(cudaMalloc(&dplain[r], (size_t)N * 2));
    CK(cudaMemcpy(dB[r], B.data() + (size_t)r * wb, wb, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dabs[r], absmax.data() + (size_t)r * ab, ab * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dlut[r], lut.data(), 64, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dx[r], x0.data(), K * 2, cudaMemcpyHostToDevice));
  }
  bool ok = true;
  std::vector<double> ref;
  std::vector<__half> got(N), x = x0;

  // ---- 1. packet chain, checked layer by layer on every rank ----
  double worst = 0;
  for (int l = 0; l < layers; l++) {
    for (int r = 0; r < G; r++)
      HQ(hq_shard_nf4_gemv(ctx, r, l % slots, l == 0 ? dx[r] : nullptr, (l + slots - 1) % slots,
                           stride, dB[r], dabs[r], dlut[r], K, bs, HQ_NF4_WEIGHTS_RESIDENT));
    for (int r = 0; r < G; r++) HQ(hq_shard_unpack(ctx, r, l % slots, dplain[r]));
    host_gemv(x, B.data(), absmax.data(), lut.data(), N, K, bs, ref);
    for (int r = 0; r < G; r++) {
      int st = 0;
      HQ(hq_shard_status(ctx, r, &st));
      if (st != 0) { printf("rank %d: a bounded wait ran out\n", r); ok = false; }
      CK(cudaSetDevice(r));
      CK(cudaMemcpy(got.data(), dplain[r], (size_t)N * 2, cudaMemcpyDeviceToHost));
      worst = std::fmax(worst, rel_err(got, 0, ref));
    }
    for (int k = 0; k < K; k++) x[k] = got[(size_t)k * stride];  // the next layer's input
  }
  printf("packet chain, %d layers on %d GPUs: max rel err %.2e\n", layers, G, worst);
  ok = ok && worst < 1e-2;

  // ---- 2. ordinary kernel + copy/flag gather, then NCCL ----
  host_gemv(x0, B.data(), absmax.data(), lut.data(), N, K, bs, ref);
  for (int form = 0; form < (nccl ? 2 : 1); form++) {
    const int slot = form;
    for (int r = 0; r < G; r++) {
      CK(cudaSetDevice(r));
      HQ(hq_nf4_gemv_f16(dx[r], dB[r], dabs[r], dlut[r], hq_shard_local_slice(ctx, r, slot),
                         n_local, K, bs, 0, hq_shard_stream(ctx, r)));
      if (form == 0) HQ(hq_shard_publish(ctx, r, slot));
    }
    if (form == 1) HQ(hq_shard_allgather_nccl(ctx, slot));
    worst = 0;
    for (int r = 0; r < G; r++) {
      int st = 0;
      HQ(hq_shard_status(ctx, r, &st));
      if (st != 0) ok = false;
      CK(cudaSetDevice(r));
      CK(cudaMemcpy(got.data(), hq_shard_gathered(ctx, r, slot), (size_t)N * 2,
                    cudaMemcpyDeviceToHost));
      worst = std::fmax(worst, rel_err(got, 0, ref));
    }
    printf("%s gather: max rel err %.2e\n", form == 0 ? "copy + flag" : "NCCL all-gather", worst);
    ok = ok && worst < 1e-2;
  }
  if (!nccl) printf("NCCL all-gather: skipped (libnccl.so.2 not loadable)\n");
  hq_shard_destroy(ctx);
  printf("%s\n", ok ? "PASS" : "FAIL");
  return ok ? 0 : 1;
}
