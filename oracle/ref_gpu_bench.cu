// Times the reference's own CUDA kernels (compiled for sm_100a from their own
// sources, see build.py) with the protocol bench.py uses for the product
// kernels: R rotating replicas of the packed weights (R x bytes several times
// the L2), one CUDA graph of R launches, CUDA events around `iters` replays.
// TEST / MEASUREMENT INFRASTRUCTURE ONLY - nothing of the product links this.
//
// The reference launchers use the default stream.  This program and the
// reference objects it links are compiled with --default-stream per-thread, so
// those launches land on cudaStreamPerThread, which is the stream captured.
// If capture is refused the launches are timed eagerly and the line says so.
//
// Output: one JSON object on stdout,
//   {"<workload>": {"us": <per launch>, "launch": "graph"|"eager", "replicas": R}, ...}
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

extern "C" {
void ref_q3_gemv_f32(float* vec, int* mat, float* mul, float* scales, float* zeros, int height,
                     int width);
void ref_q3_gemv_faster(void* vec_half, int* mat, float* mul, float* scales, float* zeros,
                        int height, int width);
void ref_bnb_quantize_gpu(const float* d_code, const float* d_A, uint8_t* d_out, int n);
void ref_lutgemm_matmul(void* output, void* input, unsigned int* bW, void* alpha, void* q_bias,
                        int M, int K, int nb, int num_groups);
void ref_aqlm_1x16(const void* A, const void* B, void* C, const void* codebook, int prob_m,
                   int prob_k, const int* sizes, int codebook_stride);
void ref_gemv_int8(int8_t* mat, void* vec_half, void* res_half, unsigned size, float scale_f,
                   float zero_point_f, unsigned bx, unsigned by);
void ref_gemv_int4(uint8_t* mat, void* vec_half, void* res_half, unsigned size, float scale_f,
                   float zero_point_f, unsigned bx, unsigned by);
int ref_mxfp4_qdq(const void* in, void* out, int numel, int bf16);
int ref_zero_point_gpu(const float* x_min, const float* x_max, int32_t qmin, int32_t qmax, int size,
                       int preserve_sparsity, float* scale, int32_t* zp);
}

#define CK(x)                                                                          \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_)); \
      exit(1);                                                                         \
    }                                                                                  \
  } while (0)

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
// kind 0: random 32-bit words; 1: fp32 uniform [lo, hi); 2: fp16 uniform [lo, hi)
__global__ void fill_kernel(void* p, size_t n, int kind, float lo, float hi, uint64_t seed) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t r = mix64(seed * 0x100000001b3ull + i);
    const float u = (float)(r >> 40) * (1.0f / 16777216.0f);
    if (kind == 0) ((uint32_t*)p)[i] = (uint32_t)r;
    else if (kind == 1) ((float*)p)[i] = lo + (hi - lo) * u;
    else ((__half*)p)[i] = __float2half_rn(lo + (hi - lo) * u);
  }
}

static std::vector<void*> g_allocs;
static void* dmalloc(size_t bytes) {
  void* p = nullptr;
  CK(cudaMalloc(&p, bytes));
  g_allocs.push_back(p);
  return p;
}
static void free_all() {
  for (void* p : g_allocs) cudaFree(p);
  g_allocs.clear();
}
static void* filled(size_t n, int kind, float lo, float hi, uint64_t seed) {
  const size_t elem = kind == 2 ? 2 : 4;
  void* p = dmalloc(n * elem);
  fill_kernel<<<1024, 256>>>(p, n, kind, lo, hi, seed);
  CK(cudaGetLastError());
  return p;
}

struct Result {
  double us;
  bool graph;
  int replicas;
};

// launch(i) issues the reference launcher on replica i (default = per-thread stream)
static Result time_launches(int R, int iters, const std::function<void(int)>& launch) {
  cudaStream_t st = cudaStreamPerThread;
  for (int w = 0; w < 2; w++)
    for (int i = 0; i < R; i++) launch(i);
  CK(cudaStreamSynchronize(st));
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  bool ok = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
  if (ok) {
    for (int i = 0; i < R; i++) launch(i);
    ok = cudaStreamEndCapture(st, &graph) == cudaSuccess && graph != nullptr;
  }
  if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();  // clear the capture error; fall back to eager launches
    exec = nullptr;
  }
  auto pass = [&]() {
    if (exec) CK(cudaGraphLaunch(exec, st));
    else
      for (int i = 0; i < R; i++) launch(i);
  };
  for (int w = 0; w < 3; w++) pass();
  CK(cudaStreamSynchronize(st));
  cudaEvent_t a, b;
  CK(cudaEventCreate(&a));
  CK(cudaEventCreate(&b));
  CK(cudaEventRecord(a, st));
  for (int it = 0; it < iters; it++) pass();
  CK(cudaEventRecord(b, st));
  CK(cudaEventSynchronize(b));
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, a, b));
  CK(cudaGetLastError());
  if (exec) cudaGraphExecDestroy(exec);
  if (graph) cudaGraphDestroy(graph);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return Result{ms * 1e3 / ((double)iters * R), exec != nullptr, R};
}

static int replicas_for(double bytes, double target) {
  int r = (int)(target / bytes + 0.999);
  return r < 2 ? 2 : r;
}

static bool g_first = true;
static void emit(const char* name, const Result& r) {
  printf("%s\"%s\": {\"us\": %.3f, \"launch\": \"%s\", \"replicas\": %d}", g_first ? "" : ", ", name,
         r.us, r.graph ? "graph" : "eager", r.replicas);
  g_first = false;
  fflush(stdout);
}

static void bench_q3(const char* name_f32, const char* name_f16, int K, int W, double target) {
  const int height = K * 3 / 32;
  const double bytes = (double)height * W * 4;
  const int R = replicas_for(bytes, target);
  std::vector<int*> mats(R);
  for (int i = 0; i < R; i++) mats[i] = (int*)filled((size_t)height * W, 0, 0, 0, 100 + i);
  float* vec = (float*)filled(K, 1, -1.f, 1.f, 1);
  __half* vh = (__half*)filled(K, 2, -1.f, 1.f, 2);
  float* sc = (float*)filled(W, 1, 0.001f, 0.01f, 3);
  float* z = (float*)filled(W, 1, 0.f, 0.07f, 4);
  float* mul = (float*)dmalloc((size_t)W * 4);
  CK(cudaMemset(mul, 0, (size_t)W * 4));
  const int iters = bytes > 5e7 ? 10 : 40;
  emit(name_f32, time_launches(R, iters, [&](int i) {
         ref_q3_gemv_f32(vec, mats[i], mul, sc, z, height, W);
       }));
  emit(name_f16, time_launches(R, iters, [&](int i) {
         ref_q3_gemv_faster(vh, mats[i], mul, sc, z, height, W);
       }));
  free_all();
}

int main(int argc, char** argv) {
  double target = 640e6;
  if (argc > 1) target = atof(argv[1]);
  CK(cudaSetDevice(0));
  printf("{");
  bench_q3("q3_gemv_f32", "q3_gemv_f16", 4096, 4096, target);
  bench_q3("q3_gemv_f32_opt175b", "q3_gemv_f16_opt175b", 49152, 12288, target);
  {  // kQuantize, 16 Mi fp32 values (quantBnB-cuda/main.cu:137-176)
    const int n = 1 << 24;
    const int R = replicas_for((double)n * 4, target);
    std::vector<float*> As(R);
    for (int i = 0; i < R; i++) As[i] = (float*)filled(n, 1, -3.f, 3.f, 200 + i);
    // any sorted table in [-1, 1] exercises the same search; the values do not
    // change the instruction stream
    std::vector<float> code(256);
    for (int i = 0; i < 256; i++) code[i] = -1.f + 2.f * i / 255.f;
    float* dcode = (float*)dmalloc(1024);
    CK(cudaMemcpy(dcode, code.data(), 1024, cudaMemcpyHostToDevice));
    uint8_t* out = (uint8_t*)dmalloc(n);
    emit("bnb_quantize",
         time_launches(R, 20, [&](int i) { ref_bnb_quantize_gpu(dcode, As[i], out, n); }));
    free_all();
  }
  {  // LUT-GEMM 12288 x 12288, 3 bit planes, group 128, with bias
    const int M = 12288, K = 12288, nb = 3, gs = 128, G = K / gs;
    const size_t words = (size_t)(K / 32) * nb * M;
    const int R = replicas_for((double)words * 4, target);
    std::vector<unsigned*> bW(R);
    for (int i = 0; i < R; i++) bW[i] = (unsigned*)filled(words, 0, 0, 0, 300 + i);
    __half* alpha = (__half*)filled((size_t)G * nb * M, 2, 0.001f, 0.05f, 5);
    __half* qb = (__half*)filled((size_t)G * M, 2, -0.02f, 0.02f, 6);
    __half* x = (__half*)filled(K, 2, -1.f, 1.f, 7);
    __half* out = (__half*)dmalloc((size_t)M * 2);
    emit("lutgemm", time_launches(R, 20, [&](int i) {
           ref_lutgemm_matmul(out, x, bW[i], alpha, qb, M, K, nb, G);
         }));
    free_all();
  }
  {  // AQLM 1x16, 4096 x 4096, one codebook
    const int m = 4096, k = 4096;
    const size_t ncodes = (size_t)m * k / 8;
    const int R = replicas_for((double)ncodes * 2, target);
    std::vector<void*> codes(R);
    for (int i = 0; i < R; i++) codes[i] = filled(ncodes / 2, 0, 0, 0, 400 + i);
    __half* cb = (__half*)filled((size_t)65536 * 8, 2, -0.05f, 0.05f, 8);
    __half* x = (__half*)filled(k, 2, -1.f, 1.f, 9);
    __half* out = (__half*)dmalloc((size_t)m * 2);
    const int sizes[4] = {m, m, m, 1 << 30};
    emit("aqlm_1x16", time_launches(R, 20, [&](int i) {
           ref_aqlm_1x16(codes[i], x, out, cb, m, k, sizes, 65536);
         }));
    free_all();
  }
  for (int bits = 8; bits >= 4; bits -= 4) {
    // gemv, square 8192 x 8192; block shapes: the driver's default 32 x 4
    // (gemv-cuda/main.cu:33-34) and 256 x 4 (both satisfy the launchers' asserts);
    // the faster of the two is reported
    const unsigned size = 8192;
    const size_t bytes = (size_t)size * size * bits / 8;
    const int R = replicas_for((double)bytes, target);
    std::vector<void*> mats(R);
    for (int i = 0; i < R; i++) mats[i] = filled(bytes / 4, 0, 0, 0, 500 + 10 * bits + i);
    __half* x = (__half*)filled(size, 2, 0.f, 1.f, 11);
    __half* out = (__half*)dmalloc((size_t)size * 2);
    Result best{1e30, false, R};
    for (unsigned bx : {32u, 256u}) {
      const Result r = time_launches(R, 20, [&](int i) {
        if (bits == 8) ref_gemv_int8((int8_t*)mats[i], x, out, size, 0.0625f, 0.01f, bx, 4);
        else ref_gemv_int4((uint8_t*)mats[i], x, out, size, 0.0625f, 0.01f, bx, 4);
      });
      if (r.us < best.us) best = r;
    }
    emit(bits == 8 ? "gemv_int8" : "gemv_int4", best);
    free_all();
  }
  {  // MXFP4 quantize-dequantize, 2^26 fp16 values per launch (128 MB in, 128 MB out)
    const int numel = 1 << 26;
    const int R = replicas_for((double)numel * 2, target);
    std::vector<void*> xs(R);
    for (int i = 0; i < R; i++) xs[i] = filled(numel, 2, -6.f, 6.f, 600 + i);
    void* out = dmalloc((size_t)numel * 2);
    emit("mxfp4_qdq_f16", time_launches(R, 20, [&](int i) { ref_mxfp4_qdq(xs[i], out, numel, 0); }));
    free_all();
  }
  {  // zero point, 2^24 channels (the driver's own run has 10^7, zeropoint-cuda/Makefile:56)
    const int size = 1 << 24;
    const int R = replicas_for((double)size * 8, target);
    std::vector<void*> lo(R), hi(R);
    for (int i = 0; i < R; i++) {
      lo[i] = filled(size, 1, -1.f, 1.f, 700 + i);
      hi[i] = filled(size, 1, -1.f, 1.f, 800 + i);
    }
    float* sc = (float*)dmalloc((size_t)size * 4);
    int32_t* zp = (int32_t*)dmalloc((size_t)size * 4);
    emit("zero_point", time_launches(R, 20, [&](int i) {
           ref_zero_point_gpu((float*)lo[i], (float*)hi[i], -127, 127, size, 1, sc, zp);
         }));
    free_all();
  }
  printf("}\n");
  return 0;
}
