// Reference AQLM 1x16 kernel built from its own source (quantAQLM-cuda/main.cu,
// included from the reference tree with main() renamed).  TEST INFRASTRUCTURE
// ONLY.  The reference driver's main() is never called: it under-allocates its
// output buffer.  Only the kernel is launched, with the launch geometry of
// code1x16_matvec (main.cu:118-128) and a caller-sized output.
#define main hecbench_quantaqlm_cuda_main
#include "main.cu"
#undef main

extern "C" void ref_aqlm_1x16(const void* A, const void* B, void* C, const void* codebook,
                              int prob_m, int prob_k, const int* sizes, int codebook_stride) {
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int waves = 0, thread_m;
  do {
    waves++;
    thread_m = ceildiv(prob_m, waves * sms);
  } while (thread_m > THREAD_M);
  int blocks = ceildiv(prob_m, thread_m);
  int threads = 32 * thread_m;
  const int4 a_sizes = make_int4(sizes[0], sizes[1], sizes[2], sizes[3]);
  Code1x16MatVec<<<blocks, threads, sizeof(int4) * 32 * F, 0>>>(
      (const int4*)A, (const int4*)B, (int4*)C, (const int4*)codebook, prob_m, prob_k, a_sizes,
      codebook_stride);
}
