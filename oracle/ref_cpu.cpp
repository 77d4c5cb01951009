// Builds the reference's own CPU implementation of the quantBnB path into
// oracle/_ref/libref_cpu.so.  TEST INFRASTRUCTURE ONLY.
//
// The translation unit below is HeCBench's quantBnB-omp/main.cpp, included
// from where it lies (the build passes -I<reference>/src/quantBnB-omp and
// -I<reference>/src/quantBnB-cuda for its code.h); nothing of it is copied.
// Its main() is renamed so the file can live in a shared object; the exports
// call the reference's dQuantize<0> and expose its 256-entry code table.
#include <cstddef>
#include <cstdint>
#include <thread>
#include <vector>

#define main hecbench_quantbnb_omp_main
#include "main.cpp"
#undef main

extern "C" {

const float* ref_bnb_code_table(void) { return code; }

// The loop of quantBnB-omp/main.cpp:105-108 / :120-122 under a host
// parallel-for (the reference's `target teams` construct degenerates to one
// thread team per 256 elements on a host without an offload device).  Built
// without -fopenmp (the reference's pragmas are then ignored) and threaded with
// std::thread, so the library does not depend on a particular OpenMP runtime.
void ref_bnb_quantize(const float* A, uint8_t* out, size_t n, int threads) {
  if (threads < 1) threads = 1;
  std::vector<std::thread> pool;
  const size_t chunk = (n + threads - 1) / threads;
  for (int t = 0; t < threads; t++) {
    const size_t lo = (size_t)t * chunk, hi = lo + chunk < n ? lo + chunk : n;
    if (lo >= hi) break;
    pool.emplace_back([=] {
      for (size_t i = lo; i < hi; i++) out[i] = dQuantize<0>(code, 0.f, A[i]);
    });
  }
  for (auto& th : pool) th.join();
}

}  // extern "C"
