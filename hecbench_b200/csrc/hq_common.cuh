// Shared helpers for the libhq kernels (sm_100a only).
#pragma once

#include <atomic>

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "hq.h"

namespace hq {

// Per-thread record of the last failing CUDA runtime call.
int& last_cuda_error_ref();

inline int cuda_status(cudaError_t e) {
  if (e == cudaSuccess) return HQ_OK;
  last_cuda_error_ref() = (int)e;
  return HQ_ERR_CUDA;
}

// Launch errors are sticky-free: cudaGetLastError clears and returns them.
inline int launch_status() { return cuda_status(cudaGetLastError()); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }
inline bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

// True when the environment variable `name` is set to something other than
// "" or "0" (read at every call: a host may switch between calls).
inline bool env_flag(const char* name) {
  const char* v = getenv(name);
  return v != nullptr && v[0] != '\0' && !(v[0] == '0' && v[1] == '\0');
}

// Number of SMs of the current device (cached per device).
int sm_count();
// Shared memory the system reserves at the start of every CTA's window on the
// current device (cached per device).
int reserved_smem_per_block();

// Raises the dynamic shared-memory limit of kernel Kern to `bytes` once per
// device (and again only if a later call needs more): the attribute call costs
// microseconds of host time, which an eager launch every few microseconds
// cannot afford.  Safe from several host threads: the attribute is idempotent
// and the record only ever grows.
constexpr int kMaxDevices = 64;
template <auto Kern>
inline cudaError_t ensure_dynamic_smem(size_t bytes) {
  static std::atomic<size_t> granted[kMaxDevices];  // zero-initialised, one array per kernel
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  if (tracked && granted[dev].load(std::memory_order_acquire) >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && tracked) granted[dev].store(bytes, std::memory_order_release);
  return e;
}

// Programmatic dependent launch.  A kernel calls pdl_launch_dependents() first
// thing, so that the next kernel of the stream may become resident while this
// grid is still running, and pdl_wait() before it touches global memory that
// earlier work in the stream may still be writing (pdl_wait returns once every
// preceding kernel has completed and its writes are visible; it returns at once
// in a kernel that was launched the ordinary way).  launch_pdl() launches with
// the attribute that allows the early start.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- index-checked build (-DHQ_BOUNDS_CHECK) --------------------------------
// compute-sanitizer may be unavailable where this library is developed, so the
// kernels carry their own bounds checks, compiled in only with
// -DHQ_BOUNDS_CHECK: every global access of an instrumented kernel is tested
// against the extent of its buffer; a violation is RECORDED (count, first
// site, first offset) and the access is SKIPPED - nothing traps, the kernel
// runs to its end, and hq_bounds_check_report returns what was seen.  Each
// translation unit has its own record; hq_capi.cu adds them up.
struct BoundsRecord {
  unsigned violations;
  unsigned site;                // first violating access: 100 * file + access number
  unsigned long long offset;    // its byte offset from the buffer's base (wraps if below)
  unsigned long long extent;    // the buffer's size in bytes
};
#ifdef HQ_BOUNDS_CHECK
static __device__ BoundsRecord g_bounds_rec;
using BoundsAccess = cudaError_t (*)(BoundsRecord*, bool reset);
void register_bounds_access(BoundsAccess fn);  // hq_capi.cu
static cudaError_t bounds_access_this_tu(BoundsRecord* out, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_bounds_rec, sizeof(BoundsRecord));
  if (e == cudaSuccess && reset) {
    const BoundsRecord zero = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(g_bounds_rec, &zero, sizeof(BoundsRecord));
  }
  return e;
}
static const int g_bounds_registered = (register_bounds_access(bounds_access_this_tu), 0);
__device__ __forceinline__ bool in_bounds(const void* p, size_t bytes, const void* base,
                                          size_t extent, unsigned site) {
  const unsigned long long off = (unsigned long long)((const char*)p - (const char*)base);
  if (off <= extent && bytes <= extent - off) return true;
  if (atomicAdd(&g_bounds_rec.violations, 1u) == 0u) {
    g_bounds_rec.site = site;
    g_bounds_rec.offset = off;
    g_bounds_rec.extent = extent;
  }
  return false;
}
#define HQ_IN_BOUNDS(p, bytes, base, extent, site) \
  hq::in_bounds((p), (size_t)(bytes), (base), (size_t)(extent), (site))
#else
#define HQ_IN_BOUNDS(p, bytes, base, extent, site) true
#endif

// Streaming 128-bit load that does not allocate in L1: packed weights are
// read exactly once.
__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(v.x), "=r"(v.y)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Loads of data that an earlier kernel of the stream may have written (the input
// vector of a mat-vec), for kernels launched with programmatic dependent launch:
// they must stay behind griddepcontrol.wait.  A non-coherent load (ld.global.nc,
// which __ldg and const __restrict__ pointers produce) promises that the data is
// read-only for the whole kernel, so the assembler may move it above the wait;
// these are ordinary coherent loads that the compiler may not reorder.
__device__ __forceinline__ uint4 ld_dependent_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_dependent_f32(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ __half ld_dependent_f16(const __half* p) {
  unsigned short v;
  asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return __ushort_as_half(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Gate of a gated linear unit, fp32: HQ_ACT_SWIGLU g * sigmoid(g)
// (swish-cuda/reference.h:4), else HQ_ACT_GEGLU 0.5 g (1 + erf(g / sqrt 2))
// (geglu-cuda/reference.h:1-5).
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == HQ_ACT_SWIGLU) return g / (1.f + expf(-g));
  return 0.5f * g * (1.f + erff(g * 0.70710678118654752440f));
}
__device__ __forceinline__ __half2 u32_as_half2(uint32_t u) {
  return *reinterpret_cast<__half2*>(&u);
}
__device__ __forceinline__ uint32_t half2_as_u32(__half2 h) {
  return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace hq
