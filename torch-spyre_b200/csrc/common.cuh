// Shared helpers for the sm_100a kernels behind the C ABI in include/spyre_b200.h.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/spyre_b200.h"

namespace tsb {

constexpr int kStickBytes = 128;   // torch_spyre/csrc/spyre_tensor_impl.cpp:27
constexpr int kStickHalfs = 64;    // fp16 elements per stick
constexpr int kMaxDims = TS_MAX_DIMS;

// Unsigned 32-bit division by a run-time constant: n / d == (umulhi(n, m) + n) >> s
// for 0 <= n < 2^31 and 1 <= d < 2^31.
struct FastDiv {
  uint32_t d, m, s;
  __host__ void init(uint32_t div) {
    d = div ? div : 1;
    for (s = 0; s < 32; ++s)
      if ((1u << s) >= d) break;
    uint64_t one = 1;
    m = (uint32_t)(((one << 32) * ((one << s) - d)) / d + 1);
  }
  __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
    return (__umulhi(n, m) + n) >> s;
#else
    return (uint32_t)((((uint64_t)n * m) >> 32) + n) >> s;
#endif
  }
  __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
};

__host__ __device__ __forceinline__ int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch ---------------------------------------------------
// A kernel launched with launch_after_tail() may be scheduled onto the SMs while the grid
// before it on the stream is still finishing, so the launch latency and the placement of the
// first CTAs overlap that grid's tail.  Such a kernel calls grid_dependency_wait() before it
// touches global memory: the call returns once the earlier grid has completed and its writes
// are visible, which keeps stream order exactly as without the attribute.  Both calls do
// nothing in a kernel launched the ordinary way, and the launch falls back to ordinary
// stream order after anything that is not a kernel or that never releases its dependents early.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_release_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

#ifdef TSB_TUNING
inline bool tune_pdl_on() {
  const char* e = getenv("TS_PDL");
  return !e || e[0] != '0';
}
#endif

template <class P, class A>
inline cudaError_t launch_after_tail(void (*kernel)(P), uint32_t grid, uint32_t block, size_t smem,
                                     cudaStream_t st, const A& arg) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#ifdef TSB_TUNING
  if (!tune_pdl_on()) cfg.numAttrs = 0;
#endif
  return cudaLaunchKernelEx(&cfg, kernel, arg);
}

inline int launch_status(cudaError_t e) { return e == cudaSuccess ? TS_OK : TS_ERR_CUDA; }

void note_cuda_error(cudaError_t e);  // runtime.cu: remembers the text for ts_last_cuda_error

#define TSB_CHECK_LAUNCH()                          \
  do {                                              \
    cudaError_t e__ = cudaGetLastError();           \
    if (e__ != cudaSuccess) {                       \
      ::tsb::note_cuda_error(e__);                  \
      return TS_ERR_CUDA;                           \
    }                                               \
  } while (0)

// 16-byte global accesses.  The streaming forms keep single-use data from
// displacing reusable lines in L1.
__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_global_v4(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
__device__ __forceinline__ void st_stream_v4(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v, int width = 32) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    if (o < width) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v, int width = 32) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    if (o < width) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

union Vec8h {
  uint4 u;
  __half2 h2[4];
  __half h[8];
};

}  // namespace tsb
