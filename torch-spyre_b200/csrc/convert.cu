// Element type conversion between stick images (fp16 / bf16 / fp32), on the device.
//
// The reference refuses a converting copy_ (torch_spyre/csrc/spyre_mem.cpp:669-671) and leaves
// `.to(dtype)` to a host round trip; here `_to_copy` with a dtype change stays on the device.
// The two images differ in more than the element type: a stick is 128 bytes, so it holds 64
// 2-byte or 32 4-byte lanes, and the image of [rows, cols] is [ceil(cols/L)][rows][L] with L the
// lanes of its own type.  A thread converts 8 consecutive columns, which lie inside one stick on
// both sides.
#include <cuda_bf16.h>

#include "common.cuh"

namespace tsb {
namespace {

template <class T> struct Lanes { static constexpr int v = kStickBytes / (int)sizeof(T); };

template <class T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

template <class S, class D>
__global__ void __launch_bounds__(256)
convert_kernel(const S* __restrict__ src, D* __restrict__ dst, uint32_t rows, uint32_t cols,
               uint32_t dst_sticks) {
  constexpr uint32_t LS = Lanes<S>::v, LD = Lanes<D>::v, G = LD / 8;   // groups of 8 per destination stick
  const uint64_t total = (uint64_t)dst_sticks * rows * G;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t gi = (uint32_t)(i % G);
    const uint64_t sr = i / G;                 // destination stick * rows + row
    const uint32_t r = (uint32_t)(sr % rows), stick = (uint32_t)(sr / rows);
    const uint32_t c0 = stick * LD + gi * 8;
    const S* sp = src + ((uint64_t)(c0 / LS) * rows + r) * LS + c0 % LS;
    D out[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = from_f32<D>(c0 + e < cols ? to_f32<S>(sp[e]) : 0.f);
    D* dp = dst + i * 8;                       // the destination image in its own order
    if (sizeof(D) == 2) {
      *reinterpret_cast<uint4*>(dp) = *reinterpret_cast<const uint4*>(out);
    } else {
      reinterpret_cast<uint4*>(dp)[0] = reinterpret_cast<const uint4*>(out)[0];
      reinterpret_cast<uint4*>(dp)[1] = reinterpret_cast<const uint4*>(out)[1];
    }
  }
}

template <class S, class D>
int launch(const void* src, void* dst, int64_t rows, int64_t cols, cudaStream_t st) {
  const int64_t sticks = ceil_div(cols, (int64_t)Lanes<D>::v);
  const int64_t total = sticks * rows * (Lanes<D>::v / 8);
  const int64_t blocks = std::min<int64_t>(ceil_div(total, 256), 148 * 16);
  convert_kernel<S, D><<<(uint32_t)blocks, 256, 0, st>>>((const S*)src, (D*)dst, (uint32_t)rows,
                                                         (uint32_t)cols, (uint32_t)sticks);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int ts_convert_sticks(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t rows,
                                 int64_t cols, void* stream) {
  if (rows < 0 || cols < 0) return TS_ERR_INVALID;
  if (src_dtype < 0 || src_dtype > 2 || dst_dtype < 0 || dst_dtype > 2) return TS_ERR_UNSUPPORTED;
  if (rows == 0 || cols == 0) return TS_OK;
  if (!src || !dst) return TS_ERR_INVALID;
  if (((uintptr_t)src | (uintptr_t)dst) % 128) return TS_ERR_ALIGNMENT;
  if (rows >= (1ll << 31) || cols >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (src_dtype * 3 + dst_dtype) {
    case 0: return launch<__half, __half>(src, dst, rows, cols, st);
    case 1: return launch<__half, __nv_bfloat16>(src, dst, rows, cols, st);
    case 2: return launch<__half, float>(src, dst, rows, cols, st);
    case 3: return launch<__nv_bfloat16, __half>(src, dst, rows, cols, st);
    case 4: return launch<__nv_bfloat16, __nv_bfloat16>(src, dst, rows, cols, st);
    case 5: return launch<__nv_bfloat16, float>(src, dst, rows, cols, st);
    case 6: return launch<float, __half>(src, dst, rows, cols, st);
    case 7: return launch<float, __nv_bfloat16>(src, dst, rows, cols, st);
    default: return launch<float, float>(src, dst, rows, cols, st);
  }
}
