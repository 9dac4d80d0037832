// Host-side construction of TMA tensor maps over stick images.  The driver entry point
// is looked up through the runtime, so the library does not link against libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace tsb {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// Tensor map over a stick image addressed as [heads][sticks][batch][rows][64 lanes] of fp16:
// rows are 128 bytes apart, batch entries rows*128 bytes, stick columns and heads at the given
// element strides.  The box is 64 lanes x box_rows rows of one stick column of one
// (batch, head); 128-byte swizzle.
inline bool make_stick_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t batch,
                           uint64_t sticks, uint64_t heads, int64_t stick_stride,
                           int64_t head_stride, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[5] = {64, rows, batch, sticks, heads};
  // a dim of extent 1 still needs a legal stride (multiple of 16 bytes)
  const cuuint64_t strides[4] = {128, rows * 128, (cuuint64_t)stick_stride * 2,
                                 (cuuint64_t)(heads > 1 ? head_stride : stick_stride) * 2};
  const cuuint32_t box[5] = {64, box_rows, 1, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tsb
