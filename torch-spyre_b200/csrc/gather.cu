// Index-driven and scan kernels of the eager op long tail: embedding (row gather), cumsum,
// nearest-neighbour upsampling.  The reference lists them in codegen/inputs/Metadata.yaml
// (embedding -> Gather :105, upsample_nearest2d -> ResizeNearestNeighbor :331) and sends cumsum
// through the host (codegen/inputs/spyre_torch_ops.cpp:501-505); here each is one kernel over
// stick images.
#include <algorithm>

#include "common.cuh"

namespace tsb {
namespace {

__device__ int g_gather_error;   // sticky: an embedding launch met an index outside the table

// out[t, :] = weight[idx[t], :].  weight image [D/64][V][64], out image [D/64][T][64]; indices are
// the stick image of a [T] (or [.., T]-flattened) integer tensor, 128 / IB lanes per stick, or a
// plain array when idx_sticks == 0.  8 threads move one 128-byte stick.
template <class I>
__global__ void __launch_bounds__(256)
embedding_kernel(const __half* __restrict__ weight, const I* __restrict__ idx, __half* __restrict__ out,
                 uint32_t tokens, uint32_t vocab, uint32_t sticks, uint32_t idx_rows, uint32_t idx_cols,
                 int idx_is_image) {
  constexpr uint32_t IL = kStickBytes / (uint32_t)sizeof(I);
  const uint64_t total = (uint64_t)sticks * tokens * 8;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t piece = (uint32_t)(i & 7);
    const uint64_t st = i >> 3;
    const uint32_t t = (uint32_t)(st % tokens), j = (uint32_t)(st / tokens);
    uint64_t ipos = t;
    if (idx_is_image) {   // token t = (row, col) of the [idx_rows, idx_cols] index tensor
      const uint32_t r = t / idx_cols, c = t - r * idx_cols;
      ipos = ((uint64_t)(c / IL) * idx_rows + r) * IL + c % IL;
    }
    const long long v = (long long)idx[ipos];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (v >= 0 && v < (long long)vocab) {
      val = ld_global_v4(weight + ((uint64_t)j * vocab + (uint64_t)v) * kStickHalfs + piece * 8);
    } else if (piece == 0 && j == 0) {
      atomicExch(&g_gather_error, 1);   // reported by ts_gather_error_state; the row is written as zeros
    }
    st_global_v4(out + st * kStickHalfs + piece * 8, val);
  }
}

// Inclusive prefix sum along the middle dim of a contiguous [outer][n][inner] fp16 array, one
// thread per (outer, inner) column, fp32 running sum, every output rounded to fp16.
__global__ void __launch_bounds__(256)
cumsum_mid_kernel(const __half* __restrict__ x, __half* __restrict__ y, uint64_t outer, uint32_t n,
                  uint32_t inner) {
  const uint64_t total = outer * inner;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t o = i / inner, c = i - o * inner;
    const __half* xp = x + o * n * inner + c;
    __half* yp = y + o * n * inner + c;
    float acc = 0.f;
    for (uint32_t k = 0; k < n; ++k) {
      acc += __half2float(xp[(uint64_t)k * inner]);
      yp[(uint64_t)k * inner] = __float2half_rn(acc);
    }
  }
}

// Inclusive prefix sum along the stick dim: image [sticks][rows][64].  One warp per row, two
// lanes of the stick per thread, a shuffle scan inside the stick and a carry from stick to stick.
__global__ void __launch_bounds__(256)
cumsum_rows_kernel(const __half* __restrict__ x, __half* __restrict__ y, uint32_t rows, uint32_t cols,
                   uint32_t sticks) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    float carry = 0.f;
    for (uint32_t j = 0; j < sticks; ++j) {
      const uint64_t at = ((uint64_t)j * rows + r) * kStickHalfs + 2 * lane;
      const __half2 v = *reinterpret_cast<const __half2*>(x + at);
      const uint32_t c = j * kStickHalfs + 2 * lane;
      const float a = c < cols ? __low2float(v) : 0.f, b = c + 1 < cols ? __high2float(v) : 0.f;
      float s = a + b;   // this thread's pair, then an inclusive scan over the 32 pairs
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, s, o);
        if ((int)lane >= o) s += up;
      }
      const float before = carry + s - (a + b);
      const __half2 out = __floats2half2_rn(c < cols ? before + a : 0.f, c + 1 < cols ? before + a + b : 0.f);
      *reinterpret_cast<__half2*>(y + at) = out;
      carry += __shfl_sync(0xffffffffu, s, 31);
    }
  }
}

// out[n, c, oh, ow] = in[n, c, ih(oh), iw(ow)] with the source index floor(dst * in / out) (the
// "nearest" rule of aten::upsample_nearest2d without explicit scales).  Images [W/64][N*C][H][64].
__global__ void __launch_bounds__(256)
upsample_nearest_kernel(const __half* __restrict__ x, __half* __restrict__ y, uint32_t planes, uint32_t ih,
                        uint32_t iw, uint32_t oh, uint32_t ow, float scale_h, float scale_w) {
  const uint32_t osticks = (ow + kStickHalfs - 1) / kStickHalfs;
  const uint64_t total = (uint64_t)osticks * planes * oh * kStickHalfs;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t lane = (uint32_t)(i % kStickHalfs);
    uint64_t rest = i / kStickHalfs;
    const uint32_t y0 = (uint32_t)(rest % oh);
    rest /= oh;
    const uint32_t p = (uint32_t)(rest % planes), j = (uint32_t)(rest / planes);
    const uint32_t x0 = j * kStickHalfs + lane;
    __half v = __float2half(0.f);
    if (x0 < ow) {
      const uint32_t sy = min((uint32_t)floorf(y0 * scale_h), ih - 1), sx = min((uint32_t)floorf(x0 * scale_w), iw - 1);
      v = x[(((uint64_t)(sx / kStickHalfs) * planes + p) * ih + sy) * kStickHalfs + sx % kStickHalfs];
    }
    y[i] = v;
  }
}

uint32_t grid_for(uint64_t total) {
  return (uint32_t)std::min<uint64_t>((total + 255) / 256, 148ull * 16);
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int ts_embedding_rows(const void* weight, const void* indices, int index_bytes, int indices_are_image,
                                 int64_t index_rows, int64_t index_cols, void* out, int64_t vocab,
                                 int64_t dim, void* stream) {
  if (index_rows < 0 || index_cols < 0 || vocab < 0 || dim < 0) return TS_ERR_INVALID;
  if (index_bytes != 4 && index_bytes != 8) return TS_ERR_UNSUPPORTED;
  const int64_t tokens = index_rows * index_cols;
  if (tokens == 0 || dim == 0) return TS_OK;
  if (!weight || !indices || !out) return TS_ERR_INVALID;
  if (((uintptr_t)weight | (uintptr_t)out) % 128 || (uintptr_t)indices % index_bytes) return TS_ERR_ALIGNMENT;
  if (tokens >= (1ll << 31) || vocab >= (1ll << 31) || dim >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  const int64_t sticks = ceil_div(dim, (int64_t)kStickHalfs);
  const uint32_t grid = grid_for((uint64_t)sticks * tokens * 8);
  if (index_bytes == 8)
    embedding_kernel<long long><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __half*)weight, (const long long*)indices, (__half*)out, (uint32_t)tokens, (uint32_t)vocab,
        (uint32_t)sticks, (uint32_t)index_rows, (uint32_t)index_cols, indices_are_image);
  else
    embedding_kernel<int><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __half*)weight, (const int*)indices, (__half*)out, (uint32_t)tokens, (uint32_t)vocab,
        (uint32_t)sticks, (uint32_t)index_rows, (uint32_t)index_cols, indices_are_image);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

// Synchronises the device and reports (and clears) whether an embedding launch met an index
// outside [0, vocab): such rows are written as zeros instead of reading outside the table.
extern "C" int ts_gather_error_state(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gather_error, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gather_error, &zero, sizeof(int));
  }
  return v;
}

extern "C" int ts_cumsum_mid(const void* x, void* y, int64_t outer, int64_t n, int64_t inner, void* stream) {
  if (outer < 0 || n < 0 || inner < 0) return TS_ERR_INVALID;
  if (outer == 0 || n == 0 || inner == 0) return TS_OK;
  if (!x || !y) return TS_ERR_INVALID;
  if (n >= (1ll << 31) || inner >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  cumsum_mid_kernel<<<grid_for((uint64_t)outer * inner), 256, 0, (cudaStream_t)stream>>>(
      (const __half*)x, (__half*)y, (uint64_t)outer, (uint32_t)n, (uint32_t)inner);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

extern "C" int ts_cumsum_rows(const void* x, void* y, int64_t rows, int64_t cols, void* stream) {
  if (rows < 0 || cols < 0) return TS_ERR_INVALID;
  if (rows == 0 || cols == 0) return TS_OK;
  if (!x || !y) return TS_ERR_INVALID;
  if (((uintptr_t)x | (uintptr_t)y) % 4) return TS_ERR_ALIGNMENT;
  if (rows >= (1ll << 31) || cols >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  const uint32_t grid = (uint32_t)std::min<int64_t>(ceil_div(rows, 8), 148 * 16);
  cumsum_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const __half*)x, (__half*)y, (uint32_t)rows, (uint32_t)cols, (uint32_t)ceil_div(cols, (int64_t)kStickHalfs));
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

extern "C" int ts_upsample_nearest2d(const void* x, void* y, int64_t planes, int64_t in_h, int64_t in_w,
                                     int64_t out_h, int64_t out_w, void* stream) {
  if (planes < 0 || in_h < 0 || in_w < 0 || out_h < 0 || out_w < 0) return TS_ERR_INVALID;
  if (planes == 0 || out_h == 0 || out_w == 0) return TS_OK;
  if (in_h == 0 || in_w == 0 || !x || !y) return TS_ERR_INVALID;
  if (planes * out_h >= (1ll << 31) || out_w >= (1ll << 31) || in_w >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  const uint64_t total = (uint64_t)ceil_div(out_w, (int64_t)kStickHalfs) * planes * out_h * kStickHalfs;
  upsample_nearest_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
      (const __half*)x, (__half*)y, (uint32_t)planes, (uint32_t)in_h, (uint32_t)in_w, (uint32_t)out_h,
      (uint32_t)out_w, (float)in_h / (float)out_h, (float)in_w / (float)out_w);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}
