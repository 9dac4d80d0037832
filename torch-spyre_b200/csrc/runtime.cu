// Status text and version of the C ABI.
#include "common.cuh"

namespace {
thread_local char g_last_cuda_error[256] = "";
}

namespace tsb {
void note_cuda_error(cudaError_t e) {
  const char* s = cudaGetErrorString(e);
  int i = 0;
  for (; s && s[i] && i < 255; ++i) g_last_cuda_error[i] = s[i];
  g_last_cuda_error[i] = 0;
}
}  // namespace tsb

extern "C" const char* ts_status_string(int status) {
  switch (status) {
    case TS_OK: return "ok";
    case TS_ERR_INVALID: return "invalid argument";
    case TS_ERR_UNSUPPORTED: return "unsupported request";
    case TS_ERR_CUDA: return "CUDA call or kernel launch failed";
    case TS_ERR_ALIGNMENT: return "pointer or stride is not aligned as required";
    case TS_ERR_TOO_LARGE: return "size exceeds the supported maximum";
    default: return "unknown status";
  }
}

extern "C" int ts_abi_version(void) { return 1; }

extern "C" const char* ts_last_cuda_error(void) { return g_last_cuda_error; }

// 2-D device-to-device copy on `stream`; either side may be a peer GPU's memory reachable from
// this device (an address obtained through CUDA IPC or symmetric memory).  `height` pieces of
// `width` bytes, `spitch` / `dpitch` bytes apart: a block of rows of a stick image is one such
// piece per stick column, which is how the tensor-parallel layer gathers its activations.
extern "C" int ts_peer_copy_2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width,
                               int64_t height, void* stream) {
  if (width < 0 || height < 0 || dpitch < width || spitch < width) return TS_ERR_INVALID;
  if (width == 0 || height == 0) return TS_OK;
  if (!dst || !src) return TS_ERR_INVALID;
  const cudaError_t e = cudaMemcpy2DAsync(dst, (size_t)dpitch, src, (size_t)spitch, (size_t)width, (size_t)height,
                                          cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    tsb::note_cuda_error(e);
    return TS_ERR_CUDA;
  }
  return TS_OK;
}

namespace tsb {
namespace {
// out = residual + sum over slots of slot[s], eight fp16 at a time, summed in fp32 and rounded once.
// Grid-stride over 16-byte vectors; the slots are equally spaced images of the same shape.
__global__ void __launch_bounds__(256) sum_slots_kernel(const uint4* __restrict__ slots, int n_slots,
                                                        int64_t slot_vecs, const uint4* __restrict__ residual,
                                                        uint4* __restrict__ out, int64_t n_vecs) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vecs; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8];
    Vec8h v;
    if (residual) {
      v.u = ld_stream_v4(residual + i);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(v.h2[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    }
    for (int s = 0; s < n_slots; ++s) {
      v.u = ld_stream_v4(slots + (int64_t)s * slot_vecs + i);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(v.h2[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) v.h2[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
    st_stream_v4(out + i, v.u);
  }
}
}  // namespace
}  // namespace tsb

// The local half of a reduce-scatter done with plain peer stores (ts_gemm_f16_scatter_store):
// `n_slots` fp16 stick images of one shape, `slot_stride` elements apart (one per rank that wrote
// a partial product into this GPU's memory), are summed in fp32, the optional `residual` image
// added, and the result rounded to fp16 once.  `n` elements per image, a multiple of 8 (whole
// sticks always are); every pointer 16-byte aligned.
extern "C" int ts_sum_slots_f16(const void* slots, int n_slots, int64_t slot_stride, const void* residual,
                                void* out, int64_t n, void* stream) {
  if (n < 0 || n_slots < 1 || n_slots > 64 || slot_stride < n) return TS_ERR_INVALID;
  if (n == 0) return TS_OK;
  if (!slots || !out) return TS_ERR_INVALID;
  if (n % 8 || slot_stride % 8) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)slots | (uintptr_t)out | (uintptr_t)residual) % 16) return TS_ERR_ALIGNMENT;
  const int64_t vecs = n / 8;
  const int64_t blocks = (vecs + 255) / 256;
  const int grid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
  tsb::sum_slots_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)slots, n_slots, slot_stride / 8,
                                                              (const uint4*)residual, (uint4*)out, vecs);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}
