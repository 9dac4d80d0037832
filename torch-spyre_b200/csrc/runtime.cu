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
