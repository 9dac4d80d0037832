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
