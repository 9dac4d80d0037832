// Reductions and softmax along a non-stick dim of a stick image.
//
// Seen from memory, reducing a dim other than the innermost one is a reduction
// over the middle dim of a contiguous [outer][red][inner] fp16 array whose inner
// extent is a whole number of 16-byte vectors (sticks are 128 bytes).  These are
// the "nonstick" reductions of the reference's sfp code generator
// (torch_spyre/_inductor/codegen/compute_ops.py:75-76).
//
// Thread block = TX vector lanes along inner x TY rows along red (TX * TY = 256).
// When outer * inner alone cannot fill the GPU the red extent is also split over
// gridDim.z blocks, which leave fp32 partials in caller-provided scratch for a
// second, small kernel to combine.
#include <algorithm>
#include <atomic>

#include "common.cuh"

namespace tsb {
namespace {

constexpr int kThreads = 256;
constexpr int kTargetBlocks = 148 * 4;

struct MidParams {
  const __half* x;
  __half* y;
  float* scratch;
  uint32_t outer, red, inner_vecs;
  uint32_t tx_log;     // TX = 1 << tx_log lanes along inner
  uint32_t splits;     // blocks along red
  uint32_t red_per_split;
  int op;
  float scale;
  int log_softmax;
};

__device__ __forceinline__ float ident(int op) {
  return op == TS_RED_SUM ? 0.f : (op == TS_RED_MAX ? -INFINITY : INFINITY);
}
__device__ __forceinline__ float comb(int op, float a, float b) {
  if (op == TS_RED_SUM) return a + b;
  if (a != a) return a;
  if (b != b) return b;
  return op == TS_RED_MAX ? fmaxf(a, b) : fminf(a, b);
}

// Combines the per-ty partial vectors of a block; result valid for ty == 0.
__device__ __forceinline__ void block_combine(float (&acc)[8], int op, int tx, int ty, int TX, int TY,
                                              float* smem) {
  // smem layout [ty][e][tx] keeps lanes of a warp on distinct banks.
  for (int stride = TY >> 1; stride > 0; stride >>= 1) {
    if (ty >= stride && ty < 2 * stride) {
#pragma unroll
      for (int e = 0; e < 8; ++e) smem[((ty - stride) * 8 + e) * TX + tx] = acc[e];
    }
    __syncthreads();
    if (ty < stride) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = comb(op, acc[e], smem[(ty * 8 + e) * TX + tx]);
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads) reduce_mid_kernel(const __grid_constant__ MidParams P) {
  __shared__ float smem[kThreads * 8 / 2];
  const int TX = 1 << P.tx_log, TY = kThreads >> P.tx_log;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> P.tx_log;
  const uint32_t iv = blockIdx.x * TX + tx;
  const uint32_t o = blockIdx.y;
  const bool live = iv < P.inner_vecs;
  const uint32_t r_begin = blockIdx.z * P.red_per_split;
  const uint32_t r_end = min(P.red, r_begin + P.red_per_split);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = ident(P.op);
  if (live) {
    const __half* base = P.x + ((int64_t)o * P.red * P.inner_vecs + iv) * 8;
    for (uint32_t r = r_begin + ty; r < r_end; r += TY) {
      Vec8h t;
      t.u = ld_stream_v4(base + (int64_t)r * P.inner_vecs * 8);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = comb(P.op, acc[e], __half2float(t.h[e]));
    }
  }
  block_combine(acc, P.op, tx, ty, TX, TY, smem);
  if (ty != 0 || !live) return;
  if (P.splits == 1) {
    Vec8h out;
#pragma unroll
    for (int e = 0; e < 8; ++e) out.h[e] = __float2half_rn(acc[e] * P.scale);
    st_global_v4(P.y + ((int64_t)o * P.inner_vecs + iv) * 8, out.u);
  } else {
    float* dst = P.scratch + (((int64_t)blockIdx.z * P.outer + o) * P.inner_vecs + iv) * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

__global__ void __launch_bounds__(kThreads) reduce_mid_finish(const __grid_constant__ MidParams P) {
  const int64_t vec = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t nvec = (int64_t)P.outer * P.inner_vecs;
  if (vec >= nvec) return;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = ident(P.op);
  for (uint32_t z = 0; z < P.splits; ++z) {
    const float* src = P.scratch + ((int64_t)z * nvec + vec) * 8;
    const float4 a = *reinterpret_cast<const float4*>(src);
    const float4 b = *reinterpret_cast<const float4*>(src + 4);
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = comb(P.op, acc[e], f[e]);
  }
  Vec8h out;
#pragma unroll
  for (int e = 0; e < 8; ++e) out.h[e] = __float2half_rn(acc[e] * P.scale);
  st_global_v4(P.y + vec * 8, out.u);
}

// Softmax along red: three sweeps over the block's [red][TX vectors] slab (the
// second and third normally hit in L2).
__global__ void __launch_bounds__(kThreads) softmax_mid_kernel(const __grid_constant__ MidParams P) {
  __shared__ float smem[kThreads * 8 / 2];
  __shared__ float bcast[8 * 32];
  const int TX = 1 << P.tx_log, TY = kThreads >> P.tx_log;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> P.tx_log;
  const uint32_t iv = blockIdx.x * TX + tx;
  const uint32_t o = blockIdx.y;
  const bool live = iv < P.inner_vecs;
  const int64_t off0 = ((int64_t)o * P.red * P.inner_vecs + iv) * 8;
  const int64_t rstride = (int64_t)P.inner_vecs * 8;
  float m[8], sum[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { m[e] = -INFINITY; sum[e] = 0.f; }
  if (live)
    for (uint32_t r = ty; r < P.red; r += TY) {
      Vec8h t;
      t.u = ld_global_v4(P.x + off0 + r * rstride);
#pragma unroll
      for (int e = 0; e < 8; ++e) m[e] = fmaxf(m[e], __half2float(t.h[e]));
    }
  block_combine(m, TS_RED_MAX, tx, ty, TX, TY, smem);
  if (ty == 0)
#pragma unroll
    for (int e = 0; e < 8; ++e) bcast[e * 32 + tx] = m[e];
  __syncthreads();
#pragma unroll
  for (int e = 0; e < 8; ++e) m[e] = bcast[e * 32 + tx];
  __syncthreads();
  if (live)
    for (uint32_t r = ty; r < P.red; r += TY) {
      Vec8h t;
      t.u = ld_global_v4(P.x + off0 + r * rstride);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum[e] += __expf(__half2float(t.h[e]) - m[e]);
    }
  block_combine(sum, TS_RED_SUM, tx, ty, TX, TY, smem);
  if (ty == 0)
#pragma unroll
    for (int e = 0; e < 8; ++e) bcast[e * 32 + tx] = sum[e];
  __syncthreads();
#pragma unroll
  for (int e = 0; e < 8; ++e) sum[e] = bcast[e * 32 + tx];
  if (!live) return;
  for (uint32_t r = ty; r < P.red; r += TY) {
    Vec8h t, out;
    t.u = ld_global_v4(P.x + off0 + r * rstride);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float d = __half2float(t.h[e]) - m[e];
      const float v = P.log_softmax ? d - __logf(sum[e]) : __fdividef(__expf(d), sum[e]);
      out.h[e] = __float2half_rn(v);
    }
    st_global_v4(P.y + off0 + r * rstride, out.u);
  }
}

int plan_mid(int64_t outer, int64_t red, int64_t inner, MidParams& P, bool allow_split) {
  if (outer < 0 || red < 0 || inner < 0 || inner % 8) return TS_ERR_INVALID;
  if (outer > 65535 || red >= (1ll << 31) || inner / 8 >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  P = MidParams{};
  P.outer = (uint32_t)outer;
  P.red = (uint32_t)red;
  P.inner_vecs = (uint32_t)(inner / 8);
  uint32_t tx_log = 0;
  while (tx_log < 5 && (1u << tx_log) < P.inner_vecs) ++tx_log;
  P.tx_log = tx_log;
  const int64_t base_blocks = ceil_div(P.inner_vecs, 1 << tx_log) * outer;
  const int64_t TY = kThreads >> tx_log;
  int64_t splits = 1;
  if (allow_split && base_blocks > 0 && base_blocks < kTargetBlocks) {
    splits = std::min<int64_t>(ceil_div(kTargetBlocks, base_blocks), ceil_div(red, TY * 4));
    splits = std::max<int64_t>(1, std::min<int64_t>(splits, 64));
  }
  P.red_per_split = (uint32_t)ceil_div(red, splits);
  P.splits = (uint32_t)ceil_div(red, std::max<uint32_t>(P.red_per_split, 1));
  if (P.splits == 0) P.splits = 1;
  return TS_OK;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int64_t ts_reduce_mid_scratch_bytes(int64_t outer, int64_t red, int64_t inner) {
  MidParams P;
  const int rc = plan_mid(outer, red, inner, P, true);
  if (rc != TS_OK) return rc;
  if (P.splits <= 1) return 0;
  return (int64_t)P.splits * outer * inner * (int64_t)sizeof(float);
}

extern "C" int ts_reduce_mid(const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
                             int reduce_op, float scale, void* scratch, void* stream) {
  if (reduce_op < TS_RED_SUM || reduce_op > TS_RED_MIN) return TS_ERR_INVALID;
  MidParams P;
  const int rc = plan_mid(outer, red, inner, P, true);
  if (rc != TS_OK) return rc;
  if (outer == 0 || inner == 0) return TS_OK;
  if (!x || !y) return TS_ERR_INVALID;
  if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)scratch) % 16) return TS_ERR_ALIGNMENT;
  if (P.splits > 1 && !scratch) return TS_ERR_INVALID;
  P.x = (const __half*)x;
  P.y = (__half*)y;
  P.scratch = (float*)scratch;
  P.op = reduce_op;
  P.scale = scale;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((uint32_t)ceil_div(P.inner_vecs, 1 << P.tx_log), P.outer, P.splits);
  reduce_mid_kernel<<<grid, kThreads, 0, st>>>(P);
  TSB_CHECK_LAUNCH();
  if (P.splits > 1) {
    const int64_t nvec = (int64_t)P.outer * P.inner_vecs;
    reduce_mid_finish<<<(uint32_t)ceil_div(nvec, kThreads), kThreads, 0, st>>>(P);
    TSB_CHECK_LAUNCH();
  }
  return TS_OK;
}

extern "C" int ts_softmax_mid(const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
                              int log_softmax, void* stream) {
  MidParams P;
  const int rc = plan_mid(outer, red, inner, P, false);
  if (rc != TS_OK) return rc;
  if (outer == 0 || inner == 0 || red == 0) return TS_OK;
  if (!x || !y) return TS_ERR_INVALID;
  if (((uintptr_t)x | (uintptr_t)y) % 16) return TS_ERR_ALIGNMENT;
  P.x = (const __half*)x;
  P.y = (__half*)y;
  P.log_softmax = log_softmax;
  dim3 grid((uint32_t)ceil_div(P.inner_vecs, 1 << P.tx_log), P.outer, 1);
  softmax_mid_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(P);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

// ---- ts_reduce_mid for callers that cannot provide scratch ---------------------------
//
// Some users of this library have no way to hand it a scratch buffer: a plug-in that is
// only ever given input and output device pointers by its host application (the
// application owns the device memory and offers the plug-in no allocator), or a caller
// inside a latency-critical loop that must not touch the CUDA allocator because an
// allocation may synchronise the whole device.  For them the split-reduction partials
// live in a fixed array that is part of the library image: every GPU that loads the
// library carries these kReduceStaticBytes until the process exits.
namespace tsb {
namespace {

constexpr size_t kReduceStaticBytes = 512u << 10;  // 512 KiB of fp32 partials
static __device__ __align__(256) unsigned char g_reduce_static_scratch[kReduceStaticBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_reduce_static_ptr[kMaxDevices];  // device address of the array, per GPU

// In host code the array's name is only a handle, not an address the GPU can use; the
// real device address has to be asked for, once per device, with that device current.
int reduce_static_scratch(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TS_ERR_CUDA;
  void* p = g_reduce_static_ptr[dev].load(std::memory_order_acquire);
  if (!p) {
    const cudaError_t e = cudaGetSymbolAddress(&p, g_reduce_static_scratch);
    if (e != cudaSuccess || !p) {
      note_cuda_error(e);
      return TS_ERR_CUDA;
    }
    g_reduce_static_ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return TS_OK;
}

}  // namespace
}  // namespace tsb

extern "C" int ts_reduce_mid_static(const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
                                    int reduce_op, float scale, void* stream) {
  if (reduce_op < TS_RED_SUM || reduce_op > TS_RED_MIN) return TS_ERR_INVALID;
  MidParams P;
  const int rc = plan_mid(outer, red, inner, P, true);
  if (rc != TS_OK) return rc;
  if (outer == 0 || inner == 0) return TS_OK;
  if (!x || !y) return TS_ERR_INVALID;
  if (((uintptr_t)x | (uintptr_t)y) % 16) return TS_ERR_ALIGNMENT;
  const size_t need = P.splits > 1 ? (size_t)P.splits * outer * inner * sizeof(float) : 0;
  if (need > kReduceStaticBytes) return TS_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int src = reduce_static_scratch(&scratch);
  if (src != TS_OK) return src;
  P.x = (const __half*)x;
  P.y = (__half*)y;
  P.scratch = (float*)scratch;
  P.op = reduce_op;
  P.scale = scale;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((uint32_t)ceil_div(P.inner_vecs, 1 << P.tx_log), P.outer, P.splits);
  reduce_mid_kernel<<<grid, kThreads, 0, st>>>(P);
  TSB_CHECK_LAUNCH();
  if (P.splits > 1) {
    const int64_t nvec = (int64_t)P.outer * P.inner_vecs;
    reduce_mid_finish<<<(uint32_t)ceil_div(nvec, kThreads), kThreads, 0, st>>>(P);
    TSB_CHECK_LAUNCH();
  }
  return TS_OK;
}

extern "C" int64_t ts_reduce_mid_static_max_bytes(void) { return (int64_t)tsb::kReduceStaticBytes; }
