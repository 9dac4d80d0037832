// Row-wise normalisations over stick images: softmax, layer norm and RMS norm along
// the innermost (stick) dim, one pass over HBM with the row held in registers.
//
// They replace, on the reference side, the sendnn Softmax graph of the eager
// wrapper (codegen/inputs/Metadata.yaml:275-277), the five kernels Inductor's
// softmax decomposition becomes once fusion is off (torch_spyre/_inductor/
// __init__.py:81-84) and the exx2 -> layernormscale -> layernormnorm chain
// (torch_spyre/_inductor/decompositions.py:26-36, lowering.py:78-153).
//
// Work split: the image of a [rows, cols] tensor is [cols/64][rows][64].  A warp
// covers 4 adjacent rows x 8 vector lanes, i.e. 512 contiguous bytes of one stick
// column; WS warps share a row group and take stick columns WS apart; a thread
// keeps up to K 16-byte vectors of its row.  Row statistics are reduced with
// shuffles across the 8 lanes and through shared memory across the WS warps.
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;

enum RowOp { kSoftmax = 0, kLogSoftmax = 1, kLayerNorm = 2, kRmsNorm = 3 };

struct RowParams {
  const __half* x;
  __half* y;
  const __half* weight;  // [cols] or null
  const __half* bias;    // [cols] or null
  uint32_t rows, cols, nsticks;
  int ws_log;
  float eps;
  int round_before_weight;
};

struct RowCtx {
  int lane, warp, ws, ws_idx, rsub;  // rsub: row within the warp's group of 4
  uint32_t row;
  bool live;
};

// Sum (or max) over every thread that holds a piece of the same row.
template <bool IS_MAX>
__device__ __forceinline__ float row_allreduce(float v, const RowCtx& c, float (*part)[4]) {
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, other) : v + other;
  }
  if (c.ws == 1) return v;
  if ((c.lane & 7) == 0) part[c.warp][c.rsub] = v;
  __syncthreads();
  const int first = c.warp - c.ws_idx;
  float total = part[first][c.rsub];
  for (int k = 1; k < c.ws; ++k) {
    const float other = part[first + k][c.rsub];
    total = IS_MAX ? fmaxf(total, other) : total + other;
  }
  __syncthreads();
  return total;
}

template <int K, int OP>
__global__ void __launch_bounds__(kThreads) row_kernel(const __grid_constant__ RowParams P) {
  __shared__ float part[kWarps][4];
  RowCtx c;
  c.lane = threadIdx.x & 31;
  c.warp = threadIdx.x >> 5;
  c.ws = 1 << P.ws_log;
  c.ws_idx = c.warp & (c.ws - 1);
  c.rsub = c.lane >> 3;
  const uint32_t group = blockIdx.x * (kWarps >> P.ws_log) + (c.warp >> P.ws_log);
  c.row = group * 4 + c.rsub;
  c.live = c.row < P.rows;
  const uint32_t lv = c.lane & 7;
  const bool ragged = (P.cols & 63) != 0;

  float v[K][8];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const uint32_t s = c.ws_idx + k * c.ws;
    const bool have = c.live && s < P.nsticks;
    Vec8h t;
    t.u = make_uint4(0, 0, 0, 0);
    if (have) t.u = ld_stream_v4(P.x + ((int64_t)s * P.rows + c.row) * kStickHalfs + lv * 8);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const bool valid = have && (!ragged || s * 64 + lv * 8 + e < P.cols);
      const float f = __half2float(t.h[e]);
      v[k][e] = valid ? f : ((OP == kSoftmax || OP == kLogSoftmax) ? -INFINITY : 0.f);
    }
  }

  const float inv_n = 1.f / (float)P.cols;
  float shift = 0.f, scale = 1.f, lse = 0.f;
  if (OP == kSoftmax || OP == kLogSoftmax) {
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int e = 0; e < 8; ++e) m = fmaxf(m, v[k][e]);
    m = row_allreduce<true>(m, c, part);
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = v[k][e] - m;
        if (OP == kSoftmax) {
          v[k][e] = __expf(d);
          sum += v[k][e];
        } else {
          v[k][e] = d;
          sum += __expf(d);
        }
      }
    sum = row_allreduce<false>(sum, c, part);
    scale = __fdividef(1.f, sum);
    lse = __logf(sum);
  } else if (OP == kLayerNorm) {
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += v[k][e];
    shift = row_allreduce<false>(sum, c, part) * inv_n;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const uint32_t s = c.ws_idx + k * c.ws;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const bool valid = s < P.nsticks && (!ragged || s * 64 + lv * 8 + e < P.cols);
        const float d = valid ? v[k][e] - shift : 0.f;
        sq += d * d;
      }
    }
    scale = rsqrtf(row_allreduce<false>(sq, c, part) * inv_n + P.eps);
  } else {  // RMS norm
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += v[k][e] * v[k][e];
    scale = rsqrtf(row_allreduce<false>(sq, c, part) * inv_n + P.eps);
  }

#pragma unroll
  for (int k = 0; k < K; ++k) {
    const uint32_t s = c.ws_idx + k * c.ws;
    if (!(c.live && s < P.nsticks)) continue;
    const uint32_t col = s * 64 + lv * 8;
    Vec8h w, b, out;
    w.u = b.u = make_uint4(0, 0, 0, 0);
    if (OP == kLayerNorm || OP == kRmsNorm) {
      if (P.weight) w.u = ld_global_v4(P.weight + col);
      if (P.bias) b.u = ld_global_v4(P.bias + col);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float r;
      if (OP == kSoftmax) r = v[k][e] * scale;
      else if (OP == kLogSoftmax) r = v[k][e] - lse;
      else r = (v[k][e] - shift) * scale;
      __half h;
      if (OP == kLayerNorm) {
        if (P.weight) r *= __half2float(w.h[e]);
        if (P.bias) r += __half2float(b.h[e]);
        h = __float2half_rn(r);
      } else if (OP == kRmsNorm) {
        if (P.weight && P.round_before_weight) h = __hmul(w.h[e], __float2half_rn(r));
        else h = __float2half_rn(P.weight ? r * __half2float(w.h[e]) : r);
      } else {
        h = __float2half_rn(r);
      }
      if (ragged && col + e >= P.cols) h = __float2half(0.f);
      out.h[e] = h;
    }
    st_global_v4(P.y + ((int64_t)s * P.rows + c.row) * kStickHalfs + lv * 8, out.u);
  }
}

template <int OP>
int launch_rows(const RowParams& P0, cudaStream_t st) {
  RowParams P = P0;
  int ws_log = 3;
  while (ws_log > 0 && (1u << ws_log) > P.nsticks) --ws_log;
  P.ws_log = ws_log;
  const uint32_t per_thread = (uint32_t)ceil_div(P.nsticks, 1 << ws_log);
  const uint32_t groups = (uint32_t)ceil_div(P.rows, 4);
  const uint32_t blocks = (uint32_t)ceil_div(groups, kWarps >> ws_log);
  if (per_thread <= 1) row_kernel<1, OP><<<blocks, kThreads, 0, st>>>(P);
  else if (per_thread <= 2) row_kernel<2, OP><<<blocks, kThreads, 0, st>>>(P);
  else if (per_thread <= 4) row_kernel<4, OP><<<blocks, kThreads, 0, st>>>(P);
  else if (per_thread <= 8) row_kernel<8, OP><<<blocks, kThreads, 0, st>>>(P);
  else if (per_thread <= 16) row_kernel<16, OP><<<blocks, kThreads, 0, st>>>(P);
  else return TS_ERR_TOO_LARGE;
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

int check_rows(const void* x, void* y, int64_t rows, int64_t cols, RowParams& P) {
  if (rows < 0 || cols < 0) return TS_ERR_INVALID;
  if (rows == 0 || cols == 0) return 1;  // nothing to do
  if (!x || !y) return TS_ERR_INVALID;
  if (((uintptr_t)x | (uintptr_t)y) % 16) return TS_ERR_ALIGNMENT;
  if (rows >= (1ll << 31) || cols > TS_ROW_MAX_COLS) return TS_ERR_TOO_LARGE;
  P = RowParams{};
  P.x = (const __half*)x;
  P.y = (__half*)y;
  P.rows = (uint32_t)rows;
  P.cols = (uint32_t)cols;
  P.nsticks = (uint32_t)ceil_div(cols, kStickHalfs);
  return TS_OK;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int ts_softmax_rows(const void* x, void* y, int64_t rows, int64_t cols, int log_softmax,
                               void* stream) {
  RowParams P;
  const int rc = check_rows(x, y, rows, cols, P);
  if (rc != TS_OK) return rc > 0 ? TS_OK : rc;
  return log_softmax ? launch_rows<kLogSoftmax>(P, (cudaStream_t)stream)
                     : launch_rows<kSoftmax>(P, (cudaStream_t)stream);
}

extern "C" int ts_layernorm_rows(const void* x, const void* weight, const void* bias, void* y,
                                 int64_t rows, int64_t cols, float eps, void* stream) {
  RowParams P;
  const int rc = check_rows(x, y, rows, cols, P);
  if (rc != TS_OK) return rc > 0 ? TS_OK : rc;
  if (((uintptr_t)weight | (uintptr_t)bias) % 16) return TS_ERR_ALIGNMENT;
  P.weight = (const __half*)weight;
  P.bias = (const __half*)bias;
  P.eps = eps;
  return launch_rows<kLayerNorm>(P, (cudaStream_t)stream);
}

extern "C" int ts_rmsnorm_rows(const void* x, const void* weight, void* y, int64_t rows,
                               int64_t cols, float eps, int round_before_weight, void* stream) {
  RowParams P;
  const int rc = check_rows(x, y, rows, cols, P);
  if (rc != TS_OK) return rc > 0 ? TS_OK : rc;
  if ((uintptr_t)weight % 16) return TS_ERR_ALIGNMENT;
  P.weight = (const __half*)weight;
  P.eps = eps;
  P.round_before_weight = round_before_weight;
  return launch_rows<kRmsNorm>(P, (cudaStream_t)stream);
}
