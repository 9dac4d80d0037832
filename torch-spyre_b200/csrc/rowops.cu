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

enum RowOp { kSoftmax = 0, kLogSoftmax = 1, kLayerNorm = 2, kRmsNorm = 3, kCausalSoftmax = 4 };

struct RowParams {
  const __half* x;
  __half* y;
  const __half* weight;  // [cols] or null
  const __half* bias;    // [cols] or null
  uint32_t rows, cols, nsticks;
  int ws_log;
  float eps;
  int round_before_weight;
  // causal softmax: row r attends to columns 0 .. (r % period) of scale * x
  uint32_t period;
  float scale;
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

__device__ __forceinline__ float ex2_f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// FULL: every (row, stick) a thread is assigned exists and cols is a stick multiple,
// so no load, store or reduction needs a predicate.
template <int K, int OP, bool FULL>
__global__ void __launch_bounds__(kThreads) row_kernel(const __grid_constant__ RowParams P) {
  __shared__ float part[kWarps][4];
  grid_dependency_wait();
  grid_release_dependents();
  constexpr bool kSoft = OP == kSoftmax || OP == kLogSoftmax || OP == kCausalSoftmax;
  constexpr bool kCausal = OP == kCausalSoftmax;
  constexpr float kLog2e = 1.4426950408889634f;
  RowCtx c;
  c.lane = threadIdx.x & 31;
  c.warp = threadIdx.x >> 5;
  c.ws = 1 << P.ws_log;
  c.ws_idx = c.warp & (c.ws - 1);
  c.rsub = c.lane >> 3;
  const uint32_t group = blockIdx.x * (kWarps >> P.ws_log) + (c.warp >> P.ws_log);
  c.row = group * 4 + c.rsub;
  c.live = FULL || c.row < P.rows;
  const uint32_t lv = c.lane & 7;
  const bool ragged = !FULL && (P.cols & 63) != 0;
  const int64_t row_off = (int64_t)c.row * kStickHalfs + lv * 8;
  const int64_t stick_stride = (int64_t)P.rows * kStickHalfs;

  const uint32_t qpos = kCausal ? c.row % P.period : 0u;  // last column this row may see
  Vec8h raw[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const uint32_t s = c.ws_idx + k * c.ws;
    bool have = FULL || (c.live && s < P.nsticks);
    if (kCausal) have = have && s * 64 <= qpos;           // sticks wholly above the diagonal are not read
    raw[k].u = make_uint4(0, 0, 0, 0);
    if (have) raw[k].u = ld_stream_v4(P.x + s * stick_stride + row_off);
    if (kCausal) {
      const __half ninf = __ushort_as_half((unsigned short)0xFC00);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (!have || s * 64 + lv * 8 + e > qpos) raw[k].h[e] = ninf;
    } else if (!FULL) {
      const __half fill = kSoft ? __ushort_as_half((unsigned short)0xFC00) : __float2half(0.f);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (!have || (ragged && s * 64 + lv * 8 + e >= P.cols)) raw[k].h[e] = fill;
    }
  }

  float v[K][8];
  const float inv_n = 1.f / (float)P.cols;
  float shift = 0.f, scale = 1.f, lse = 0.f;
  if (kSoft) {
    __half2 m2 = raw[0].h2[0];
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, raw[k].h2[j]);
    float m = fmaxf(__low2float(m2), __high2float(m2));
    m = row_allreduce<true>(m, c, part);
    const float kmul = kCausal ? P.scale * kLog2e : kLog2e;   // scale > 0: max commutes with it
    const float ml = m * kmul;
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(raw[k].h2[j]);
        const float e0 = ex2_f(fmaf(f.x, kmul, -ml)), e1 = ex2_f(fmaf(f.y, kmul, -ml));
        sum += e0 + e1;
        if (OP == kSoftmax || OP == kCausalSoftmax) {
          // keep exp(x - max) packed in fp16 in place of x: half the registers of an fp32
          // copy, hence twice the resident warps; costs one extra fp16 rounding (the result
          // is within 1 ulp of rounding once)
          raw[k].h2[j] = __floats2half2_rn(e0, e1);
        } else {
          v[k][2 * j] = f.x - m;
          v[k][2 * j + 1] = f.y - m;
        }
      }
    sum = row_allreduce<false>(sum, c, part);
    scale = __fdividef(1.f, sum);
    lse = __logf(sum);
  } else {
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(raw[k].h2[j]);
        v[k][2 * j] = f.x;
        v[k][2 * j + 1] = f.y;
      }
    if (OP == kLayerNorm) {
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
          const bool valid = FULL || (s < P.nsticks && (!ragged || s * 64 + lv * 8 + e < P.cols));
          const float d = valid ? v[k][e] - shift : 0.f;
          v[k][e] = d;
          sq = fmaf(d, d, sq);
        }
      }
      scale = rsqrtf(row_allreduce<false>(sq, c, part) * inv_n + P.eps);
    } else {  // RMS norm
      float sq = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) sq = fmaf(v[k][e], v[k][e], sq);
      scale = rsqrtf(row_allreduce<false>(sq, c, part) * inv_n + P.eps);
    }
  }

#pragma unroll
  for (int k = 0; k < K; ++k) {
    const uint32_t s = c.ws_idx + k * c.ws;
    if (!FULL && !(c.live && s < P.nsticks)) continue;
    const uint32_t col = s * 64 + lv * 8;
    Vec8h w, b, out;
    w.u = b.u = make_uint4(0, 0, 0, 0);
    if (OP == kLayerNorm || OP == kRmsNorm) {
      if (P.weight) w.u = ld_global_v4(P.weight + col);
      if (P.bias) b.u = ld_global_v4(P.bias + col);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float r0, r1;
      if (OP == kSoftmax || OP == kCausalSoftmax) {
        const float2 e = __half22float2(raw[k].h2[j]);
        r0 = e.x * scale;
        r1 = e.y * scale;
      } else if (OP == kLogSoftmax) {
        r0 = v[k][2 * j] - lse;
        r1 = v[k][2 * j + 1] - lse;
      } else {
        r0 = v[k][2 * j] * scale;      // layer norm: v already holds x - mean
        r1 = v[k][2 * j + 1] * scale;
      }
      __half2 h;
      if (OP == kLayerNorm) {
        const float2 wf = __half22float2(w.h2[j]), bf = __half22float2(b.h2[j]);
        if (P.weight) { r0 *= wf.x; r1 *= wf.y; }
        if (P.bias) { r0 += bf.x; r1 += bf.y; }
        h = __floats2half2_rn(r0, r1);
      } else if (OP == kRmsNorm) {
        if (P.weight && P.round_before_weight) {
          h = __hmul2(w.h2[j], __floats2half2_rn(r0, r1));
        } else {
          const float2 wf = __half22float2(w.h2[j]);
          h = P.weight ? __floats2half2_rn(r0 * wf.x, r1 * wf.y) : __floats2half2_rn(r0, r1);
        }
      } else {
        h = __floats2half2_rn(r0, r1);
      }
      out.h2[j] = h;
    }
    if (ragged) {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (col + e >= P.cols) out.h[e] = __float2half(0.f);
    }
    st_global_v4(P.y + s * stick_stride + row_off, out.u);
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
  const bool full = P.cols % 64 == 0 && P.nsticks % (1u << ws_log) == 0 &&
                    P.rows % (4 * (kWarps >> ws_log)) == 0;
#define TSB_ROW_CASE(KK)                                                        \
  if (full && per_thread == KK) launch_after_tail(row_kernel<KK, OP, true>, blocks, kThreads, 0, st, P); \
  else launch_after_tail(row_kernel<KK, OP, false>, blocks, kThreads, 0, st, P)
  if (per_thread <= 1) { TSB_ROW_CASE(1); }
  else if (per_thread <= 2) { TSB_ROW_CASE(2); }
  else if (per_thread <= 4) { TSB_ROW_CASE(4); }
  else if (per_thread <= 8) { TSB_ROW_CASE(8); }
  else if (per_thread <= 16) { TSB_ROW_CASE(16); }
  else return TS_ERR_TOO_LARGE;
#undef TSB_ROW_CASE
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

extern "C" int ts_softmax_rows_causal(const void* x, void* y, int64_t rows, int64_t cols,
                                      int64_t period, float scale, void* stream) {
  RowParams P;
  const int rc = check_rows(x, y, rows, cols, P);
  if (rc != TS_OK) return rc > 0 ? TS_OK : rc;
  if (period < 1 || period > cols || !(scale > 0.f)) return TS_ERR_INVALID;
  P.period = (uint32_t)period;
  P.scale = scale;
  return launch_rows<kCausalSoftmax>(P, (cudaStream_t)stream);
}
