// Rotary position embedding on a stick image, head_dim = 128 (two sticks per head).
//
// For x[rows, heads*128] with rows = batch*seq, and cos/sin[seq, 128]:
//     y = x * cos + rotate_half(x) * sin,   rotate_half(x) = cat(-x[64:], x[:64])
// per head, i.e. the two sticks of a head trade places (one negated) in the second term.
// Each product and the sum are rounded to fp16 in that order, as eager fp16 does.  In the
// reference this would be a chain of mul / neg / slice / cat / add device programs
// (torch_spyre/_inductor/opfuncs.py:49-72, codegen/data_ops.py:490-630).
#include <algorithm>

#include "common.cuh"

namespace tsb {
namespace {

__global__ void __launch_bounds__(256)
rotary_kernel(const __half* __restrict__ x, const __half* __restrict__ cs, const __half* __restrict__ sn,
              __half* __restrict__ y, uint32_t rows, uint32_t seq, uint32_t heads) {
  // one thread: the same 16-byte lane vector of a head's low and high stick
  const int64_t total = (int64_t)rows * heads * 8;
  const int64_t stick_stride = (int64_t)rows * kStickHalfs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t lv = (uint32_t)(i & 7);
    const int64_t rh = i >> 3;
    const uint32_t row = (uint32_t)(rh % rows), h = (uint32_t)(rh / rows);
    const uint32_t pos = row % seq;
    const int64_t lo = (int64_t)(2 * h) * stick_stride + (int64_t)row * kStickHalfs + lv * 8;
    const int64_t hi = lo + stick_stride;
    const int64_t tlo = (int64_t)pos * kStickHalfs + lv * 8, thi = tlo + (int64_t)seq * kStickHalfs;
    Vec8h xl, xh, cl, ch, sl, sh, yl, yh;
    xl.u = ld_stream_v4(x + lo);
    xh.u = ld_stream_v4(x + hi);
    cl.u = ld_global_v4(cs + tlo);
    ch.u = ld_global_v4(cs + thi);
    sl.u = ld_global_v4(sn + tlo);
    sh.u = ld_global_v4(sn + thi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      yl.h2[j] = __hadd2(__hmul2(xl.h2[j], cl.h2[j]), __hmul2(__hneg2(xh.h2[j]), sl.h2[j]));
      yh.h2[j] = __hadd2(__hmul2(xh.h2[j], ch.h2[j]), __hmul2(xl.h2[j], sh.h2[j]));
    }
    st_global_v4(y + lo, yl.u);
    st_global_v4(y + hi, yh.u);
  }
}

}  // namespace
}  // namespace tsb

extern "C" int ts_rotary_f16(const void* x, const void* cos_table, const void* sin_table, void* y,
                             int64_t batch, int64_t seq, int64_t heads, int64_t head_dim,
                             void* stream) {
  using namespace tsb;
  if (batch < 0 || seq < 0 || heads < 0) return TS_ERR_INVALID;
  if (head_dim != 128) return TS_ERR_UNSUPPORTED;
  if (batch == 0 || seq == 0 || heads == 0) return TS_OK;
  if (!x || !y || !cos_table || !sin_table) return TS_ERR_INVALID;
  if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)cos_table | (uintptr_t)sin_table) % 16) return TS_ERR_ALIGNMENT;
  const int64_t rows = batch * seq;
  if (rows >= (1ll << 31) || heads >= (1 << 20)) return TS_ERR_TOO_LARGE;
  const int64_t total = rows * heads * 8;
  const uint32_t blocks = (uint32_t)std::min<int64_t>(ceil_div(total, 256), 148 * 16);
  rotary_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __half*)x, (const __half*)cos_table,
                                                          (const __half*)sin_table, (__half*)y,
                                                          (uint32_t)rows, (uint32_t)seq, (uint32_t)heads);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}
