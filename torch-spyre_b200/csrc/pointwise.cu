// Fused fp16 pointwise chains over stick images, with an optional reduction along
// the stick (innermost) dim.
//
// One kernel evaluates a whole fused group, so a graph such as
// exp(x * a + b).sum(-1) makes a single pass over x.  The reference lowers the
// same graph to one device program per op (fusion is switched off in
// torch_spyre/_inductor/choices.py:58-83) through generate_sfp_op
// (torch_spyre/_inductor/codegen/compute_ops.py:60-393).
//
// The group arrives as a short program for an accumulator machine; the kernel is
// an interpreter whose registers are statically allocated (the accumulator, two
// operand buffers and four saved slots, each 8 fp16 values per work item), so no
// register is ever indexed dynamically and every branch is uniform across the
// grid.  Values are carried as packed half2: add / sub / mul / max / min /
// compares run on the fp16 pipe two at a time, transcendental ops go through
// fp32 and the special-function unit.
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kThreads = 256;
constexpr int U = 2;  // work items (16-byte vectors) per thread per step

struct PwTensorDesc {
  const __half* ptr;
  int64_t stick_stride;  // elements between consecutive stick columns of this tensor
  int32_t m0, m1, m2;    // tensor row = i0*m0 + i1*m1 + i2*m2
  int32_t col_bcast;     // tensor has a single column: its value sits in lane 0
  int32_t flat;          // same shape as the iteration space
};

struct PwParams {
  int n_insns, n_in, n_out;
  ts_pw_insn insn[TS_PW_MAX_INSNS];
  PwTensorDesc in[TS_PW_MAX_INPUTS];
  __half* out[TS_PW_MAX_OUTPUTS];
  uint32_t rows, nsticks, cols, total_sticks;
  FastDiv div_rows, div_d2, div_d1;
  int need_index;  // some input is not flat
  int ragged;      // cols is not a stick multiple
  int red_op, red_keepdim, ws_log;
  float red_scale;
  __half* red_out;
  uint32_t red_inner, red_outer;
  FastDiv div_red_inner;
};

struct Item {
  uint32_t s, r, lv, i0, i1, i2;
  int64_t flat_off;  // element offset in a full-shape stick image
  bool live;
};

using V = __half2[4];

__device__ __forceinline__ void set_all(V& v, __half2 x) {
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = x;
}

__device__ __forceinline__ void load_vec(V& v, const __half* p, bool streaming) {
  Vec8h t;
  t.u = streaming ? ld_stream_v4(p) : ld_global_v4(p);
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = t.h2[j];
}

__device__ __forceinline__ void fetch_tensor(const PwParams& P, int t, const Item& it, V& v) {
  const PwTensorDesc& d = P.in[t];
  if (!it.live) {
    set_all(v, __float2half2_rn(0.f));
    return;
  }
  if (d.flat) {
    load_vec(v, d.ptr + it.flat_off, true);
  } else {
    const int64_t row = (int64_t)it.i0 * d.m0 + (int64_t)it.i1 * d.m1 + (int64_t)it.i2 * d.m2;
    if (!d.col_bcast) {
      load_vec(v, d.ptr + (int64_t)it.s * d.stick_stride + row * kStickHalfs + it.lv * 8, false);
    } else {
      set_all(v, __half2half2(__ldg(d.ptr + row * kStickHalfs)));
    }
  }
}

template <class F>
__device__ __forceinline__ void map_f32(V (&acc)[U], F f) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = __half22float2(acc[u][j]);
      x.x = f(x.x);
      x.y = f(x.y);
      acc[u][j] = __floats2half2_rn(x.x, x.y);
    }
}
template <class F>
__device__ __forceinline__ void zip_f32(V (&acc)[U], const V (&b)[U], F f) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = __half22float2(acc[u][j]);
      const float2 y = __half22float2(b[u][j]);
      x.x = f(x.x, y.x);
      x.y = f(x.y, y.y);
      acc[u][j] = __floats2half2_rn(x.x, x.y);
    }
}
template <class F>
__device__ __forceinline__ void zip_h2(V (&acc)[U], const V (&b)[U], F f) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[u][j] = f(acc[u][j], b[u][j]);
}
template <class F>
__device__ __forceinline__ void map_h2(V (&acc)[U], F f) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[u][j] = f(acc[u][j]);
}

__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float tanh_f(float x) {
  // 1 - 2 / (e^{2x} + 1): exact limits at +-inf, relative error of a few fp32 ulp.
  return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f);
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

struct Slots {
  V a[U], b[U], c[U], d[U];
};

__device__ __forceinline__ void copy_v(V (&dst)[U], const V (&src)[U]) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[u][j] = src[u][j];
}

__device__ __forceinline__ void read_slot(const Slots& sl, int idx, V (&v)[U]) {
  switch (idx) {
    case 0: copy_v(v, sl.a); break;
    case 1: copy_v(v, sl.b); break;
    case 2: copy_v(v, sl.c); break;
    default: copy_v(v, sl.d); break;
  }
}
__device__ __forceinline__ void write_slot(Slots& sl, int idx, const V (&v)[U]) {
  switch (idx) {
    case 0: copy_v(sl.a, v); break;
    case 1: copy_v(sl.b, v); break;
    case 2: copy_v(sl.c, v); break;
    default: copy_v(sl.d, v); break;
  }
}

__device__ __forceinline__ void fetch(const PwParams& P, const Slots& sl, int kind, int idx, float imm,
                                      const Item (&it)[U], V (&v)[U]) {
  if (kind == TS_PW_TENSOR) {
#pragma unroll
    for (int u = 0; u < U; ++u) fetch_tensor(P, idx, it[u], v[u]);
  } else if (kind == TS_PW_IMM) {
    const __half2 x = __float2half2_rn(imm);
#pragma unroll
    for (int u = 0; u < U; ++u) set_all(v[u], x);
  } else if (kind == TS_PW_SAVED) {
    read_slot(sl, idx, v);
  }
}

__device__ __forceinline__ void store_full(const PwParams& P, __half* out, const Item& it, const V& v) {
  if (!it.live) return;
  Vec8h t;
#pragma unroll
  for (int j = 0; j < 4; ++j) t.h2[j] = v[j];
  if (P.ragged) {
    const uint32_t col = it.s * kStickHalfs + it.lv * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (col + e >= P.cols) t.h[e] = __float2half(0.f);
  }
  st_global_v4(out + it.flat_off, t.u);
}

// Runs the whole program on U items; the result is left in acc.
__device__ __forceinline__ void run_program(const PwParams& P, const Item (&it)[U], V (&acc)[U]) {
  Slots sl;
  V opa[U], opb[U];
  const __half2 zero2 = __float2half2_rn(0.f), one2 = __float2half2_rn(1.f);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    set_all(acc[u], zero2);
    set_all(sl.a[u], zero2);
    set_all(sl.b[u], zero2);
    set_all(sl.c[u], zero2);
    set_all(sl.d[u], zero2);
    set_all(opa[u], zero2);
    set_all(opb[u], zero2);
  }
  for (int pc = 0; pc < P.n_insns; ++pc) {
    const ts_pw_insn ins = P.insn[pc];
    if (ins.op != TS_PW_SAVE && ins.op != TS_PW_STORE)
      fetch(P, sl, ins.a_kind, ins.a_idx, ins.a_imm, it, opa);
    if (ins.op == TS_PW_WHERE) fetch(P, sl, ins.b_kind, ins.b_idx, ins.b_imm, it, opb);
    switch (ins.op) {
      case TS_PW_LOAD: copy_v(acc, opa); break;
      case TS_PW_SAVE: write_slot(sl, ins.a_idx, acc); break;
      case TS_PW_STORE:
#pragma unroll
        for (int u = 0; u < U; ++u) store_full(P, P.out[ins.a_idx], it[u], acc[u]);
        break;
      case TS_PW_ADD: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hadd2(x, y); }); break;
      case TS_PW_SUB: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hsub2(x, y); }); break;
      case TS_PW_RSUB: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hsub2(y, x); }); break;
      case TS_PW_MUL: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hmul2(x, y); }); break;
      case TS_PW_DIV: zip_f32(acc, opa, [](float x, float y) { return x / y; }); break;
      case TS_PW_RDIV: zip_f32(acc, opa, [](float x, float y) { return y / x; }); break;
      case TS_PW_MAX: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hmax2_nan(x, y); }); break;
      case TS_PW_MIN: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hmin2_nan(x, y); }); break;
      case TS_PW_POW: zip_f32(acc, opa, [](float x, float y) { return powf(x, y); }); break;
      case TS_PW_EQ: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __heq2(x, y); }); break;
      case TS_PW_NE: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hneu2(x, y); }); break;
      case TS_PW_LT: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hlt2(x, y); }); break;
      case TS_PW_LE: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hle2(x, y); }); break;
      case TS_PW_GT: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hgt2(x, y); }); break;
      case TS_PW_GE: zip_h2(acc, opa, [](__half2 x, __half2 y) { return __hge2(x, y); }); break;
      case TS_PW_WHERE:
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t m = __hneu2_mask(acc[u][j], zero2);
            const uint32_t a = *reinterpret_cast<const uint32_t*>(&opa[u][j]);
            const uint32_t b = *reinterpret_cast<const uint32_t*>(&opb[u][j]);
            const uint32_t r = (a & m) | (b & ~m);
            acc[u][j] = *reinterpret_cast<const __half2*>(&r);
          }
        break;
      case TS_PW_NEG: map_h2(acc, [](__half2 x) { return __hneg2(x); }); break;
      case TS_PW_ABS: map_h2(acc, [](__half2 x) { return __habs2(x); }); break;
      case TS_PW_EXP: map_f32(acc, [](float x) { return __expf(x); }); break;
      case TS_PW_LOG: map_f32(acc, [](float x) { return __logf(x); }); break;
      case TS_PW_SQRT: map_f32(acc, [](float x) { return sqrtf(x); }); break;
      case TS_PW_RSQRT: map_f32(acc, [](float x) { return rsqrtf(x); }); break;
      case TS_PW_RECIP: map_f32(acc, [](float x) { return 1.f / x; }); break;
      case TS_PW_SIGMOID: map_f32(acc, [](float x) { return sigmoid_f(x); }); break;
      case TS_PW_TANH: map_f32(acc, [](float x) { return tanh_f(x); }); break;
      case TS_PW_RELU: map_h2(acc, [zero2](__half2 x) { return __hmax2_nan(x, zero2); }); break;
      case TS_PW_SILU: map_f32(acc, [](float x) { return x * sigmoid_f(x); }); break;
      case TS_PW_GELU:
        map_f32(acc, [](float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); });
        break;
      case TS_PW_GELU_TANH:
        map_f32(acc, [](float x) {
          const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
          return 0.5f * x * (1.f + tanh_f(inner));
        });
        break;
      case TS_PW_SQUARE: map_h2(acc, [](__half2 x) { return __hmul2(x, x); }); break;
      case TS_PW_LOGICAL_NOT: map_h2(acc, [zero2](__half2 x) { return __heq2(x, zero2); }); break;
      case TS_PW_SIN: map_f32(acc, [](float x) { return sinf(x); }); break;
      case TS_PW_COS: map_f32(acc, [](float x) { return cosf(x); }); break;
      case TS_PW_ERF: map_f32(acc, [](float x) { return erff(x); }); break;
      case TS_PW_FLOOR: map_h2(acc, [](__half2 x) { return h2floor(x); }); break;
      case TS_PW_CEIL: map_h2(acc, [](__half2 x) { return h2ceil(x); }); break;
      case TS_PW_SIGN:
        map_f32(acc, [](float x) { return x > 0.f ? 1.f : (x < 0.f ? -1.f : x); });
        break;
      case TS_PW_LOG1P: map_f32(acc, [](float x) { return log1pf(x); }); break;
      case TS_PW_EXPM1: map_f32(acc, [](float x) { return expm1f(x); }); break;
      case TS_PW_SOFTPLUS: map_f32(acc, [](float x) { return softplus_f(x); }); break;
      case TS_PW_MISH: map_f32(acc, [](float x) { return x * tanh_f(softplus_f(x)); }); break;
      default: break;
    }
    (void)one2;
  }
}

__device__ __forceinline__ void split_row(const PwParams& P, Item& it) {
  uint32_t q, r2;
  P.div_d2.divmod(it.r, q, r2);
  it.i2 = r2;
  P.div_d1.divmod(q, it.i0, it.i1);
}

// ---- no reduction: items are the 16-byte vectors of the output image ----------
__global__ void __launch_bounds__(kThreads) pw_flat_kernel(const __grid_constant__ PwParams P) {
  Item it[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint32_t stick = blockIdx.x * (32 * U) + u * 32 + (threadIdx.x >> 3);
    it[u].lv = threadIdx.x & 7;
    it[u].live = stick < P.total_sticks;
    it[u].flat_off = (int64_t)stick * kStickHalfs + it[u].lv * 8;
    it[u].s = it[u].r = it[u].i0 = it[u].i1 = it[u].i2 = 0;
    if (P.need_index || P.ragged) {
      P.div_rows.divmod(stick, it[u].s, it[u].r);
      if (P.need_index) split_row(P, it[u]);
    }
  }
  V acc[U];
  run_program(P, it, acc);
}

__device__ __forceinline__ float red_identity(int op) {
  return op == TS_RED_SUM ? 0.f : (op == TS_RED_MAX ? -INFINITY : INFINITY);
}
__device__ __forceinline__ float red_combine(int op, float a, float b) {
  if (op == TS_RED_SUM) return a + b;
  if (a != a) return a;
  if (b != b) return b;
  return op == TS_RED_MAX ? fmaxf(a, b) : fminf(a, b);
}

// ---- reduction along the stick dim ----------------------------------------------
// A warp covers 4 adjacent rows x 8 vector lanes (512 contiguous bytes per stick
// column).  2^ws_log warps share a row group and split its stick columns.
__global__ void __launch_bounds__(kThreads) pw_rowred_kernel(const __grid_constant__ PwParams P) {
  __shared__ float part[8][4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ws = 1 << P.ws_log;
  const int ws_idx = warp & (ws - 1);
  const uint32_t group = blockIdx.x * (8 >> P.ws_log) + (warp >> P.ws_log);
  const uint32_t row = group * 4 + (lane >> 3);
  const bool row_live = row < P.rows;
  Item it[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    it[u].r = row;
    it[u].lv = lane & 7;
    it[u].i0 = it[u].i1 = it[u].i2 = 0;
    if (P.need_index && row_live) split_row(P, it[u]);
  }
  float partial = red_identity(P.red_op);
  for (uint32_t s0 = ws_idx; s0 < P.nsticks; s0 += ws * U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t s = s0 + u * ws;
      it[u].s = s;
      it[u].live = row_live && s < P.nsticks;
      it[u].flat_off = ((int64_t)s * P.rows + row) * kStickHalfs + it[u].lv * 8;
    }
    V acc[U];
    run_program(P, it, acc);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!it[u].live) continue;
      const uint32_t col = it[u].s * kStickHalfs + it[u].lv * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __half22float2(acc[u][j]);
        if (!P.ragged || col + 2 * j < P.cols) partial = red_combine(P.red_op, partial, x.x);
        if (!P.ragged || col + 2 * j + 1 < P.cols) partial = red_combine(P.red_op, partial, x.y);
      }
    }
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1)
    partial = red_combine(P.red_op, partial, __shfl_xor_sync(0xffffffffu, partial, o));
  if ((lane & 7) == 0) part[warp][lane >> 3] = partial;
  __syncthreads();
  if (ws_idx != 0 || !row_live) return;
  float total = part[warp][lane >> 3];
  for (int k = 1; k < ws; ++k) total = red_combine(P.red_op, total, part[warp + k][lane >> 3]);
  const __half result = __float2half_rn(total * P.red_scale);
  const uint32_t lv = lane & 7;
  if (P.red_keepdim) {
    Vec8h t;
    t.u = make_uint4(0, 0, 0, 0);
    if (lv == 0) t.h[0] = result;
    st_global_v4(P.red_out + (int64_t)row * kStickHalfs + lv * 8, t.u);
  } else {
    uint32_t o, l;
    P.div_red_inner.divmod(row, o, l);
    __half* base = P.red_out + ((int64_t)(l >> 6) * P.red_outer + o) * kStickHalfs;
    if (lv == 0) base[l & 63] = result;
    if (l == P.red_inner - 1)
      for (uint32_t e = (l & 63) + 1 + lv; e < 64; e += 8) base[e] = __float2half(0.f);
  }
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int ts_pointwise_chain(const ts_pw_insn* insns, int n_insns, const void* const* inputs,
                                  const int64_t* input_shapes, int n_inputs, void* const* outputs,
                                  int n_outputs, const int64_t* shape, int reduce_op,
                                  float reduce_scale, void* reduce_out, int reduce_keepdim,
                                  int64_t reduce_inner, void* stream) {
  if (!insns || !shape || n_insns < 1 || n_insns > TS_PW_MAX_INSNS) return TS_ERR_INVALID;
  if (n_inputs < 0 || n_inputs > TS_PW_MAX_INPUTS || n_outputs < 0 || n_outputs > TS_PW_MAX_OUTPUTS)
    return TS_ERR_INVALID;
  if ((n_inputs && (!inputs || !input_shapes)) || (n_outputs && !outputs)) return TS_ERR_INVALID;
  if (reduce_op < TS_RED_NONE || reduce_op > TS_RED_MIN) return TS_ERR_INVALID;
  if (reduce_op == TS_RED_NONE && n_outputs == 0) return TS_ERR_INVALID;
  for (int k = 0; k < 4; ++k)
    if (shape[k] < 0) return TS_ERR_INVALID;
  const int64_t rows = shape[0] * shape[1] * shape[2], cols = shape[3];
  if (rows == 0 || cols == 0) return TS_OK;
  const int64_t nsticks = ceil_div(cols, kStickHalfs);
  if (rows >= (1ll << 31) || nsticks * rows >= (1ll << 31)) return TS_ERR_TOO_LARGE;

  PwParams P{};
  P.n_insns = n_insns;
  P.n_in = n_inputs;
  P.n_out = n_outputs;
  for (int i = 0; i < n_insns; ++i) {
    const ts_pw_insn& in = insns[i];
    if (in.op < 0 || in.op >= TS_PW_OPCOUNT) return TS_ERR_INVALID;
    auto ok_operand = [&](int kind, int idx) {
      if (kind == TS_PW_TENSOR) return idx >= 0 && idx < n_inputs;
      if (kind == TS_PW_SAVED) return idx >= 0 && idx < TS_PW_SAVED_SLOTS;
      return kind == TS_PW_IMM || kind == TS_PW_NONE;
    };
    if (in.op == TS_PW_STORE) {
      if (in.a_idx < 0 || in.a_idx >= n_outputs) return TS_ERR_INVALID;
    } else if (in.op == TS_PW_SAVE) {
      if (in.a_idx < 0 || in.a_idx >= TS_PW_SAVED_SLOTS) return TS_ERR_INVALID;
    } else if (!ok_operand(in.a_kind, in.a_idx) || !ok_operand(in.b_kind, in.b_idx)) {
      return TS_ERR_INVALID;
    }
    P.insn[i] = in;
  }
  for (int t = 0; t < n_inputs; ++t) {
    if (!inputs[t]) return TS_ERR_INVALID;
    if ((uintptr_t)inputs[t] % 16) return TS_ERR_ALIGNMENT;
    const int64_t* ts = input_shapes + 4 * t;
    for (int k = 0; k < 4; ++k)
      if (ts[k] != shape[k] && ts[k] != 1) return TS_ERR_INVALID;
    PwTensorDesc& d = P.in[t];
    d.ptr = (const __half*)inputs[t];
    const int64_t trows = ts[0] * ts[1] * ts[2];
    d.col_bcast = (ts[3] == 1 && cols != 1) ? 1 : 0;
    d.stick_stride = trows * kStickHalfs;
    d.m2 = ts[2] == 1 ? 0 : 1;
    d.m1 = ts[1] == 1 ? 0 : (int32_t)ts[2];
    d.m0 = ts[0] == 1 ? 0 : (int32_t)(ts[1] * ts[2]);
    d.flat = (trows == rows && !d.col_bcast) ? 1 : 0;
    if (!d.flat) P.need_index = 1;
  }
  for (int o = 0; o < n_outputs; ++o) {
    if (!outputs[o]) return TS_ERR_INVALID;
    if ((uintptr_t)outputs[o] % 16) return TS_ERR_ALIGNMENT;
    P.out[o] = (__half*)outputs[o];
  }
  P.rows = (uint32_t)rows;
  P.cols = (uint32_t)cols;
  P.nsticks = (uint32_t)nsticks;
  P.total_sticks = (uint32_t)(nsticks * rows);
  P.ragged = cols % kStickHalfs ? 1 : 0;
  P.div_rows.init((uint32_t)rows);
  P.div_d2.init((uint32_t)shape[2]);
  P.div_d1.init((uint32_t)shape[1]);
  P.red_op = reduce_op;
  cudaStream_t st = (cudaStream_t)stream;
  if (reduce_op == TS_RED_NONE) {
    const uint32_t blocks = (uint32_t)ceil_div(P.total_sticks, 32 * U);
    pw_flat_kernel<<<blocks, kThreads, 0, st>>>(P);
    TSB_CHECK_LAUNCH();
    return TS_OK;
  }
  if (!reduce_out) return TS_ERR_INVALID;
  if ((uintptr_t)reduce_out % 16) return TS_ERR_ALIGNMENT;
  P.red_out = (__half*)reduce_out;
  P.red_scale = reduce_scale;
  P.red_keepdim = reduce_keepdim ? 1 : 0;
  if (!reduce_keepdim) {
    if (reduce_inner < 1 || rows % reduce_inner) return TS_ERR_INVALID;
    P.red_inner = (uint32_t)reduce_inner;
    P.red_outer = (uint32_t)(rows / reduce_inner);
    P.div_red_inner.init(P.red_inner);
  }
  // Warps per row group: as many as there are stick columns to share (up to 8),
  // fewer when that would leave too few CTAs to fill the machine.
  const int64_t groups = ceil_div(rows, 4);
  int ws_log = 3;
  while (ws_log > 0 && (1 << ws_log) > nsticks) --ws_log;
  P.ws_log = ws_log;
  const uint32_t blocks = (uint32_t)ceil_div(groups, 8 >> ws_log);
  pw_rowred_kernel<<<blocks, kThreads, 0, st>>>(P);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}
