// Fused fp16 pointwise chains over stick images: program encoding, the per-item
// executor, and the two kernel templates (plain pointwise, and pointwise followed
// by a reduction along the stick dim).
//
// A program is a list of 32-bit code words (opcode and operand selectors) plus a
// pair of immediates per instruction.  The executor is one function,
// exec_insn(code, ...); the kernels are templated on where the code words come
// from:
//   * Dyn      - read from the kernel parameters at run time (an interpreter whose
//                registers are statically allocated: accumulator, operand buffers
//                and four saved slots, so nothing is indexed dynamically and every
//                branch is uniform across the grid);
//   * Fixed<…> - compile-time constants: the switch folds away and the compiler
//                schedules the whole chain as straight-line code.  Frequently fused
//                patterns are pre-instantiated this way; anything else runs on Dyn.
// Values travel as packed half2 and every op result is rounded to fp16, which is
// what eager fp16 does op by op.
#pragma once

#include "common.cuh"

namespace tsb {
namespace pw {

constexpr int kThreads = 256;

constexpr uint32_t enc(int op, int a_kind = 0, int a_idx = 0, int b_kind = 0, int b_idx = 0) {
  return (uint32_t)op | ((uint32_t)a_kind << 8) | ((uint32_t)a_idx << 12) | ((uint32_t)b_kind << 16) |
         ((uint32_t)b_idx << 20);
}
__host__ __device__ constexpr int code_op(uint32_t c) { return (int)(c & 0xff); }
__host__ __device__ constexpr int code_ak(uint32_t c) { return (int)((c >> 8) & 0xf); }
__host__ __device__ constexpr int code_ai(uint32_t c) { return (int)((c >> 12) & 0xf); }
__host__ __device__ constexpr int code_bk(uint32_t c) { return (int)((c >> 16) & 0xf); }
__host__ __device__ constexpr int code_bi(uint32_t c) { return (int)((c >> 20) & 0xf); }

struct TensorDesc {
  const __half* ptr;
  int64_t stick_stride;  // elements between consecutive stick columns of this tensor
  int32_t m0, m1, m2;    // tensor row = i0*m0 + i1*m1 + i2*m2
  int32_t col_bcast;     // single column: the value sits in lane 0 of its stick
  int32_t flat;          // same shape as the iteration space
};

struct Params {
  int n_insns, n_in, n_out;
  uint32_t code[TS_PW_MAX_INSNS];
  float imm_a[TS_PW_MAX_INSNS], imm_b[TS_PW_MAX_INSNS];
  TensorDesc in[TS_PW_MAX_INPUTS];
  __half* out[TS_PW_MAX_OUTPUTS];
  uint32_t rows, nsticks, cols, total_sticks;
  FastDiv div_rows, div_d2, div_d1;
  int need_index;  // some input is not flat
  uint32_t opaque_zero;  // always 0, but only known at run time (see fetch)
  int ragged;      // cols is not a stick multiple
  int red_keepdim, ws_log;
  float red_scale;
  __half* red_out;
  uint32_t red_inner, red_outer;
  FastDiv div_red_inner;
};

struct Dyn {
  static constexpr bool kStatic = false;
};
template <uint32_t... C>
struct Fixed {
  static constexpr bool kStatic = true;
  static constexpr int n = sizeof...(C);
  template <int I>
  __host__ __device__ static constexpr uint32_t at() {
    constexpr uint32_t a[] = {C...};
    return a[I];
  }
};

struct Item {
  uint32_t s, r, lv, i0, i1, i2;
  int64_t flat_off;  // element offset in a full-shape stick image
  bool live;
};

using V = __half2[4];

template <int U>
struct Regs {
  V acc[U], opa[U], opb[U], s0[U], s1[U], s2[U], s3[U];
};

__device__ __forceinline__ void set_all(V& v, __half2 x) {
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = x;
}
template <int U>
__device__ __forceinline__ void copy_v(V (&dst)[U], const V (&src)[U]) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[u][j] = src[u][j];
}

__device__ __forceinline__ void fetch_tensor(const Params& P, int t, const Item& it, V& v) {
  const TensorDesc& d = P.in[t];
  if (!it.live) {
    set_all(v, __float2half2_rn(0.f));
    return;
  }
  Vec8h x;
  if (d.flat) {
    x.u = ld_stream_v4(d.ptr + it.flat_off);
  } else {
    const uint32_t row = it.i0 * (uint32_t)d.m0 + it.i1 * (uint32_t)d.m1 + it.i2 * (uint32_t)d.m2;
    if (!d.col_bcast) {
      x.u = ld_global_v4(d.ptr + (int64_t)it.s * d.stick_stride + (int64_t)row * kStickHalfs +
                         it.lv * 8);
    } else {
      set_all(v, __half2half2(__ldg(d.ptr + (int64_t)row * kStickHalfs)));
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = x.h2[j];
}

__device__ __forceinline__ void store_full(const Params& P, __half* out, const Item& it, const V& v) {
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

// ---- operand contexts ---------------------------------------------------------------
// General: every item carries its own coordinates.
template <int U>
struct ItemCtx {
  static constexpr int kPrefetch = -1;
  const Params& P;
  Item it[U];
  __device__ __forceinline__ explicit ItemCtx(const Params& p) : P(p) {}
  __device__ __forceinline__ void tensor(int t, int u, V& v) const { fetch_tensor(P, t, it[u], v); }
  __device__ __forceinline__ void store(int o, int u, const V& v) const {
    store_full(P, P.out[o], it[u], v);
  }
};

// Row kernels with a compile-time program: all items of a thread lie in one row, so
// each tensor needs one base pointer and one stride per stick column, set up once.
// FULL: no item is ever out of range and cols is a stick multiple.
// Operand classes, two bits per input tensor, fixed at compile time per instantiation:
// how a tensor is addressed decides how many instructions each fetch costs.
constexpr int kClsFlat = 0;     // same shape as the iteration space
constexpr int kClsRowVec = 1;   // [cols] vector broadcast along rows
constexpr int kClsGeneric = 2;  // anything else: resolved from the run-time descriptor
constexpr uint32_t kClsAllGeneric = 0xAAAAu;
__host__ __device__ constexpr int cls_of(uint32_t mask, int t) { return (int)((mask >> (2 * t)) & 3u); }

template <int U, bool FULL, int RG, uint32_t CLS, int PF = -1>
struct RowCtx {
  // PF >= 0: input PF (a flat operand) is not loaded by tensor(); the kernel loads it one
  // step ahead and hands it over in `cur`.
  static constexpr int kPrefetch = PF;
  V cur[PF >= 0 ? U : 1];
  // U items = RG row groups (rows 4 apart) x U/RG stick columns; item i belongs to row
  // group i / (U/RG).  A row vector is fetched once for all RG rows (same address).
  static constexpr int kPerGroup = U / RG;
  const Params& P;
  int64_t flat_base;    // element offset of (row, lane vector) in stick column 0 of a flat image
  int64_t flat_stride;  // elements between stick columns of a flat image
  const __half* gbase[TS_PW_MAX_INPUTS][RG];   // generic operands only
  int64_t gstride[TS_PW_MAX_INPUTS];
  __half2 bval[TS_PW_MAX_INPUTS][RG];
  uint32_t lv, s[U];
  bool live[U];
  __device__ __forceinline__ RowCtx(const Params& p, uint32_t row, uint32_t lane_vec, bool row_live)
      : P(p), lv(lane_vec) {
    flat_base = (int64_t)row * kStickHalfs + lane_vec * 8;
    flat_stride = (int64_t)p.rows * kStickHalfs;
#pragma unroll
    for (int t = 0; t < TS_PW_MAX_INPUTS; ++t) {
      gstride[t] = 0;
#pragma unroll
      for (int g = 0; g < RG; ++g) {
        gbase[t][g] = nullptr;
        bval[t][g] = __float2half2_rn(0.f);
      }
    }
    bool any_generic = false;
#pragma unroll
    for (int t = 0; t < TS_PW_MAX_INPUTS; ++t) any_generic = any_generic || cls_of(CLS, t) == kClsGeneric;
    if (any_generic) {
#pragma unroll
      for (int g = 0; g < RG; ++g) {
        const uint32_t r = row + 4 * g;
        uint32_t i0 = 0, i1 = 0, i2 = 0;
        if (p.need_index && row_live) {
          uint32_t q;
          p.div_d2.divmod(r, q, i2);
          p.div_d1.divmod(q, i0, i1);
        }
#pragma unroll
        for (int t = 0; t < TS_PW_MAX_INPUTS; ++t) {
          if (cls_of(CLS, t) == kClsGeneric && t < p.n_in) {
            const TensorDesc& d = p.in[t];
            const uint32_t trow = d.flat ? r : i0 * (uint32_t)d.m0 + i1 * (uint32_t)d.m1 +
                                                   i2 * (uint32_t)d.m2;
            gbase[t][g] = d.ptr + (int64_t)trow * kStickHalfs + (d.col_bcast ? 0 : lane_vec * 8);
            gstride[t] = d.col_bcast ? 0 : d.stick_stride;
            if (d.col_bcast && row_live) bval[t][g] = __half2half2(__ldg(gbase[t][g]));
          }
        }
      }
    }
  }
  __device__ __forceinline__ void tensor(int t, int u, V& v) const {
    if (!FULL && !live[u]) {
      set_all(v, __float2half2_rn(0.f));
      return;
    }
    const int g = u / kPerGroup;
    const int cls = cls_of(CLS, t);
    Vec8h x;
    if (PF >= 0 && t == PF) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = cur[PF >= 0 ? u : 0][j];
      return;
    }
    if (cls == kClsFlat) {
      x.u = ld_stream_v4(P.in[t].ptr + flat_base + (int64_t)(4 * g) * kStickHalfs +
                         (int64_t)s[u] * flat_stride);
    } else if (cls == kClsRowVec) {
      x.u = ld_global_v4(P.in[t].ptr + s[u] * kStickHalfs + lv * 8);
    } else {
      if (P.in[t].col_bcast) {
        set_all(v, bval[t][g]);
        return;
      }
      const __half* p = gbase[t][g] + (int64_t)s[u] * gstride[t];
      x.u = P.in[t].flat ? ld_stream_v4(p) : ld_global_v4(p);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = x.h2[j];
  }
  // the 16 bytes of flat input t that item u reads in stick column `stick`
  __device__ __forceinline__ uint4 load_flat(int t, int u, uint32_t stick) const {
    return ld_stream_v4(P.in[t].ptr + flat_base + (int64_t)(4 * (u / kPerGroup)) * kStickHalfs +
                        (int64_t)stick * flat_stride);
  }
  __device__ __forceinline__ void store(int o, int u, const V& v) const {
    if (!FULL && !live[u]) return;
    Vec8h t;
#pragma unroll
    for (int j = 0; j < 4; ++j) t.h2[j] = v[j];
    if (!FULL && P.ragged) {
      const uint32_t col = s[u] * kStickHalfs + lv * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (col + e >= P.cols) t.h[e] = __float2half(0.f);
    }
    const int g = u / kPerGroup;
    st_global_v4(P.out[o] + flat_base + (int64_t)(4 * g) * kStickHalfs + (int64_t)s[u] * flat_stride, t.u);
  }
};

template <int U, class Ctx>
__device__ __forceinline__ void fetch(const Ctx& ctx, Regs<U>& R, int kind, int idx, float imm,
                                      V (&v)[U]) {
  if (kind == TS_PW_TENSOR) {
#pragma unroll
    for (int u = 0; u < U; ++u) ctx.tensor(idx, u, v[u]);
    if (U > 1 && idx != Ctx::kPrefetch) {
      // Make every item's value depend on all U loads (through a mask that is zero at
      // run time), so that the U loads are issued back to back instead of each one
      // being scheduled next to its own use, which would leave one load in flight.
      uint32_t m = 0;
#pragma unroll
      for (int u = 0; u < U; ++u) m ^= *reinterpret_cast<const uint32_t*>(&v[u][0]);
      m &= ctx.P.opaque_zero;
#pragma unroll
      for (int u = 0; u < U; ++u) *reinterpret_cast<uint32_t*>(&v[u][0]) ^= m;
    }
  } else if (kind == TS_PW_IMM) {
    const __half2 x = __float2half2_rn(imm);
#pragma unroll
    for (int u = 0; u < U; ++u) set_all(v[u], x);
  } else if (kind == TS_PW_SAVED) {
    switch (idx) {
      case 0: copy_v<U>(v, R.s0); break;
      case 1: copy_v<U>(v, R.s1); break;
      case 2: copy_v<U>(v, R.s2); break;
      default: copy_v<U>(v, R.s3); break;
    }
  }
}

template <int U, class F>
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
template <int U, class F>
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
template <int U, class F>
__device__ __forceinline__ void zip_h2(V (&acc)[U], const V (&b)[U], F f) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[u][j] = f(acc[u][j], b[u][j]);
}
template <int U, class F>
__device__ __forceinline__ void map_h2(V (&acc)[U], F f) {
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[u][j] = f(acc[u][j]);
}

// e^x through the special-function unit: one multiply and one ex2.approx.ftz.
__device__ __forceinline__ float exp_f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + exp_f(-x)); }
// 1 - 2 / (e^{2x} + 1): exact limits at +-inf, relative error of a few fp32 ulp.
__device__ __forceinline__ float tanh_f(float x) {
  return 1.f - __fdividef(2.f, exp_f(2.f * x) + 1.f);
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(exp_f(x)); }

// Unary ops evaluated in fp32.  `op` is a literal at every call site.
__host__ __device__ constexpr bool is_unary_f32(int op) {
  return op == TS_PW_EXP || op == TS_PW_LOG || op == TS_PW_SQRT || op == TS_PW_RSQRT ||
         op == TS_PW_RECIP || op == TS_PW_SIGMOID || op == TS_PW_TANH || op == TS_PW_SILU ||
         op == TS_PW_GELU || op == TS_PW_GELU_TANH || op == TS_PW_SIN || op == TS_PW_COS ||
         op == TS_PW_ERF || op == TS_PW_SIGN || op == TS_PW_LOG1P || op == TS_PW_EXPM1 ||
         op == TS_PW_SOFTPLUS || op == TS_PW_MISH || op == TS_PW_SQUARE;
}
__device__ __forceinline__ float unary_f32(int op, float x) {
  switch (op) {
    case TS_PW_EXP: return exp_f(x);
    case TS_PW_LOG: return __logf(x);
    case TS_PW_SQRT: return sqrtf(x);
    case TS_PW_RSQRT: return rsqrtf(x);
    case TS_PW_RECIP: return 1.f / x;
    case TS_PW_SIGMOID: return sigmoid_f(x);
    case TS_PW_TANH: return tanh_f(x);
    case TS_PW_SILU: return x * sigmoid_f(x);
    case TS_PW_GELU: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case TS_PW_GELU_TANH: {
      const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanh_f(inner));
    }
    case TS_PW_SIN: return sinf(x);
    case TS_PW_COS: return cosf(x);
    case TS_PW_ERF: return erff(x);
    case TS_PW_SIGN: return x > 0.f ? 1.f : (x < 0.f ? -1.f : x);
    case TS_PW_LOG1P: return log1pf(x);
    case TS_PW_EXPM1: return expm1f(x);
    case TS_PW_SOFTPLUS: return softplus_f(x);
    case TS_PW_MISH: return x * tanh_f(softplus_f(x));
    case TS_PW_SQUARE: return x * x;   // exact in fp32: a sum of squares cannot overflow per term
    default: return x;
  }
}

// One instruction on U items.  With a compile-time `code` everything but the
// selected case disappears.
#define TSB_PW_F32_CASE(OPC) \
  case OPC: map_f32<U>(acc, [](float x) { return unary_f32(OPC, x); }); break;

template <int U, class Ctx>
__device__ __forceinline__ void exec_insn(const Params& P, Regs<U>& R, const Ctx& ctx, uint32_t code,
                                          float imm_a, float imm_b) {
  const int op = code_op(code);
  const __half2 zero2 = __float2half2_rn(0.f);
  V(&acc)[U] = R.acc;
  V(&opa)[U] = R.opa;
  if (op != TS_PW_SAVE && op != TS_PW_STORE)
    fetch<U>(ctx, R, code_ak(code), code_ai(code), imm_a, R.opa);
  if (op == TS_PW_WHERE) fetch<U>(ctx, R, code_bk(code), code_bi(code), imm_b, R.opb);
  switch (op) {
    case TS_PW_LOAD: copy_v<U>(acc, opa); break;
    case TS_PW_SAVE:
      switch (code_ai(code)) {
        case 0: copy_v<U>(R.s0, acc); break;
        case 1: copy_v<U>(R.s1, acc); break;
        case 2: copy_v<U>(R.s2, acc); break;
        default: copy_v<U>(R.s3, acc); break;
      }
      break;
    case TS_PW_STORE:
#pragma unroll
      for (int u = 0; u < U; ++u) ctx.store(code_ai(code), u, acc[u]);
      break;
    case TS_PW_ADD: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hadd2(x, y); }); break;
    case TS_PW_SUB: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hsub2(x, y); }); break;
    case TS_PW_RSUB: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hsub2(y, x); }); break;
    case TS_PW_MUL: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hmul2(x, y); }); break;
    case TS_PW_DIV: zip_f32<U>(acc, opa, [](float x, float y) { return x / y; }); break;
    case TS_PW_RDIV: zip_f32<U>(acc, opa, [](float x, float y) { return y / x; }); break;
    case TS_PW_MAX: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hmax2_nan(x, y); }); break;
    case TS_PW_MIN: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hmin2_nan(x, y); }); break;
    case TS_PW_POW: zip_f32<U>(acc, opa, [](float x, float y) { return powf(x, y); }); break;
    case TS_PW_EQ: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __heq2(x, y); }); break;
    case TS_PW_NE: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hneu2(x, y); }); break;
    case TS_PW_LT: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hlt2(x, y); }); break;
    case TS_PW_LE: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hle2(x, y); }); break;
    case TS_PW_GT: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hgt2(x, y); }); break;
    case TS_PW_GE: zip_h2<U>(acc, opa, [](__half2 x, __half2 y) { return __hge2(x, y); }); break;
    case TS_PW_WHERE:
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t m = __hneu2_mask(acc[u][j], zero2);
          const uint32_t a = *reinterpret_cast<const uint32_t*>(&opa[u][j]);
          const uint32_t b = *reinterpret_cast<const uint32_t*>(&R.opb[u][j]);
          const uint32_t r = (a & m) | (b & ~m);
          acc[u][j] = *reinterpret_cast<const __half2*>(&r);
        }
      break;
    case TS_PW_NEG: map_h2<U>(acc, [](__half2 x) { return __hneg2(x); }); break;
    case TS_PW_ABS: map_h2<U>(acc, [](__half2 x) { return __habs2(x); }); break;
    case TS_PW_RELU: map_h2<U>(acc, [zero2](__half2 x) { return __hmax2_nan(x, zero2); }); break;
    case TS_PW_SQUARE: map_h2<U>(acc, [](__half2 x) { return __hmul2(x, x); }); break;
    case TS_PW_LOGICAL_NOT: map_h2<U>(acc, [zero2](__half2 x) { return __heq2(x, zero2); }); break;
    case TS_PW_FLOOR: map_h2<U>(acc, [](__half2 x) { return h2floor(x); }); break;
    case TS_PW_CEIL: map_h2<U>(acc, [](__half2 x) { return h2ceil(x); }); break;
    TSB_PW_F32_CASE(TS_PW_EXP) TSB_PW_F32_CASE(TS_PW_LOG) TSB_PW_F32_CASE(TS_PW_SQRT)
    TSB_PW_F32_CASE(TS_PW_RSQRT) TSB_PW_F32_CASE(TS_PW_RECIP) TSB_PW_F32_CASE(TS_PW_SIGMOID)
    TSB_PW_F32_CASE(TS_PW_TANH) TSB_PW_F32_CASE(TS_PW_SILU) TSB_PW_F32_CASE(TS_PW_GELU)
    TSB_PW_F32_CASE(TS_PW_GELU_TANH) TSB_PW_F32_CASE(TS_PW_SIN) TSB_PW_F32_CASE(TS_PW_COS)
    TSB_PW_F32_CASE(TS_PW_ERF) TSB_PW_F32_CASE(TS_PW_SIGN) TSB_PW_F32_CASE(TS_PW_LOG1P)
    TSB_PW_F32_CASE(TS_PW_EXPM1) TSB_PW_F32_CASE(TS_PW_SOFTPLUS) TSB_PW_F32_CASE(TS_PW_MISH)
    default: break;
  }
}
#undef TSB_PW_F32_CASE

template <class Prog, int U, int I, int END, class Ctx>
__device__ __forceinline__ void run_fixed(const Params& P, Regs<U>& R, const Ctx& ctx) {
  if constexpr (I < END) {
    exec_insn<U>(P, R, ctx, Prog::template at<I>(), P.imm_a[I], P.imm_b[I]);
    run_fixed<Prog, U, I + 1, END>(P, R, ctx);
  }
}

template <int U>
__device__ __forceinline__ void clear_regs(Regs<U>& R) {
  const __half2 zero2 = __float2half2_rn(0.f);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    set_all(R.acc[u], zero2);
    set_all(R.opa[u], zero2);
    set_all(R.opb[u], zero2);
    set_all(R.s0[u], zero2);
    set_all(R.s1[u], zero2);
    set_all(R.s2[u], zero2);
    set_all(R.s3[u], zero2);
  }
}

// Runs instructions [0, END) (all of them when END < 0); the result is left in R.acc.
template <class Prog, int U, int END = -1, class Ctx>
__device__ __forceinline__ void run_program(const Params& P, Regs<U>& R, const Ctx& ctx) {
  clear_regs<U>(R);
  if constexpr (Prog::kStatic) {
    run_fixed<Prog, U, 0, (END < 0 ? Prog::n : END)>(P, R, ctx);
  } else {
    for (int pc = 0; pc < P.n_insns; ++pc) exec_insn<U>(P, R, ctx, P.code[pc], P.imm_a[pc], P.imm_b[pc]);
  }
}

__device__ __forceinline__ void split_row(const Params& P, Item& it) {
  uint32_t q, r2;
  P.div_d2.divmod(it.r, q, r2);
  it.i2 = r2;
  P.div_d1.divmod(q, it.i0, it.i1);
}

// ---- no reduction: items are the 16-byte vectors of the output image ----------
template <class Prog, int U>
__global__ void __launch_bounds__(kThreads) flat_kernel(const __grid_constant__ Params P) {
  grid_dependency_wait();
  grid_release_dependents();
  ItemCtx<U> ctx(P);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    Item& it = ctx.it[u];
    const uint32_t stick = blockIdx.x * (32 * U) + u * 32 + (threadIdx.x >> 3);
    it.lv = threadIdx.x & 7;
    it.live = stick < P.total_sticks;
    it.flat_off = (int64_t)stick * kStickHalfs + it.lv * 8;
    it.s = it.r = it.i0 = it.i1 = it.i2 = 0;
    if (P.need_index || P.ragged) {
      P.div_rows.divmod(stick, it.s, it.r);
      if (P.need_index) split_row(P, it);
    }
  }
  Regs<U> R;
  run_program<Prog, U>(P, R, ctx);
}

// acc + float(h) in one instruction (mixed-precision add, sm_100).
__device__ __forceinline__ float add_f16(float acc, __half h) {
  asm("add.rn.f32.f16 %0, %1, %0;" : "+f"(acc) : "h"(__half_as_ushort(h)));
  return acc;
}

// Two fp32 lanes per instruction (sm_100 packed fp32): halves the issue slots the
// multiply by log2(e) and the accumulation cost.
__device__ __forceinline__ float2 mul_f32x2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float2 add_f32x2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float ex2_f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int RED>
__device__ __forceinline__ float red_identity() {
  return RED == TS_RED_SUM ? 0.f : (RED == TS_RED_MAX ? -INFINITY : INFINITY);
}
template <int RED>
__device__ __forceinline__ float red_combine(float a, float b) {
  if (RED == TS_RED_SUM) return a + b;
  const float r = RED == TS_RED_MAX ? fmaxf(a, b) : fminf(a, b);
  return (b != b) ? b : ((a != a) ? a : r);  // NaN propagates, as torch.max / torch.min do
}

// Cross-lane / cross-warp part of a row reduction and the write of the result.
template <int RED>
__device__ __forceinline__ void finish_row(const Params& P, float partial, uint32_t row,
                                           bool row_live, int lane, int warp, int ws, int ws_idx,
                                           float (*part)[4]) {
#pragma unroll
  for (int o = 1; o < 8; o <<= 1)
    partial = red_combine<RED>(partial, __shfl_xor_sync(0xffffffffu, partial, o));
  if ((lane & 7) == 0) part[warp][lane >> 3] = partial;
  __syncthreads();
  if (ws_idx != 0 || !row_live) return;
  float total = part[warp][lane >> 3];
  for (int k = 1; k < ws; ++k) total = red_combine<RED>(total, part[warp + k][lane >> 3]);
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

// ---- reduction along the stick dim ----------------------------------------------
// A warp covers 4 adjacent rows x 8 vector lanes (512 contiguous bytes per stick
// column).  2^ws_log warps share a row group and split its stick columns.
//
// Interpreter form: items carry full coordinates, every flag is read at run time.
template <int RED, int U>
__global__ void __launch_bounds__(kThreads) rowred_dyn_kernel(const __grid_constant__ Params P) {
  __shared__ float part[8][4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ws = 1 << P.ws_log;
  const int ws_idx = warp & (ws - 1);
  const uint32_t group = blockIdx.x * (8 >> P.ws_log) + (warp >> P.ws_log);
  const uint32_t row = group * 4 + (lane >> 3);
  const bool row_live = row < P.rows;
  ItemCtx<U> ctx(P);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    Item& it = ctx.it[u];
    it.r = row;
    it.lv = lane & 7;
    it.i0 = it.i1 = it.i2 = 0;
    if (P.need_index && row_live) split_row(P, it);
  }
  float partial = red_identity<RED>();
  Regs<U> R;
  for (uint32_t s0 = ws_idx; s0 < P.nsticks; s0 += ws * U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      Item& it = ctx.it[u];
      const uint32_t s = s0 + u * ws;
      it.s = s;
      it.live = row_live && s < P.nsticks;
      it.flat_off = ((int64_t)s * P.rows + row) * kStickHalfs + it.lv * 8;
    }
    run_program<Dyn, U>(P, R, ctx);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!ctx.it[u].live) continue;
      const uint32_t col = ctx.it[u].s * kStickHalfs + ctx.it[u].lv * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __half22float2(R.acc[u][j]);
        if (!P.ragged || col + 2 * j < P.cols) partial = red_combine<RED>(partial, x.x);
        if (!P.ragged || col + 2 * j + 1 < P.cols) partial = red_combine<RED>(partial, x.y);
      }
    }
  }
  finish_row<RED>(P, partial, row, row_live, lane, warp, ws, ws_idx, part);
}

// Compile-time program.  When the program ends in a unary op evaluated in fp32, that
// op's fp32 results feed the reduction directly, skipping the fp16 round trip (the
// reduction accumulates in fp32 either way).
// Input a program's first instruction loads, if that input is flat: the one worth loading a
// step ahead.  -1 otherwise.
template <class Prog, uint32_t CLS>
__host__ __device__ constexpr int prefetch_operand() {
  constexpr uint32_t c0 = Prog::template at<0>();
  return (code_op(c0) == TS_PW_LOAD && code_ak(c0) == TS_PW_TENSOR &&
          cls_of(CLS, code_ai(c0)) == kClsFlat) ? code_ai(c0) : -1;
}

template <class Prog, int RED, int U, bool FULL, int RG, uint32_t CLS, int PF = -1>
__global__ void __launch_bounds__(kThreads, (CLS == kClsAllGeneric ? 1 : 4)) rowred_kernel(const __grid_constant__ Params P) {
  __shared__ float part[8][4];
  grid_dependency_wait();
  grid_release_dependents();
  constexpr int kLastOp = code_op(Prog::template at<Prog::n - 1>());
  constexpr bool kFuseTail = is_unary_f32(kLastOp);
  constexpr int kPerGroup = U / RG;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ws = 1 << P.ws_log;
  const int ws_idx = warp & (ws - 1);
  const uint32_t group = blockIdx.x * (8 >> P.ws_log) + (warp >> P.ws_log);
  const uint32_t row = group * (4 * RG) + (lane >> 3);
  const bool row_live = FULL || row < P.rows;   // RG > 1 is only used with FULL
  static_assert(PF < 0 || FULL, "prefetch needs full steps");
  RowCtx<U, FULL, RG, CLS, PF> ctx(P, row, lane & 7, row_live);
  float partial[RG];
#pragma unroll
  for (int g = 0; g < RG; ++g) partial[g] = red_identity<RED>();
  Regs<U> R;
  uint4 pre[PF >= 0 ? U : 1];
  if (PF >= 0) {
#pragma unroll
    for (int u = 0; u < U; ++u) pre[u] = ctx.load_flat(PF, u, ws_idx + (u % kPerGroup) * ws);
  }
  for (uint32_t s0 = ws_idx; s0 < P.nsticks; s0 += ws * kPerGroup) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      ctx.s[u] = s0 + (u % kPerGroup) * ws;
      ctx.live[u] = FULL || (row_live && ctx.s[u] < P.nsticks);
    }
    if (PF >= 0) {
      // Take over the vectors loaded during the previous step (every one of them must have
      // arrived: the mask, zero at run time, ties each value to all U loads), then start the
      // next step's loads so that they are in flight during this step's arithmetic.
      uint32_t m = 0;
#pragma unroll
      for (int u = 0; u < U; ++u) m ^= pre[u].x;
      m &= P.opaque_zero;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        Vec8h x;
        x.u = pre[u];
        x.u.x ^= m;
#pragma unroll
        for (int j = 0; j < 4; ++j) ctx.cur[PF >= 0 ? u : 0][j] = x.h2[j];
      }
      const uint32_t sn = s0 + ws * kPerGroup;
      if (sn < P.nsticks) {
#pragma unroll
        for (int u = 0; u < U; ++u) pre[u] = ctx.load_flat(PF, u, sn + (u % kPerGroup) * ws);
      }
    }
    run_program<Prog, U, (kFuseTail ? Prog::n - 1 : Prog::n)>(P, R, ctx);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!FULL && !ctx.live[u]) continue;
      const uint32_t col = ctx.s[u] * kStickHalfs + ctx.lv * 8;
      float t = red_identity<RED>();
      if (RED == TS_RED_SUM && kFuseTail && kLastOp == TS_PW_EXP && FULL) {
        // sum of e^x: same values as the generic branch below, added pairwise
        float2 t2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 x = mul_f32x2(__half22float2(R.acc[u][j]),
                               make_float2(1.4426950408889634f, 1.4426950408889634f));
          x.x = ex2_f(x.x);
          x.y = ex2_f(x.y);
          t2 = add_f32x2(t2, x);
        }
        t = t2.x + t2.y;
      } else if (RED == TS_RED_SUM && !kFuseTail && FULL) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          t = add_f16(add_f16(t, __low2half(R.acc[u][j])), __high2half(R.acc[u][j]));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 x = __half22float2(R.acc[u][j]);
          if (kFuseTail) {
            x.x = unary_f32(kLastOp, x.x);
            x.y = unary_f32(kLastOp, x.y);
          }
          if (!FULL && P.ragged) {
            if (col + 2 * j >= P.cols) x.x = red_identity<RED>();
            if (col + 2 * j + 1 >= P.cols) x.y = red_identity<RED>();
          }
          t = red_combine<RED>(t, red_combine<RED>(x.x, x.y));
        }
      }
      partial[u / kPerGroup] = red_combine<RED>(partial[u / kPerGroup], t);
    }
  }
#pragma unroll
  for (int g = 0; g < RG; ++g) {
    if (g > 0) __syncthreads();   // `part` is reused
    finish_row<RED>(P, partial[g], row + 4 * g, row_live, lane, warp, ws, ws_idx, part);
  }
}

// ---- registry of pre-instantiated programs ----------------------------------------
using LaunchFn = void (*)(const Params&, uint32_t blocks, cudaStream_t);

struct StaticEntry {
  const uint32_t* codes;
  int n;
  int red;  // TS_RED_*
  int items;  // work items per thread per step (U)
  uint32_t cls;  // operand classes the instance was compiled for (kClsAllGeneric = any)
  LaunchFn fn;
};
void register_static(const StaticEntry& e);  // pointwise.cu

// Whether the row kernels may drop every predicate for this launch.
inline bool rows_full(const Params& P, int U) {
  const uint32_t ws = 1u << P.ws_log;
  return P.cols % 64 == 0 && P.nsticks % (ws * U) == 0 && P.rows % (4 * (8 >> P.ws_log)) == 0;
}

template <class Prog, int RED, int U, uint32_t CLS = kClsAllGeneric>
void launch_instance(const Params& P, uint32_t blocks, cudaStream_t st) {
  if constexpr (RED == TS_RED_NONE) {
    launch_after_tail(flat_kernel<Prog, U>, blocks, kThreads, 0, st, P);
  } else if constexpr (!Prog::kStatic) {
    rowred_dyn_kernel<RED, U><<<blocks, kThreads, 0, st>>>(P);
  } else {
    const bool full = rows_full(P, U);
    const uint32_t groups_per_block = 8u >> P.ws_log;
    if (full && P.rows % (8 * groups_per_block) == 0) {
      // two row groups per warp step: operands broadcast along rows are fetched once for both
      constexpr int kPF = prefetch_operand<Prog, CLS>();
      const uint32_t grid = P.rows / (8 * groups_per_block);
      if constexpr (kPF >= 0 && CLS != kClsAllGeneric) {
        // the streamed operand is loaded one step ahead: half the items per step, so that the
        // extra buffer still fits 64 registers (4 CTAs per SM); measured 8 % faster than the
        // wider step without the look-ahead on [8192, 8192]
        launch_after_tail(rowred_kernel<Prog, RED, U, true, 2, CLS, kPF>, grid, kThreads, 0, st, P);
      } else {
        launch_after_tail(rowred_kernel<Prog, RED, 2 * U, true, 2, CLS>, grid, kThreads, 0, st, P);
      }
    } else if (full) {
      launch_after_tail(rowred_kernel<Prog, RED, U, true, 1, CLS>, blocks, kThreads, 0, st, P);
    } else {
      launch_after_tail(rowred_kernel<Prog, RED, U, false, 1, CLS>, blocks, kThreads, 0, st, P);
    }
  }
}

template <int RED, int U, uint32_t CLS, uint32_t... C>
struct Registrar {
  Registrar() {
    static const uint32_t codes[] = {C...};
    register_static(StaticEntry{codes, (int)sizeof...(C), RED, U, CLS,
                                &launch_instance<Fixed<C...>, RED, U, CLS>});
  }
};

}  // namespace pw
}  // namespace tsb
