// C-ABI entry of the fused pointwise chains: argument checks, program encoding,
// choice between a pre-instantiated program and the interpreter, launch.
// Replaces the one-op-per-kernel sfp programs of the reference
// (torch_spyre/_inductor/codegen/compute_ops.py:60-393; fusion is off there,
// torch_spyre/_inductor/choices.py:58-83).
#include <vector>

#include "pointwise_core.cuh"

namespace tsb {
namespace pw {

namespace {
std::vector<StaticEntry>& registry() {
  static std::vector<StaticEntry> r;
  return r;
}
constexpr int kDynU = 2;
}  // namespace

void register_static(const StaticEntry& e) { registry().push_back(e); }

}  // namespace pw
}  // namespace tsb

using namespace tsb;
using namespace tsb::pw;

// Number of pre-instantiated programs (diagnostics / tests).
extern "C" int ts_pointwise_static_count(void) { return (int)registry().size(); }

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
  const int64_t nsticks = ceil_div(cols, kStickHalfs);

  Params P{};
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
      P.code[i] = enc(in.op, 0, in.a_idx);
    } else if (in.op == TS_PW_SAVE) {
      if (in.a_idx < 0 || in.a_idx >= TS_PW_SAVED_SLOTS) return TS_ERR_INVALID;
      P.code[i] = enc(in.op, 0, in.a_idx);
    } else {
      if (!ok_operand(in.a_kind, in.a_idx) || !ok_operand(in.b_kind, in.b_idx)) return TS_ERR_INVALID;
      const bool has_b = in.op == TS_PW_WHERE;
      const int ai = in.a_kind == TS_PW_IMM || in.a_kind == TS_PW_NONE ? 0 : in.a_idx;
      const int bi = !has_b || in.b_kind == TS_PW_IMM || in.b_kind == TS_PW_NONE ? 0 : in.b_idx;
      P.code[i] = enc(in.op, in.a_kind, ai, has_b ? in.b_kind : 0, bi);
    }
    P.imm_a[i] = in.a_imm;
    P.imm_b[i] = in.b_imm;
  }
  for (int t = 0; t < n_inputs; ++t) {
    if (!inputs[t]) return TS_ERR_INVALID;
    if ((uintptr_t)inputs[t] % 16) return TS_ERR_ALIGNMENT;
    const int64_t* ts = input_shapes + 4 * t;
    for (int k = 0; k < 4; ++k)
      if (ts[k] != shape[k] && ts[k] != 1) return TS_ERR_INVALID;
    TensorDesc& d = P.in[t];
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
  if (reduce_op != TS_RED_NONE) {
    if (!reduce_out) return TS_ERR_INVALID;
    if ((uintptr_t)reduce_out % 16) return TS_ERR_ALIGNMENT;
    if (!reduce_keepdim && (reduce_inner < 1 || rows % reduce_inner)) return TS_ERR_INVALID;
  }
  if (rows == 0 || cols == 0) return TS_OK;
  if (rows >= (1ll << 31) || nsticks * rows >= (1ll << 31)) return TS_ERR_TOO_LARGE;

  P.rows = (uint32_t)rows;
  P.cols = (uint32_t)cols;
  P.nsticks = (uint32_t)nsticks;
  P.total_sticks = (uint32_t)(nsticks * rows);
  P.ragged = cols % kStickHalfs ? 1 : 0;
  P.div_rows.init((uint32_t)rows);
  P.div_d2.init((uint32_t)shape[2]);
  P.div_d1.init((uint32_t)shape[1]);

  // Operand classes of this call (two bits per input; unused inputs count as generic).
  uint32_t cls = kClsAllGeneric;
  for (int t = 0; t < n_inputs; ++t) {
    const TensorDesc& d = P.in[t];
    int c = kClsGeneric;
    if (d.flat) c = kClsFlat;
    else if (!d.col_bcast && d.m0 == 0 && d.m1 == 0 && d.m2 == 0) c = kClsRowVec;
    cls = (cls & ~(3u << (2 * t))) | ((uint32_t)c << (2 * t));
  }
  // A pre-instantiated program with the same code words?  Prefer one compiled for exactly
  // these operand classes, else one compiled for any.
  const StaticEntry* hit = nullptr;
  for (const StaticEntry& e : registry()) {
    if (e.red != reduce_op || e.n != n_insns) continue;
    if (e.cls != cls && e.cls != kClsAllGeneric) continue;
    bool same = true;
    for (int i = 0; i < n_insns && same; ++i) same = e.codes[i] == P.code[i];
    if (!same) continue;
    if (!hit || e.cls == cls) hit = &e;
    if (e.cls == cls) break;
  }
  const int items = hit ? hit->items : kDynU;

  cudaStream_t st = (cudaStream_t)stream;
  uint32_t blocks;
  if (reduce_op == TS_RED_NONE) {
    blocks = (uint32_t)ceil_div(P.total_sticks, 32 * items);
  } else {
    P.red_out = (__half*)reduce_out;
    P.red_scale = reduce_scale;
    P.red_keepdim = reduce_keepdim ? 1 : 0;
    if (!reduce_keepdim) {
      P.red_inner = (uint32_t)reduce_inner;
      P.red_outer = (uint32_t)(rows / reduce_inner);
      P.div_red_inner.init(P.red_inner);
    }
    // Warps per row group: as many as there are stick columns to share, up to 8.
    int ws_log = 3;
    while (ws_log > 0 && (1 << ws_log) > nsticks) --ws_log;
    P.ws_log = ws_log;
    blocks = (uint32_t)ceil_div(ceil_div(rows, 4), 8 >> ws_log);
  }
  if (hit) {
    hit->fn(P, blocks, st);
  } else {
    switch (reduce_op) {
      case TS_RED_NONE: launch_instance<Dyn, TS_RED_NONE, kDynU>(P, blocks, st); break;
      case TS_RED_SUM: launch_instance<Dyn, TS_RED_SUM, kDynU>(P, blocks, st); break;
      case TS_RED_MAX: launch_instance<Dyn, TS_RED_MAX, kDynU>(P, blocks, st); break;
      default: launch_instance<Dyn, TS_RED_MIN, kDynU>(P, blocks, st); break;
    }
  }
  TSB_CHECK_LAUNCH();
  return TS_OK;
}
