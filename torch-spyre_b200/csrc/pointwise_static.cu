// Pre-instantiated fused programs: the patterns eager ops and common fused groups
// produce.  Each line compiles one straight-line kernel and registers it; a chain
// whose code words match runs on it instead of the interpreter.
#include "pointwise_core.cuh"

namespace tsb {
namespace pw {
namespace {

constexpr int T = TS_PW_TENSOR, I = TS_PW_IMM;
constexpr uint32_t LD0 = enc(TS_PW_LOAD, T, 0);
constexpr uint32_t ST0 = enc(TS_PW_STORE, 0, 0);
constexpr int UP = 4;  // items per thread for pointwise programs
constexpr int UR = 4;  // ... for programs ending in a row reduction

#define PW_CAT2(a, b) a##b
#define PW_CAT(a, b) PW_CAT2(a, b)
#define PW_REG(red, u, ...) static Registrar<red, u, kClsAllGeneric, __VA_ARGS__> PW_CAT(reg_, __COUNTER__);
#define PW_REG_CLS(red, u, cls, ...) static Registrar<red, u, cls, __VA_ARGS__> PW_CAT(reg_, __COUNTER__);
constexpr uint32_t cls3(int a, int b, int c) { return (uint32_t)a | ((uint32_t)b << 2) | ((uint32_t)c << 4) | 0xAA80u; }

#define PW_UNARY(op) PW_REG(TS_RED_NONE, UP, LD0, enc(op), ST0)
#define PW_BINARY(op)                                          \
  PW_REG(TS_RED_NONE, UP, LD0, enc(op, T, 1), ST0)             \
  PW_REG(TS_RED_NONE, UP, LD0, enc(op, I, 0), ST0)             \
  PW_REG(TS_RED_NONE, UP, LD0, enc(op, T, 0), ST0)

PW_UNARY(TS_PW_NEG) PW_UNARY(TS_PW_ABS) PW_UNARY(TS_PW_EXP) PW_UNARY(TS_PW_LOG)
PW_UNARY(TS_PW_SQRT) PW_UNARY(TS_PW_RSQRT) PW_UNARY(TS_PW_RECIP) PW_UNARY(TS_PW_SIGMOID)
PW_UNARY(TS_PW_TANH) PW_UNARY(TS_PW_RELU) PW_UNARY(TS_PW_SILU) PW_UNARY(TS_PW_GELU)
PW_UNARY(TS_PW_GELU_TANH) PW_UNARY(TS_PW_SQUARE) PW_UNARY(TS_PW_LOGICAL_NOT)
PW_UNARY(TS_PW_SIN) PW_UNARY(TS_PW_COS) PW_UNARY(TS_PW_ERF)

PW_BINARY(TS_PW_ADD) PW_BINARY(TS_PW_SUB) PW_BINARY(TS_PW_MUL) PW_BINARY(TS_PW_DIV)
PW_BINARY(TS_PW_MAX) PW_BINARY(TS_PW_MIN) PW_BINARY(TS_PW_EQ) PW_BINARY(TS_PW_NE)
PW_BINARY(TS_PW_LT) PW_BINARY(TS_PW_LE) PW_BINARY(TS_PW_GT) PW_BINARY(TS_PW_GE)
PW_REG(TS_RED_NONE, UP, LD0, enc(TS_PW_RSUB, I, 0), ST0)
PW_REG(TS_RED_NONE, UP, LD0, enc(TS_PW_RDIV, I, 0), ST0)
PW_REG(TS_RED_NONE, UP, LD0, enc(TS_PW_POW, I, 0), ST0)
PW_REG(TS_RED_NONE, UP, LD0, ST0)  // copy / clone

// where(cond, a, b) on three tensors
PW_REG(TS_RED_NONE, UP, LD0, enc(TS_PW_WHERE, T, 1, T, 2), ST0)
// SwiGLU gate: silu(g) * u
PW_REG(TS_RED_NONE, UP, LD0, enc(TS_PW_SILU), enc(TS_PW_MUL, T, 1), ST0)
// a*x + b style affine maps
PW_REG(TS_RED_NONE, UP, LD0, enc(TS_PW_MUL, T, 1), enc(TS_PW_ADD, T, 2), ST0)
PW_REG(TS_RED_NONE, UP, LD0, enc(TS_PW_MUL, I, 0), enc(TS_PW_ADD, I, 0), ST0)

// plain reductions and the fused reduce prologues
PW_REG(TS_RED_SUM, UR, LD0)
PW_REG(TS_RED_MAX, UR, LD0)
PW_REG(TS_RED_MIN, UR, LD0)
PW_REG_CLS(TS_RED_SUM, UR, cls3(kClsFlat, kClsGeneric, kClsGeneric), LD0)
PW_REG_CLS(TS_RED_MAX, UR, cls3(kClsFlat, kClsGeneric, kClsGeneric), LD0)
PW_REG_CLS(TS_RED_MIN, UR, cls3(kClsFlat, kClsGeneric, kClsGeneric), LD0)
PW_REG(TS_RED_SUM, UR, LD0, enc(TS_PW_SQUARE))
PW_REG(TS_RED_MAX, UR, LD0, enc(TS_PW_ABS))
PW_REG(TS_RED_SUM, UR, LD0, enc(TS_PW_EXP))
// exp(x * a + b).sum(-1): generic operands, and x full-shape with a, b row vectors
PW_REG(TS_RED_SUM, UR, LD0, enc(TS_PW_MUL, T, 1), enc(TS_PW_ADD, T, 2), enc(TS_PW_EXP))
PW_REG_CLS(TS_RED_SUM, UR, cls3(kClsFlat, kClsRowVec, kClsRowVec), LD0, enc(TS_PW_MUL, T, 1),
           enc(TS_PW_ADD, T, 2), enc(TS_PW_EXP))
// exp(x - rowmax) and its row sum (softmax pieces when not taken by the fused kernel)
PW_REG(TS_RED_SUM, UR, LD0, enc(TS_PW_SUB, T, 1), enc(TS_PW_EXP))

}  // namespace
}  // namespace pw
}  // namespace tsb

