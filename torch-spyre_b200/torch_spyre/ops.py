"""aten kernels for ``spyre`` tensors, registered on the PrivateUse1 dispatch key.

The reference generates one C++ wrapper per op from codegen/inputs/Metadata.yaml
(codegen/templates/base.jinja2:16-241) and hand-writes mm / bmm / addmm / mean /
fill_ / clone (codegen/inputs/spyre_torch_ops.cpp:214-601); each wrapper builds a
sendnn graph and runs it.  Here each op marshals its arguments and calls one entry
point of the kernel library.  Results follow torch CPU eager semantics; where the
reference's wrappers deviate from them (addmm ignoring beta, mean dividing per dim,
layer norm returning its input) the CPU semantics win.

fp16 is the compute dtype of the device.  Comparison ops return fp16 0/1 tensors, as
the reference's do (tests/test_ops.py:141-152 cast them with .bool()).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import contextlib
import threading

import torch

from . import _C, _abi, stick_ops as K
from .stick_ops import Chain, StickTensor

_lib = torch.library.Library("aten", "IMPL")
_KEY = "PrivateUse1"
_registered: List[str] = []


def _impl(name: str):
    def deco(fn):
        _lib.impl(name, fn, _KEY)
        _registered.append(name)
        return fn

    return deco


def registered_ops() -> List[str]:
    return list(_registered)


def _check_fp16(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t.dtype != torch.float16:
            raise NotImplementedError(
                f"spyre kernels compute in float16; got {t.dtype} (convert on the host first)")


def _canonical(t: torch.Tensor) -> torch.Tensor:
    """The tensor itself if its storage is its own stick image, else a fresh copy that is."""
    if _C.is_canonical(t):
        return t
    out = torch.empty(t.shape, dtype=t.dtype, device=t.device)
    out.copy_(t)
    return out


def _st(t: torch.Tensor) -> StickTensor:
    t = _canonical(t)
    shape = tuple(t.shape) if t.dim() else (1,)
    st = StickTensor(_C.storage_as_cuda_bytes(t), shape, t.dtype)
    st.owner = t  # keeps a temporary copy alive for the launch
    return st


def _broadcast_shapes(*shapes) -> tuple:
    """torch.broadcast_shapes for plain integer shapes (the torch function goes through symbolic-shape
    guards and costs tens of microseconds per eager op)."""
    rank = max((len(s) for s in shapes), default=0)
    out = [1] * rank
    for s in shapes:
        off = rank - len(s)
        for i, d in enumerate(s):
            d = int(d)
            if d != 1:
                if out[off + i] not in (1, d):
                    raise RuntimeError(f"shapes {[tuple(x) for x in shapes]} cannot be broadcast together")
                out[off + i] = d
    return tuple(out)


def _new(shape: Sequence[int], like: torch.Tensor) -> torch.Tensor:
    return torch.empty(tuple(shape), dtype=like.dtype, device=like.device)


def _is_number(x) -> bool:
    return isinstance(x, (int, float, bool)) or (isinstance(x, torch.Tensor) and x.device.type == "cpu"
                                                 and x.dim() == 0)


def _number(x) -> float:
    return float(x.item()) if isinstance(x, torch.Tensor) else float(x)


_NO_SWITCH = contextlib.nullcontext()


def _with_device(t: torch.Tensor):
    """Context in which the tensor's CUDA device is current (nothing to do when it already is)."""
    index = t.device.index if t.device.index is not None else 0
    if torch._C._cuda_getDevice() == index:
        return _NO_SWITCH
    return torch.cuda.device(index)


# ---- pointwise -------------------------------------------------------------------------

# One-output chains of the eager ops, marshalled once per (program, shapes) and thread: a call
# patches the operand pointers (and the immediate) into the cached ctypes arrays and enqueues.
# Building the instruction structs, the shape arrays and a CUDA view of every operand's storage
# anew for each op was most of an eager op's host time.
_tls = threading.local()
_PLACEHOLDER = [object() for _ in range(4)]


def _launch_cached(key, program, out_shape, in_shapes, in_tensors, out: torch.Tensor, imm=None) -> bool:
    """False, having done nothing, if an operand is a view that is not its own stick image (the
    caller then takes the general route, which copies such views first)."""
    for t in in_tensors:
        if not _C.is_canonical(t):
            return False
    plans = getattr(_tls, "plans", None)
    if plans is None:
        plans = _tls.plans = {}
    plan = plans.get(key)
    if plan is None:
        if len(plans) >= 1024:
            plans.clear()
        chain = Chain()
        program(chain, [chain.tensor(_PLACEHOLDER[i]) for i in range(len(in_shapes))])
        shape = tuple(out_shape) if len(out_shape) else (1,)
        flat: List[int] = []
        for s_in in in_shapes:
            flat += K.broadcast_shape4(shape, s_in)
        shape4 = [1] * (4 - len(shape)) + list(shape) if len(shape) <= 4 else K.broadcast_shape4(shape, shape)
        imm_at = next((i for i, ins in enumerate(chain.insns) if ins.a_kind == K.IMM), -1)   # emit() puts it in slot a
        plan = plans[key] = ((_abi.PwInsn * len(chain.insns))(*chain.insns), len(chain.insns),
                             _abi.ptrs([0] * len(in_shapes)), _abi.i64(flat), len(in_shapes), _abi.ptrs([0]),
                             _abi.i64(shape4), imm_at, _abi.lib().ts_pointwise_chain)
    insns, n, in_ptrs, shapes, n_in, out_ptrs, shape4, imm_at, fn = plan
    for i, t in enumerate(in_tensors):
        in_ptrs[i] = _C.storage_ptr(t)
    out_ptrs[0] = _C.storage_ptr(out)
    if imm_at >= 0:
        insns[imm_at].a_imm = imm
    rc = fn(insns, n, in_ptrs, shapes, n_in, out_ptrs, 1, shape4, 0, 1.0, None, 0, 1, K._stream())
    if rc != 0:
        _abi.check(rc, "ts_pointwise_chain")
    return True


def _unary(op: str, x: torch.Tensor) -> torch.Tensor:
    _check_fp16(x)
    out = _new(x.shape, x)
    if x.numel() == 0:
        return out
    with _with_device(x):
        shape = tuple(x.shape)
        if _launch_cached(("u", op, shape), lambda c, t: c.emit("LOAD", t[0]).emit(op).store(0), shape, (shape,),
                          (x,), out):
            return out
        c = Chain()
        c.emit("LOAD", c.tensor(_st(x))).emit(op).store(0)
        K.run_chain(c, x.shape, outputs=[_st(out)])
    return out


def _operand(c: Chain, x, like: torch.Tensor):
    if _is_number(x):
        return c.imm(_number(x))
    if x.device != like.device:
        raise RuntimeError(f"expected all tensors on {like.device}, got {x.device}")
    _check_fp16(x)
    return c.tensor(_st(x))


def _binary(op: str, a, b, rop: Optional[str] = None, alpha=1) -> torch.Tensor:
    """a <op> (alpha * b); `rop` is the opcode to use when a is the scalar."""
    if _is_number(a):
        if rop is None:
            raise NotImplementedError(f"scalar {op} tensor")
        if alpha != 1:
            # scalar <op> (alpha * tensor): scale the tensor, then apply the reversed opcode
            _check_fp16(b)
            out = _new(b.shape, b)
            if out.numel() == 0:
                return out
            with _with_device(b):
                c = Chain()
                c.emit("LOAD", c.tensor(_st(b))).emit("MUL", c.imm(alpha)).emit(rop, c.imm(_number(a))).store(0)
                K.run_chain(c, b.shape, outputs=[_st(out)])
            return out
        a, b, op = b, a, rop
    _check_fp16(a)
    shape_b = () if _is_number(b) else tuple(b.shape)
    shape = _broadcast_shapes(tuple(a.shape), shape_b)
    out = _new(shape, a)
    if out.numel() == 0:
        return out
    with _with_device(a):
        if alpha == 1 or _is_number(b):
            sa = tuple(a.shape)
            if _is_number(b):
                if _launch_cached(("s", op, sa), lambda c, t: c.emit("LOAD", t[0]).emit(op, c.imm(0.0)).store(0),
                                  shape, (sa,), (a,), out, imm=_number(b) * alpha):
                    return out
            elif b.device == a.device and b.dtype == torch.float16:
                if _launch_cached(("b", op, sa, shape_b), lambda c, t: c.emit("LOAD", t[0]).emit(op, t[1]).store(0),
                                  shape, (sa, shape_b), (a, b), out):
                    return out
        c = Chain()
        if alpha != 1 and not _is_number(b):
            c.emit("LOAD", _operand(c, b, a)).emit("MUL", c.imm(alpha)).save(0)
            c.emit("LOAD", c.tensor(_st(a))).emit(op, c.saved(0)).store(0)
        else:
            rhs = c.imm(_number(b) * alpha) if _is_number(b) else None
            c.emit("LOAD", c.tensor(_st(a)))
            c.emit(op, rhs if rhs is not None else _operand(c, b, a)).store(0)
        K.run_chain(c, shape, outputs=[_st(out)])
    return out


_UNARY_OPS = {
    "abs": "ABS", "neg": "NEG", "exp": "EXP", "log": "LOG", "sqrt": "SQRT", "rsqrt": "RSQRT",
    "reciprocal": "RECIP", "sigmoid": "SIGMOID", "tanh": "TANH", "relu": "RELU", "silu": "SILU",
    "sin": "SIN", "cos": "COS", "erf": "ERF", "floor": "FLOOR", "ceil": "CEIL", "sign": "SIGN",
    "log1p": "LOG1P", "expm1": "EXPM1", "mish": "MISH", "logical_not": "LOGICAL_NOT",
}


def _copy_into(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    dst.copy_(src)
    return dst


def _register_unary(name: str, opcode: str) -> None:
    _impl(name)(lambda x: _unary(opcode, x))
    _impl(name + ".out")(lambda x, *, out: _copy_into(out, _unary(opcode, x)))
    _impl(name + "_")(lambda x: _copy_into(x, _unary(opcode, x)))


for _name, _opcode in _UNARY_OPS.items():
    _register_unary(_name, _opcode)


@_impl("gelu")
def _gelu(x, *, approximate="none"):
    return _unary("GELU_TANH" if approximate == "tanh" else "GELU", x)


@_impl("softplus")
def _softplus(x, beta=1, threshold=20):
    if float(beta) != 1.0 or float(threshold) != 20.0:
        raise NotImplementedError("softplus with beta != 1 or threshold != 20")
    return _unary("SOFTPLUS", x)


def _register_binary(name: str, opcode: str, rop: Optional[str], with_alpha: bool) -> None:
    if with_alpha:
        fn_t = lambda a, b, *, alpha=1: _binary(opcode, a, b, rop, alpha)  # noqa: E731
    else:
        fn_t = lambda a, b: _binary(opcode, a, b, rop)  # noqa: E731
    _impl(name + ".Tensor")(fn_t)
    _impl(name + ".Scalar")(fn_t)
    if with_alpha:
        _impl(name + ".out")(lambda a, b, *, alpha=1, out: _copy_into(out, fn_t(a, b, alpha=alpha)))
        _impl(name + "_.Tensor")(lambda a, b, *, alpha=1: _copy_into(a, fn_t(a, b, alpha=alpha)))
        _impl(name + "_.Scalar")(lambda a, b, alpha=1: _copy_into(a, fn_t(a, b, alpha=alpha)))
    else:
        _impl(name + ".out")(lambda a, b, *, out: _copy_into(out, fn_t(a, b)))
        _impl(name + "_.Tensor")(lambda a, b: _copy_into(a, fn_t(a, b)))
        _impl(name + "_.Scalar")(lambda a, b: _copy_into(a, fn_t(a, b)))


_register_binary("add", "ADD", "ADD", True)
_register_binary("sub", "SUB", "RSUB", True)
_register_binary("mul", "MUL", "MUL", False)
_register_binary("div", "DIV", "RDIV", False)

for _name, _opcode in {"eq": "EQ", "ne": "NE", "lt": "LT", "le": "LE", "gt": "GT", "ge": "GE"}.items():
    _impl(_name + ".Tensor")(lambda a, b, _o=_opcode: _binary(_o, a, b))
    _impl(_name + ".Scalar")(lambda a, b, _o=_opcode: _binary(_o, a, b))

_impl("maximum")(lambda a, b: _binary("MAX", a, b, "MAX"))
_impl("minimum")(lambda a, b: _binary("MIN", a, b, "MIN"))
_impl("pow.Tensor_Scalar")(lambda a, b: _binary("POW", a, b))
_impl("pow.Tensor_Tensor")(lambda a, b: _binary("POW", a, b))
# rsub(a, b, alpha) = b - alpha * a
_impl("rsub.Scalar")(lambda a, b, alpha=1: _binary("SUB", _number(b), a, "RSUB", alpha))


@_impl("where.self")
def _where(cond, a, b):
    _check_fp16(cond)
    like = cond
    shape = _broadcast_shapes(tuple(cond.shape), () if _is_number(a) else tuple(a.shape),
                                   () if _is_number(b) else tuple(b.shape))
    out = _new(shape, like)
    with _with_device(like):
        c = Chain()
        c.emit("LOAD", c.tensor(_st(cond)))
        c.emit("WHERE", _operand(c, a, like), _operand(c, b, like)).store(0)
        K.run_chain(c, shape, outputs=[_st(out)])
    return out


@_impl("fill_.Scalar")
def _fill(x, value):
    _check_fp16(x)
    if x.numel() == 0:
        return x
    target = x if _C.is_canonical(x) else _new(x.shape, x)
    with _with_device(x):
        c = Chain()
        c.emit("LOAD", c.imm(_number(value))).store(0)
        K.run_chain(c, target.shape if target.dim() else (1,), outputs=[_st(target)])
    if target is not x:
        x.copy_(target)
    return x


@_impl("zero_")
def _zero(x):
    return _fill(x, 0.0)


@_impl("clone")
def _clone(x, *, memory_format=None):
    out = _new(x.shape, x)
    out.copy_(x)
    return out


# ---- reductions ------------------------------------------------------------------------

def _reduce_one(x: torch.Tensor, dim: int, op: str, keepdim: bool, scale: float = 1.0) -> torch.Tensor:
    nd = x.dim()
    dim = dim % nd if nd else 0
    shape = list(x.shape) if nd else [1]
    out_shape = shape[:dim] + ([1] if keepdim else []) + shape[dim + 1:]
    if not out_shape:
        out_shape = [1]
    out = _new(out_shape, x)
    if x.numel() == 0:
        return out
    with _with_device(x):
        sx = _st(x)
        if dim == len(shape) - 1:
            c = Chain()
            c.emit("LOAD", c.tensor(sx))
            K.run_chain(c, shape, n_outputs=0, reduce=op, reduce_scale=scale, keepdim=keepdim,
                        red_out=_st(out))
        else:
            outer, red, inner = K._mid_view(shape, dim)
            nbytes = K._abi.lib().ts_reduce_mid_scratch_bytes(outer, red, inner)
            scratch = torch.empty(max(int(nbytes), 0), dtype=torch.uint8, device=sx.image.device) \
                if nbytes else None
            rc = K._abi.lib().ts_reduce_mid(sx.ptr(), _st(out).ptr(), outer, red, inner, K.RED[op],
                                            scale, scratch.data_ptr() if scratch is not None else None,
                                            K._stream())
            K._abi.check(rc, "ts_reduce_mid")
    return out


def _reduce(x: torch.Tensor, dims, op: str, keepdim: bool, mean: bool = False) -> torch.Tensor:
    _check_fp16(x)
    nd = max(x.dim(), 1)
    if dims is None or (isinstance(dims, (list, tuple)) and len(dims) == 0):
        dims = list(range(nd))
    if isinstance(dims, int):
        dims = [dims]
    dims = sorted({d % nd for d in dims}, reverse=True)
    count = 1
    for d in dims:
        count *= x.shape[d] if x.dim() else 1
    out = x
    for d in dims:  # innermost first, so earlier results keep their positions
        # a mean divides stage by stage: every fp16 intermediate is then a mean itself and stays
        # within the range of its inputs (partial sums would pass 65504 long before the end)
        extent = x.shape[d] if x.dim() else 1
        out = _reduce_one(out, d, op, keepdim, (1.0 / max(extent, 1)) if mean else 1.0)
    return out


@_impl("sum.dim_IntList")
def _sum_dim(x, dim, keepdim=False, *, dtype=None):
    return _reduce(x, dim, "sum", keepdim)


@_impl("sum")
def _sum_all(x, *, dtype=None):
    return _reduce(x, None, "sum", False)


@_impl("mean.dim")
def _mean_dim(x, dim, keepdim=False, *, dtype=None):
    return _reduce(x, dim, "sum", keepdim, mean=True)


@_impl("mean")
def _mean_all(x, *, dtype=None):
    return _reduce(x, None, "sum", False, mean=True)


@_impl("amax")
def _amax(x, dim=(), keepdim=False):
    return _reduce(x, list(dim), "max", keepdim)


@_impl("amin")
def _amin(x, dim=(), keepdim=False):
    return _reduce(x, list(dim), "min", keepdim)


@_impl("linalg_vector_norm")
def _vector_norm(x, ord=2, dim=None, keepdim=False, *, dtype=None):
    """1-, 2- and inf-norms.  fp16 cannot hold the squares of values it can hold, so the 2-norm
    is taken relative to the largest magnitude: amax * sqrt(mean((x / amax)^2)) * sqrt(N)."""
    _check_fp16(x)
    if ord in (float("inf"), 1, 1.0):
        return _reduce(_unary("ABS", x), dim, "max" if ord == float("inf") else "sum", keepdim)
    if ord not in (2, 2.0):
        raise NotImplementedError(f"linalg_vector_norm on spyre: ord={ord}")
    nd = max(x.dim(), 1)
    dims = list(range(nd)) if dim is None or len(dim) == 0 else sorted({d % nd for d in dim})
    shape = list(x.shape) if x.dim() else [1]
    count = 1
    for d in dims:
        count *= shape[d]
    kept = [1 if i in dims else n for i, n in enumerate(shape)]
    out_shape = kept if keepdim else ([n for i, n in enumerate(shape) if i not in dims] or [1])
    if x.numel() == 0 or count == 0:
        return torch.zeros(out_shape, dtype=x.dtype, device=x.device)
    x = x if x.dim() else x.reshape(1)
    amax = _binary("MAX", _reduce(_unary("ABS", x), dims, "max", True), 6e-8)   # never zero
    rel = _binary("DIV", x, amax)
    if dims == [nd - 1]:
        ms = _new(kept, x)
        with _with_device(x):
            c = Chain()
            c.emit("LOAD", c.tensor(_st(rel))).emit("SQUARE")
            K.run_chain(c, shape, n_outputs=0, reduce="sum", reduce_scale=1.0 / count, keepdim=True,
                        red_out=_st(ms))
    else:
        ms = _reduce(_unary("SQUARE", rel), dims, "sum", True, mean=True)
    out = _new(kept, x)
    with _with_device(x):
        c = Chain()
        c.emit("LOAD", c.tensor(_st(ms))).emit("SQRT").emit("MUL", c.imm(float(count) ** 0.5))
        c.emit("MUL", c.tensor(_st(amax))).store(0)
        K.run_chain(c, kept, outputs=[_st(out)])
    return out if keepdim else out.reshape(out_shape)


# ---- joining and masking ---------------------------------------------------------------

def _cuda_device(t: torch.Tensor) -> torch.device:
    return torch.device("cuda", t.device.index if t.device.index is not None else 0)


@_impl("cat")
def _cat(tensors, dim=0):
    """One image-to-image pass per input when the inputs land on stick boundaries of the result
    (any dim but the last, or widths that are multiples of a stick).  Otherwise the inputs are
    unpacked side by side into one row-major scratch tensor (the relayout kernel writes through
    any strides) which is then laid out as the result: two passes over the data."""
    tensors = [t for t in tensors if not (t.dim() == 1 and t.numel() == 0)]   # legacy empties
    if not tensors:
        raise RuntimeError("torch.cat(): expected a non-empty list of Tensors")
    like = tensors[0]
    nd = like.dim()
    if nd == 0:
        raise RuntimeError("zero-dimensional tensor cannot be concatenated")
    dim = dim % nd
    out_shape = list(like.shape)
    out_shape[dim] = 0
    for t in tensors:
        if t.device != like.device or t.dtype != like.dtype:
            raise RuntimeError("torch.cat on spyre: tensors must share device and dtype")
        if t.dim() != nd or any(t.shape[i] != like.shape[i] for i in range(nd) if i != dim):
            raise RuntimeError(f"Sizes of tensors must match except in dimension {dim}")
        out_shape[dim] += t.shape[dim]
    out = _new(out_shape, like)
    if out.numel() == 0:
        return out
    lanes = 128 // like.element_size()
    if dim != nd - 1 or all(t.shape[dim] % lanes == 0 for t in tensors[:-1]):
        # every input lands on stick boundaries of the result: one image-to-image pass each,
        # straight into its slice (pad lanes are zeroed by the slice that reaches the end)
        off = 0
        for t in tensors:
            n = t.shape[dim]
            if n:
                out.narrow(dim, off, n).copy_(t)
            off += n
        return out
    with _with_device(like):
        raw = torch.empty(out_shape, dtype=like.dtype, device=_cuda_device(like))
        off = 0
        for t in tensors:
            n = t.shape[dim]
            if n:
                K.from_sticks(_st(t), out=raw.narrow(dim, off, n))
            off += n
        K.to_sticks(raw, out=_st(out))
    return out


@_impl("stack")
def _stack(tensors, dim=0):
    nd = tensors[0].dim() + 1
    dim = dim % nd
    return _cat([t.unsqueeze(dim) for t in tensors], dim)


_tri_masks: dict = {}


def _tri(x: torch.Tensor, diagonal: int, lower: bool) -> torch.Tensor:
    """tril / triu as where(mask, x, 0) with a cached fp16 0/1 mask of the last two dims."""
    _check_fp16(x)
    if x.dim() < 2:
        raise RuntimeError("tril / triu: input tensor must have at least 2 dimensions")
    rows, cols = x.shape[-2], x.shape[-1]
    key = (rows, cols, int(diagonal), lower, x.device)
    mask = _tri_masks.get(key)
    if mask is None:
        ones = torch.ones(rows, cols, dtype=torch.float16)
        mask = (torch.tril(ones, diagonal) if lower else torch.triu(ones, diagonal)).to(x.device)
        if len(_tri_masks) > 16:
            _tri_masks.clear()
        _tri_masks[key] = mask
    return _where(mask, x, 0.0)


_impl("tril")(lambda x, diagonal=0: _tri(x, diagonal, True))
_impl("triu")(lambda x, diagonal=0: _tri(x, diagonal, False))


# ---- softmax / norms -------------------------------------------------------------------

def _softmax_impl(x, dim, log):
    _check_fp16(x)
    out = _new(x.shape, x)
    if x.numel() == 0:
        return out
    with _with_device(x):
        sx, so = _st(x), _st(out)
        nd = max(x.dim(), 1)
        d = dim % nd
        if d == nd - 1:
            K.softmax_rows(sx, log, out=so)
        else:
            outer, red, inner = K._mid_view(sx.shape, d)
            rc = K._abi.lib().ts_softmax_mid(sx.ptr(), so.ptr(), outer, red, inner, int(log), K._stream())
            K._abi.check(rc, "ts_softmax_mid")
    return out


@_impl("_softmax")
def _softmax(x, dim, half_to_float):
    if half_to_float:
        raise NotImplementedError("softmax with half_to_float")
    return _softmax_impl(x, dim, False)


@_impl("_log_softmax")
def _log_softmax(x, dim, half_to_float):
    if half_to_float:
        raise NotImplementedError("log_softmax with half_to_float")
    return _softmax_impl(x, dim, True)


@_impl("native_layer_norm")
def _native_layer_norm(x, normalized_shape, weight, bias, eps):
    _check_fp16(x)
    if len(normalized_shape) != 1 or normalized_shape[0] != x.shape[-1]:
        raise NotImplementedError("layer_norm over more than the last dim")
    out = _new(x.shape, x)
    with _with_device(x):
        K.layernorm_rows(_st(x), _st(weight) if weight is not None else None,
                         _st(bias) if bias is not None else None, float(eps), out=_st(out))
    stat_shape = list(x.shape[:-1]) + [1]
    # mean / rstd are only consumed by a backward pass, which this device does not run
    return out, _new(stat_shape, x), _new(stat_shape, x)


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
             round_before_weight: bool = True) -> torch.Tensor:
    """Fused RMSNorm over the last dim (module semantics by default: the normalised value is
    rounded to fp16 before the fp16 multiply by weight)."""
    _check_fp16(x)
    out = _new(x.shape, x)
    with _with_device(x):
        K.rmsnorm_rows(_st(x), _st(weight) if weight is not None else None, float(eps),
                       round_before_weight, out=_st(out))
    return out


# ---- matmul ----------------------------------------------------------------------------

def _weight_operand(b: torch.Tensor) -> Tuple[StickTensor, bool]:
    """(stick tensor, b_kmajor): a transposed view of a canonical [.., N, K] tensor is used in
    place, as the K-major operand of a @ b^T; anything else is laid out as [.., K, N]."""
    if b.dim() >= 2 and not _C.is_canonical(b):
        bt = b.transpose(-1, -2)
        if _C.is_canonical(bt):
            return _st(bt), True
    return _st(b), False


def _matmul(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _check_fp16(a, b)
    if a.shape[-1] != b.shape[-2]:
        raise RuntimeError(f"mat1 and mat2 shapes cannot be multiplied ({tuple(a.shape)} and {tuple(b.shape)})")
    shape = tuple(a.shape[:-1]) + (b.shape[-1],)
    given = out
    if out is None or tuple(out.shape) != shape or out.dtype != a.dtype or not _C.is_canonical(out) or \
            (residual is not None and out.data_ptr() == residual.data_ptr()):
        out = _new(shape, a)      # written here, then copied into the caller's tensor below
    if out.numel() == 0:
        return out if given is None else given
    out = _matmul_into(a, b, bias, residual, out)
    if given is not None and given is not out:
        given.copy_(out)
        return given
    return out


def _matmul_into(a, b, bias, residual, out):
    if out.numel() == 0:
        return out
    if a.shape[-1] == 0:
        return _fill(out, 0.0)
    with _with_device(a):
        sb, kmajor = _weight_operand(b)
        K.matmul(_st(a), sb, bias=_st(bias) if bias is not None else None, b_kmajor=kmajor,
                 out=_st(out), residual=_st(residual) if residual is not None else None)
    return out


@_impl("mm")
def _mm(a, b):
    return _matmul(a, b)


@_impl("bmm")
def _bmm(a, b):
    return _matmul(a, b)


@_impl("addmm")
def _addmm(bias, a, b, *, beta=1, alpha=1, out=None):
    if float(beta) == 1.0 and float(alpha) == 1.0 and bias.dim() == 1 and bias.shape[0] == b.shape[-1]:
        return _matmul(a, b, bias, out=out)
    if float(beta) == 1.0 and float(alpha) == 1.0 and a.dim() == 2 and a.shape[-1] > 0 and \
            tuple(bias.shape) == (a.shape[0], b.shape[-1]) and bias.dtype == torch.float16:
        return _matmul(a, b, residual=bias, out=out)     # matrix-shaped bias: added in the GEMM epilogue
    prod = _matmul(a, b)
    if float(alpha) != 1.0:
        prod = _binary("MUL", prod, float(alpha))
    res = prod if float(beta) == 0.0 else _binary("ADD", prod, bias, alpha=float(beta))
    return res if out is None else _copy_into(out, res)


# the out= forms are what a generated Inductor wrapper calls (extern_kernels.mm / bmm / addmm)
_impl("mm.out")(lambda a, b, *, out: _matmul(a, b, out=out))
_impl("bmm.out")(lambda a, b, *, out: _matmul(a, b, out=out))
_impl("addmm.out")(lambda bias, a, b, *, beta=1, alpha=1, out: _addmm(bias, a, b, beta=beta, alpha=alpha, out=out))


_CONVERTIBLE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _convert_on_device(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """fp16 / bf16 / fp32 conversion of a spyre tensor by the device kernel (no host round trip)."""
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    if x.numel() == 0:
        return out
    with _with_device(x):
        sx, so = _st(x), _st(out)
        rc = K._abi.lib().ts_convert_sticks(sx.ptr(), _CONVERTIBLE[x.dtype], so.ptr(), _CONVERTIBLE[dtype],
                                            sx.rows, sx.cols, K._stream())
        K._abi.check(rc, "ts_convert_sticks")
    return out


@_impl("_to_copy")
def _to_copy(x, *, dtype=None, layout=None, device=None, pin_memory=None, non_blocking=False,
             memory_format=None):
    device = torch.device(device) if device is not None else x.device
    dtype = dtype or x.dtype
    if dtype != x.dtype:
        if x.device.type == "cpu":
            # the data is on the host anyway: convert there, then it is an ordinary copy
            return x.to(dtype).to(device)
        if dtype not in _CONVERTIBLE or x.dtype not in _CONVERTIBLE:
            # as the reference's copy path (torch_spyre/csrc/spyre_mem.cpp:669-671)
            raise RuntimeError(f"Spyre backend does not support type conversion from {x.dtype} to {dtype} "
                               "on the device (float16, bfloat16 and float32 convert)")
        converted = _convert_on_device(x, dtype)
        return converted if device == x.device else converted.to(device)
    out = torch.empty(x.shape, dtype=dtype, device=device)
    out.copy_(x, non_blocking=non_blocking)
    return out


# ---- the rest of the reference's eager op list ------------------------------------------
# (codegen/inputs/Metadata.yaml: embedding :105, bitwise_not :31, repeat :245, _unsafe_view :325,
# upsample_nearest2d :331, native_dropout_backward :93; codegen/inputs/spyre_torch_ops.cpp:494-505:
# ne.Scalar_out and cumsum, which the reference bounces through the host)

@_impl("embedding")
def _embedding(weight, indices, padding_idx=-1, scale_grad_by_freq=False, sparse=False):
    """Row gather.  Indices: an int32 / int64 spyre tensor, or a host tensor (copied over)."""
    _check_fp16(weight)
    if weight.dim() != 2:
        raise RuntimeError("embedding: 'weight' must be 2-D")
    if indices.dtype not in (torch.int32, torch.int64):
        raise RuntimeError(f"embedding: indices must be int32 or int64, got {indices.dtype}")
    vocab, dim = weight.shape
    out = torch.empty(tuple(indices.shape) + (dim,), dtype=weight.dtype, device=weight.device)
    if out.numel() == 0:
        return out
    with _with_device(weight):
        if indices.device.type == "cpu":
            idx = indices.contiguous().to(_cuda_device(weight), non_blocking=False)
            ptr, is_image, rows, cols = idx.data_ptr(), 0, 1, idx.numel()
        else:
            idx = _st(indices if indices.dim() else indices.reshape(1))
            ptr, is_image, rows, cols = idx.ptr(), 1, idx.rows, idx.cols
        rc = K._abi.lib().ts_embedding_rows(_st(weight).ptr(), ptr, indices.element_size(), is_image, rows, cols,
                                            _st(out).ptr(), vocab, dim, K._stream())
        K._abi.check(rc, "ts_embedding_rows")
        del idx
    return out


@_impl("bitwise_not")
def _bitwise_not(x):
    """The device's masks are fp16 0 / 1 tensors (what its comparisons return), so this is the
    logical not, as the reference maps it (LogicalNot)."""
    if x.dtype != torch.float16:
        raise NotImplementedError(f"bitwise_not on spyre is defined for fp16 0/1 masks, got {x.dtype}")
    return _unary("LOGICAL_NOT", x)


for _name, _opcode in {"eq": "EQ", "ne": "NE", "lt": "LT", "le": "LE", "gt": "GT", "ge": "GE"}.items():
    _impl(_name + ".Scalar_out")(lambda a, b, *, out, _o=_opcode: _copy_into(out, _binary(_o, a, b)))
    _impl(_name + ".Tensor_out")(lambda a, b, *, out, _o=_opcode: _copy_into(out, _binary(_o, a, b)))


@_impl("_unsafe_view")
def _unsafe_view(x, size):
    return x.view(size)


@_impl("repeat")
def _repeat(x, repeats):
    """out viewed as [r0, s0, r1, s1, ...] takes x expanded over the r dims: one image-to-image
    pass when the innermost dim is not repeated, the general copy route otherwise."""
    repeats = [int(r) for r in repeats]
    if len(repeats) < x.dim():
        raise RuntimeError("Number of dimensions of repeat dims can not be smaller than number of "
                           "dimensions of tensor")
    shape = [1] * (len(repeats) - x.dim()) + list(x.shape)
    out_shape = [r * s for r, s in zip(repeats, shape)]
    out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    if out.numel() == 0:
        return out
    inter, src_shape = [], []
    for r, s in zip(repeats, shape):
        inter += [r, s]
        src_shape += [1, s]
    out.view(inter).copy_(x.reshape(src_shape).expand(inter))
    return out


@_impl("cumsum")
def _cumsum(x, dim, *, dtype=None):
    _check_fp16(x)
    if dtype not in (None, torch.float16):
        raise NotImplementedError("cumsum on spyre accumulates in fp32 and returns fp16")
    out = _new(x.shape, x)
    if x.numel() == 0:
        return out
    nd = max(x.dim(), 1)
    d = dim % nd
    with _with_device(x):
        sx, so = _st(x), _st(out)
        if d == nd - 1:
            rc = K._abi.lib().ts_cumsum_rows(sx.ptr(), so.ptr(), sx.rows, sx.cols, K._stream())
        else:
            outer, n, inner = K._mid_view(sx.shape, d)
            rc = K._abi.lib().ts_cumsum_mid(sx.ptr(), so.ptr(), outer, n, inner, K._stream())
        K._abi.check(rc, "ts_cumsum")
    return out


@_impl("upsample_nearest2d")
def _upsample_nearest2d(x, output_size, scales_h=None, scales_w=None):
    _check_fp16(x)
    if x.dim() != 4:
        raise RuntimeError("upsample_nearest2d expects a [N, C, H, W] tensor")
    n, c, ih, iw = x.shape
    oh, ow = (int(v) for v in output_size)
    for given, i, o in ((scales_h, ih, oh), (scales_w, iw, ow)):
        if given is not None and abs(float(given) - o / i) > 1e-6:
            raise NotImplementedError("upsample_nearest2d with scale factors that differ from the size ratio")
    out = torch.empty((n, c, oh, ow), dtype=x.dtype, device=x.device)
    if out.numel() == 0:
        return out
    with _with_device(x):
        rc = K._abi.lib().ts_upsample_nearest2d(_st(x).ptr(), _st(out).ptr(), n * c, ih, iw, oh, ow, K._stream())
        K._abi.check(rc, "ts_upsample_nearest2d")
    return out


@_impl("native_dropout")
def _native_dropout(x, p, train):
    """(x * mask / (1 - p), mask) with an fp16 0 / 1 mask drawn from the CUDA generator of the
    tensor's device; identity (mask of ones) when not training.  The reference returns its input
    untouched (codegen/inputs/spyre_torch_ops.cpp:186-194)."""
    _check_fp16(x)
    p = float(p)
    if not train or p == 0.0:
        return x.clone(), _fill(_new(x.shape, x), 1.0)
    if p >= 1.0:
        return _fill(_new(x.shape, x), 0.0), _fill(_new(x.shape, x), 0.0)
    with _with_device(x):
        keep = (torch.rand(tuple(x.shape) or (1,), device=_cuda_device(x)) >= p).to(torch.float16)
        mask = _new(x.shape, x)
        K.to_sticks(keep, out=_st(mask))
    return _native_dropout_backward(x, mask, 1.0 / (1.0 - p)), mask


@_impl("native_dropout_backward")
def _native_dropout_backward(grad, mask, scale):
    _check_fp16(grad, mask)
    out = _new(grad.shape, grad)
    if out.numel() == 0:
        return out
    with _with_device(grad):
        c = Chain()
        c.emit("LOAD", c.tensor(_st(grad))).emit("MUL", c.tensor(_st(mask))).emit("MUL", c.imm(float(scale))).store(0)
        K.run_chain(c, grad.shape, outputs=[_st(out)])
    return out
