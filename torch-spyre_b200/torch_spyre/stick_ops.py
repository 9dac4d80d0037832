"""Kernel launches over stick images held in CUDA memory.

A ``StickTensor`` is a logical fp16 tensor plus the flat CUDA buffer holding its
stick image (generic SpyreTensorLayout: [ceil(cols/64)][leading dims...][64], pad
lanes zero).  Every function here is a thin argument-marshalling layer over one
C-ABI entry point; PyTorch is used for device memory and streams only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import _abi
from ._abi import PwInsn
from .layout import SpyreTensorLayout

# Opcode / operand-kind numbers of include/spyre_b200.h.
NONE, TENSOR, IMM, SAVED = 0, 1, 2, 3
_OPS = ("LOAD SAVE STORE ADD SUB RSUB MUL DIV RDIV MAX MIN POW EQ NE LT LE GT GE WHERE NEG ABS "
        "EXP LOG SQRT RSQRT RECIP SIGMOID TANH RELU SILU GELU GELU_TANH SQUARE LOGICAL_NOT SIN "
        "COS ERF FLOOR CEIL SIGN LOG1P EXPM1 SOFTPLUS MISH").split()
OP = {name: i for i, name in enumerate(_OPS)}
RED = {None: 0, "sum": 1, "max": 2, "min": 3}


def _stream() -> int:
    """Raw handle of the current CUDA stream of the current device (the direct binding: the Stream
    object torch.cuda.current_stream() builds costs several microseconds per launch)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


@dataclass
class StickTensor:
    image: torch.Tensor          # flat CUDA tensor holding the stick image
    shape: Tuple[int, ...]       # logical (host) shape
    dtype: torch.dtype = torch.float16

    @property
    def layout(self) -> SpyreTensorLayout:
        return SpyreTensorLayout(list(self.shape) if self.shape else [1], self.dtype)

    @property
    def rows(self) -> int:
        n = 1
        for s in self.shape[:-1]:
            n *= s
        return n

    @property
    def cols(self) -> int:
        return self.shape[-1] if self.shape else 1

    def ptr(self) -> int:
        return self.image.data_ptr()


def empty(shape: Sequence[int], dtype: torch.dtype = torch.float16, device=None) -> StickTensor:
    shape = tuple(int(s) for s in shape)
    lay = SpyreTensorLayout(list(shape) if shape else [1], dtype)
    n = 0 if any(s == 0 for s in shape) else lay.numel()
    return StickTensor(torch.empty(n, dtype=dtype, device=device or "cuda"), shape, dtype)


def _layout_args(lay: SpyreTensorLayout):
    return (_abi.i64(lay.device_size), _abi.i64(lay.device_strides), _abi.i32(lay.dim_map),
            len(lay.device_size))


def to_sticks(raw: torch.Tensor, layout: Optional[SpyreTensorLayout] = None,
              out: Optional[StickTensor] = None) -> StickTensor:
    """raw: CUDA tensor of any strides (a device-resident image of a host tensor)."""
    shape = tuple(raw.shape) if raw.dim() else (1,)
    strides = tuple(raw.stride()) if raw.dim() else (1,)
    lay = layout or SpyreTensorLayout(list(shape), raw.dtype)
    if out is None:
        out = StickTensor(torch.empty(lay.numel(), dtype=raw.dtype, device=raw.device), shape,
                          raw.dtype)
    ds, dst, dm, nd = _layout_args(lay)
    rc = _abi.lib().ts_relayout_to_sticks(raw.data_ptr(), out.ptr(), raw.element_size(),
                                          _abi.i64(shape), _abi.i64(strides), len(shape),
                                          ds, dst, dm, nd, _stream())
    _abi.check(rc, "ts_relayout_to_sticks")
    return out


def from_sticks(st: StickTensor, out: Optional[torch.Tensor] = None,
                layout: Optional[SpyreTensorLayout] = None) -> torch.Tensor:
    """Returns (or fills) a CUDA tensor with the logical contents; ``out`` may have any strides."""
    shape = st.shape if st.shape else (1,)
    if out is None:
        out = torch.empty(shape, dtype=st.dtype, device=st.image.device)
    lay = layout or st.layout
    ds, dst, dm, nd = _layout_args(lay)
    rc = _abi.lib().ts_relayout_from_sticks(st.ptr(), out.data_ptr(), out.element_size(),
                                            _abi.i64(shape), _abi.i64(tuple(out.stride())),
                                            len(shape), ds, dst, dm, nd, _stream())
    _abi.check(rc, "ts_relayout_from_sticks")
    return out


def host_span(t: torch.Tensor) -> int:
    shape = tuple(t.shape) if t.dim() else (1,)
    strides = tuple(t.stride()) if t.dim() else (1,)
    n = _abi.lib().ts_host_span_bytes(t.element_size(), _abi.i64(shape), _abi.i64(strides),
                                      len(shape))
    if n < 0:
        _abi.check(int(n), "ts_host_span_bytes")
    return int(n)


def _staging_for(t: torch.Tensor, staging: Optional[torch.Tensor], device) -> torch.Tensor:
    """A staging block for the pipelined copies: the caller's if it is large enough for two
    chunks, else a fresh one of the size the library asks for."""
    shape = tuple(t.shape) if t.dim() else (1,)
    strides = tuple(t.stride()) if t.dim() else (1,)
    want = int(_abi.lib().ts_copy_staging_bytes(t.element_size(), _abi.i64(shape), _abi.i64(strides), len(shape)))
    if want < 0:
        _abi.check(want, "ts_copy_staging_bytes")
    if staging is not None and staging.numel() * staging.element_size() >= want:
        return staging
    return torch.empty(max(want, 256), dtype=torch.uint8, device=device)


def copy_host_to_sticks(host: torch.Tensor, out: Optional[StickTensor] = None,
                        staging: Optional[torch.Tensor] = None) -> StickTensor:
    """Host tensor (any non-negative strides; pinned memory makes the copy asynchronous)
    -> stick image on the current CUDA device, in chunks whose PCIe copies overlap the relayout
    kernels.  A tensor that cannot be cut into chunks goes in one piece."""
    shape = tuple(host.shape) if host.dim() else (1,)
    strides = tuple(host.stride()) if host.dim() else (1,)
    lay = SpyreTensorLayout(list(shape), host.dtype)
    if out is None:
        out = empty(shape, host.dtype)
    staging = _staging_for(host, staging, out.image.device)
    nbytes = staging.numel() * staging.element_size()
    ds, dst, dm, nd = _layout_args(lay)
    args = (host.element_size(), _abi.i64(shape), _abi.i64(strides), len(shape), ds, dst, dm, nd, _stream())
    rc = _abi.lib().ts_copy_host_to_sticks_pipelined(host.data_ptr(), staging.data_ptr(), nbytes, out.ptr(), *args)
    if rc == _abi.TS_ERR_TOO_LARGE:      # not cuttable: the whole span through one staging block
        staging = torch.empty(max(host_span(host), 16), dtype=torch.uint8, device=out.image.device)
        rc = _abi.lib().ts_copy_host_to_sticks(host.data_ptr(), staging.data_ptr(), out.ptr(), *args)
    _abi.check(rc, "ts_copy_host_to_sticks")
    return out


def copy_sticks_to_host(st: StickTensor, host: torch.Tensor,
                        staging: Optional[torch.Tensor] = None) -> torch.Tensor:
    shape = st.shape if st.shape else (1,)
    strides = tuple(host.stride()) if host.dim() else (1,)
    staging = _staging_for(host, staging, st.image.device)
    nbytes = staging.numel() * staging.element_size()
    ds, dst, dm, nd = _layout_args(st.layout)
    args = (host.element_size(), _abi.i64(shape), _abi.i64(strides), len(shape), ds, dst, dm, nd, _stream())
    rc = _abi.lib().ts_copy_sticks_to_host_pipelined(st.ptr(), staging.data_ptr(), nbytes, host.data_ptr(), *args)
    if rc == _abi.TS_ERR_TOO_LARGE:
        staging = torch.empty(max(host_span(host), 16), dtype=torch.uint8, device=st.image.device)
        rc = _abi.lib().ts_copy_sticks_to_host(st.ptr(), staging.data_ptr(), host.data_ptr(), *args)
    _abi.check(rc, "ts_copy_sticks_to_host")
    return host


# ---- row-wise ops ---------------------------------------------------------------

def softmax_rows(x: StickTensor, log: bool = False, out: Optional[StickTensor] = None) -> StickTensor:
    out = out or empty(x.shape, x.dtype, x.image.device)
    rc = _abi.lib().ts_softmax_rows(x.ptr(), out.ptr(), x.rows, x.cols, int(log), _stream())
    _abi.check(rc, "ts_softmax_rows")
    return out


def layernorm_rows(x: StickTensor, weight: Optional[StickTensor], bias: Optional[StickTensor],
                   eps: float, out: Optional[StickTensor] = None) -> StickTensor:
    out = out or empty(x.shape, x.dtype, x.image.device)
    rc = _abi.lib().ts_layernorm_rows(x.ptr(), weight.ptr() if weight else None,
                                      bias.ptr() if bias else None, out.ptr(), x.rows, x.cols,
                                      eps, _stream())
    _abi.check(rc, "ts_layernorm_rows")
    return out


def rmsnorm_rows(x: StickTensor, weight: Optional[StickTensor], eps: float,
                 round_before_weight: bool = True, out: Optional[StickTensor] = None) -> StickTensor:
    out = out or empty(x.shape, x.dtype, x.image.device)
    rc = _abi.lib().ts_rmsnorm_rows(x.ptr(), weight.ptr() if weight else None, out.ptr(), x.rows,
                                    x.cols, eps, int(round_before_weight), _stream())
    _abi.check(rc, "ts_rmsnorm_rows")
    return out


# ---- non-stick-dim ops ----------------------------------------------------------

def _mid_view(shape: Sequence[int], dim: int) -> Tuple[int, int, int]:
    """[outer][red][inner] view of the stick image for a reduction over `dim` (not the last)."""
    nsticks = -(-shape[-1] // 64)
    a = 1
    for s in shape[:dim]:
        a *= s
    b = 1
    for s in shape[dim + 1:-1]:
        b *= s
    return nsticks * a, shape[dim], b * 64


def reduce_mid(x: StickTensor, dim: int, op: str, scale: float = 1.0, keepdim: bool = False) -> StickTensor:
    outer, red, inner = _mid_view(x.shape, dim)
    new_shape = list(x.shape)
    if keepdim:
        new_shape[dim] = 1
    else:
        del new_shape[dim]
    out = empty(new_shape, x.dtype, x.image.device)
    nbytes = _abi.lib().ts_reduce_mid_scratch_bytes(outer, red, inner)
    if nbytes < 0:
        _abi.check(int(nbytes), "ts_reduce_mid_scratch_bytes")
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.image.device) if nbytes else None
    rc = _abi.lib().ts_reduce_mid(x.ptr(), out.ptr(), outer, red, inner, RED[op], scale,
                                  scratch.data_ptr() if scratch is not None else None, _stream())
    _abi.check(rc, "ts_reduce_mid")
    return out


def softmax_mid(x: StickTensor, dim: int, log: bool = False) -> StickTensor:
    outer, red, inner = _mid_view(x.shape, dim)
    out = empty(x.shape, x.dtype, x.image.device)
    rc = _abi.lib().ts_softmax_mid(x.ptr(), out.ptr(), outer, red, inner, int(log), _stream())
    _abi.check(rc, "ts_softmax_mid")
    return out


def softmax(x: StickTensor, dim: int, log: bool = False) -> StickTensor:
    nd = len(x.shape)
    dim = dim % nd
    return softmax_rows(x, log) if dim == nd - 1 else softmax_mid(x, dim, log)


# ---- fused pointwise chains -----------------------------------------------------

class Chain:
    """Builder for a ts_pointwise_chain program."""

    def __init__(self):
        self.insns: List[PwInsn] = []
        self.inputs: List[StickTensor] = []

    def tensor(self, t: StickTensor) -> Tuple[int, int, float]:
        for i, u in enumerate(self.inputs):
            if u is t:
                return (TENSOR, i, 0.0)
        self.inputs.append(t)
        return (TENSOR, len(self.inputs) - 1, 0.0)

    @staticmethod
    def imm(v: float) -> Tuple[int, int, float]:
        return (IMM, 0, float(v))

    @staticmethod
    def saved(k: int) -> Tuple[int, int, float]:
        return (SAVED, k, 0.0)

    def emit(self, op: str, a=(NONE, 0, 0.0), b=(NONE, 0, 0.0)) -> "Chain":
        self.insns.append(PwInsn(OP[op], a[0], a[1], b[0], b[1], a[2], b[2]))
        return self

    def save(self, k: int) -> "Chain":
        return self.emit("SAVE", (NONE, k, 0.0))

    def store(self, k: int = 0) -> "Chain":
        return self.emit("STORE", (NONE, k, 0.0))


def _shape4(shape: Sequence[int], ref4: Optional[Sequence[int]] = None) -> List[int]:
    """Collapse a logical shape to [d0, d1, d2, cols] (leading dims merged into d0)."""
    shape = list(shape) if len(shape) else [1]
    cols = shape[-1]
    lead = shape[:-1]
    while len(lead) > 3:
        lead = [lead[0] * lead[1]] + lead[2:]
    lead = [1] * (3 - len(lead)) + lead
    return lead + [cols]


def broadcast_shape4(out_shape: Sequence[int], in_shape: Sequence[int]) -> List[int]:
    """Operand shape aligned (from the right) to out_shape, as the 4 numbers the ABI wants.
    Only works when the out shape has at most 4 dims or leading dims can be merged safely."""
    out_shape = list(out_shape) if len(out_shape) else [1]
    in_shape = list(in_shape) if len(in_shape) else [1]
    in_full = [1] * (len(out_shape) - len(in_shape)) + in_shape
    if len(out_shape) <= 4:
        return [1] * (4 - len(out_shape)) + in_full
    # merge leading dims beyond 4: only legal if the operand is uniform over them
    extra = len(out_shape) - 4
    head_out, head_in = out_shape[:extra + 1], in_full[:extra + 1]
    if all(a == b for a, b in zip(head_out, head_in)):
        merged = 1
        for v in head_in:
            merged *= v
    elif all(b == 1 for b in head_in):
        merged = 1
    else:
        raise _abi.SpyreKernelError("broadcast pattern needs more than 4 iteration dims")
    return [merged] + in_full[extra + 1:]


def prepare_chain(chain: Chain, out_shape: Sequence[int], n_outputs: int = 1,
                  reduce: Optional[str] = None, reduce_scale: float = 1.0,
                  keepdim: bool = False, outputs: Optional[List[StickTensor]] = None,
                  red_out: Optional[StickTensor] = None):
    """Allocates outputs and marshals every argument once.  Returns (launch, outputs,
    reduced output); launch() enqueues the kernel on the current stream."""
    out_shape = tuple(out_shape) if len(out_shape) else (1,)
    if len(out_shape) <= 4:
        shape4 = [1] * (4 - len(out_shape)) + list(out_shape)
    else:
        shape4 = broadcast_shape4(out_shape, out_shape)
    if chain.inputs:
        dev = chain.inputs[0].image.device
    elif outputs:
        dev = outputs[0].image.device
    else:
        dev = torch.device("cuda")
    if outputs is None:
        outputs = [empty(out_shape, torch.float16, dev) for _ in range(n_outputs)]
    in_shapes: List[int] = []
    for t in chain.inputs:
        in_shapes += broadcast_shape4(out_shape, t.shape)
    red_inner = 1
    if reduce is not None:
        lead = list(out_shape[:-1])
        if keepdim:
            red_out = red_out or empty(lead + [1], torch.float16, dev)
        else:
            red_out = red_out or empty(lead if lead else [1], torch.float16, dev)
            red_inner = lead[-1] if lead else 1
    else:
        red_out = None
    insns = (PwInsn * len(chain.insns))(*chain.insns)
    args = (insns, len(chain.insns), _abi.ptrs([t.ptr() for t in chain.inputs]),
            _abi.i64(in_shapes), len(chain.inputs), _abi.ptrs([o.ptr() for o in outputs]),
            len(outputs), _abi.i64(shape4), RED[reduce], reduce_scale,
            red_out.ptr() if red_out is not None else None, int(keepdim), red_inner)
    fn = _abi.lib().ts_pointwise_chain
    keep = (chain, outputs, red_out)  # the launch closure keeps every buffer alive

    def launch():
        rc = fn(*args, _stream())
        if rc != 0:
            _abi.check(rc, "ts_pointwise_chain")
        return keep

    return launch, outputs, red_out


def run_chain(chain: Chain, out_shape: Sequence[int], n_outputs: int = 1,
              reduce: Optional[str] = None, reduce_scale: float = 1.0,
              keepdim: bool = False, outputs: Optional[List[StickTensor]] = None,
              red_out: Optional[StickTensor] = None
              ) -> Tuple[List[StickTensor], Optional[StickTensor]]:
    """Launches the chain over `out_shape`.  Returns (full-shape outputs, reduced output)."""
    launch, outs, red = prepare_chain(chain, out_shape, n_outputs, reduce, reduce_scale, keepdim,
                                      outputs, red_out)
    launch()
    return outs, red


# ---- matmul ---------------------------------------------------------------------

def matmul(a: StickTensor, b: StickTensor, bias: Optional[StickTensor] = None,
           b_kmajor: bool = False, out: Optional[StickTensor] = None,
           residual: Optional[StickTensor] = None) -> StickTensor:
    """a: [..., M, K].  b: [K, N] or [batch..., K, N] (b_kmajor=False), or [N, K] /
    [batch..., N, K] (b_kmajor=True, i.e. a @ b^T).  fp32 accumulation, fp16 result; `residual`
    (shaped like the result) is added to the rounded product in the epilogue."""
    if len(a.shape) < 2 or len(b.shape) < 2:
        raise _abi.SpyreKernelError("matmul operands need at least 2 dims")
    M, K = a.shape[-2], a.shape[-1]
    if b_kmajor:
        N, Kb = b.shape[-2], b.shape[-1]
    else:
        Kb, N = b.shape[-2], b.shape[-1]
    if K != Kb:
        raise _abi.SpyreKernelError(f"matmul shape mismatch: {a.shape} x {b.shape}")
    batch = 1
    for s in a.shape[:-2]:
        batch *= s
    b_batched = len(b.shape) > 2
    if b_batched:
        nb = 1
        for s in b.shape[:-2]:
            nb *= s
        if nb != batch:
            raise _abi.SpyreKernelError("batched matmul needs equal batch extents")
    else:
        # a shared B sees [batch*M, K] as one matrix
        M, batch = M * batch, 1
    if out is None:
        out = empty(tuple(a.shape[:-1]) + (N,), torch.float16, a.image.device)
    if residual is not None:
        if tuple(residual.shape) != tuple(out.shape):
            raise _abi.SpyreKernelError(f"residual shape {residual.shape} != result shape {out.shape}")
        rc = _abi.lib().ts_gemm_f16_residual(a.ptr(), b.ptr(), bias.ptr() if bias is not None else None,
                                             residual.ptr(), out.ptr(), batch, M, N, K, int(b_kmajor),
                                             int(b_batched), _stream())
        _abi.check(rc, "ts_gemm_f16_residual")
        return out
    rc = _abi.lib().ts_gemm_f16(a.ptr(), b.ptr(), bias.ptr() if bias is not None else None,
                                out.ptr(), batch, M, N, K, int(b_kmajor), int(b_batched),
                                _stream())
    _abi.check(rc, "ts_gemm_f16")
    return out


def matmul_scatter_add(a: StickTensor, b: StickTensor, owner_ptrs: Sequence[int], b_kmajor: bool = True) -> None:
    """Partial product a[M, K_local] @ b added, block of rows by block of rows, into the result
    buffers at `owner_ptrs` (device addresses of fp16 stick images of [M / len(owner_ptrs), N]; this
    GPU's or peers').  See ts_gemm_f16_scatter_add for what the caller has to order."""
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-2] if b_kmajor else b.shape[-1]
    rc = _abi.lib().ts_gemm_f16_scatter_add(a.ptr(), b.ptr(), _abi.ptrs(list(owner_ptrs)), len(owner_ptrs), M, N, K,
                                            int(b_kmajor), _stream())
    _abi.check(rc, "ts_gemm_f16_scatter_add")


def matmul_scatter_store(a: StickTensor, b: StickTensor, slot_ptrs: Sequence[int], b_kmajor: bool = True) -> None:
    """Partial product a[M, K_local] @ b stored, block of rows by block of rows, at `slot_ptrs`: the
    address, inside each owner's memory, of the [M / len(slot_ptrs), N] image reserved for this rank.
    See ts_gemm_f16_scatter_store for what the caller has to order."""
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-2] if b_kmajor else b.shape[-1]
    rc = _abi.lib().ts_gemm_f16_scatter_store(a.ptr(), b.ptr(), _abi.ptrs(list(slot_ptrs)), len(slot_ptrs), M, N, K,
                                              int(b_kmajor), _stream())
    _abi.check(rc, "ts_gemm_f16_scatter_store")


def sum_slots(slots: torch.Tensor, n_slots: int, shape: Sequence[int], residual: Optional[StickTensor] = None,
              out: Optional[StickTensor] = None) -> StickTensor:
    """Sum of `n_slots` stick images of `shape` lying back to back in `slots` (a flat fp16 CUDA tensor),
    plus `residual`, in fp32 with one rounding."""
    if out is None:
        out = empty(tuple(shape), torch.float16, slots.device)
    n = out.image.numel()
    if slots.numel() < n_slots * n:
        raise _abi.SpyreKernelError("sum_slots: the slot buffer is smaller than n_slots images")
    rc = _abi.lib().ts_sum_slots_f16(slots.data_ptr(), n_slots, n, residual.ptr() if residual is not None else None,
                                     out.ptr(), n, _stream())
    _abi.check(rc, "ts_sum_slots_f16")
    return out


def swiglu_matmul(a: StickTensor, w_gate_up: StickTensor, out: Optional[StickTensor] = None) -> StickTensor:
    """silu(a @ Wg^T) * (a @ Wu^T) in one GEMM.  a: [..., M, K]; w_gate_up: [2*N, K], rows alternating
    between Wg and Wu in blocks of 64 (see ``interleave_gate_up``)."""
    K = a.shape[-1]
    n_out = w_gate_up.shape[0] // 2
    if w_gate_up.shape[1] != K or n_out % 64:
        raise _abi.SpyreKernelError(f"swiglu_matmul: weight {w_gate_up.shape} does not fit input {a.shape}")
    m = 1
    for s in a.shape[:-1]:
        m *= s
    if out is None:
        out = empty(tuple(a.shape[:-1]) + (n_out,), torch.float16, a.image.device)
    rc = _abi.lib().ts_gemm_f16_swiglu(a.ptr(), w_gate_up.ptr(), out.ptr(), 1, m, n_out, K, _stream())
    _abi.check(rc, "ts_gemm_f16_swiglu")
    return out


# ---- row gather -----------------------------------------------------------------------

def embedding_rows(table: StickTensor, ids: torch.Tensor) -> StickTensor:
    """out[i, :] = table[ids[i], :] for the flattened `ids` (int32 or int64, contiguous, on the
    table's GPU).  An index outside the table gives a row of zeros and raises the flag that
    `ts_gather_error_state` reports."""
    if len(table.shape) != 2:
        raise _abi.SpyreKernelError("embedding_rows: the table must be 2-D")
    if ids.dtype not in (torch.int32, torch.int64) or ids.device != table.image.device or not ids.is_contiguous():
        raise _abi.SpyreKernelError("embedding_rows: ids must be contiguous int32 / int64 on the table's GPU")
    vocab, dim = table.shape
    out = empty((ids.numel(), dim), torch.float16, table.image.device)
    rc = _abi.lib().ts_embedding_rows(table.ptr(), ids.data_ptr(), ids.element_size(), 0, 1, ids.numel(),
                                      out.ptr(), vocab, dim, _stream())
    _abi.check(rc, "ts_embedding_rows")
    return out


# ---- attention pieces -------------------------------------------------------------

def rotary(x: StickTensor, cos: StickTensor, sin: StickTensor, batch: int, seq: int, heads: int,
           head_dim: int = 128, out: Optional[StickTensor] = None) -> StickTensor:
    """x: [batch, seq, heads*head_dim]; cos / sin: [seq, head_dim]."""
    out = out or empty(x.shape, x.dtype, x.image.device)
    rc = _abi.lib().ts_rotary_f16(x.ptr(), cos.ptr(), sin.ptr(), out.ptr(), batch, seq, heads,
                                  head_dim, _stream())
    _abi.check(rc, "ts_rotary_f16")
    return out


# False routes every shape through the three-launch path (kept for comparison in tests / bench)
fused_attention = True

# the only head size the attention kernels are built for (their tensor maps span 2 sticks a head)
ATTENTION_HEAD_DIM = 128


def check_attention_args(q_shape, k_shape, v_shape, heads: int, dtypes, out_shape=None,
                         batch: Optional[int] = None, seq: Optional[int] = None) -> None:
    """Host-side validation done before any attention launch: the kernels index q / k / v / out
    as [batch, seq, heads*128] fp16 images of one common shape, so anything else would make them
    read and write outside the buffers."""
    q_shape, k_shape, v_shape = tuple(q_shape), tuple(k_shape), tuple(v_shape)
    if len(q_shape) != 3:
        raise _abi.SpyreKernelError(f"causal_attention: q must be [batch, seq, heads*head_dim], got {q_shape}")
    if k_shape != q_shape or v_shape != q_shape:
        raise _abi.SpyreKernelError(
            f"causal_attention: q, k and v must have one shape, got {q_shape}, {k_shape}, {v_shape}")
    if out_shape is not None and tuple(out_shape) != q_shape:
        raise _abi.SpyreKernelError(f"causal_attention: out shape {tuple(out_shape)} != q shape {q_shape}")
    if heads < 1 or q_shape[2] != heads * ATTENTION_HEAD_DIM:
        raise _abi.SpyreKernelError(
            f"causal_attention: width {q_shape[2]} with {heads} heads is head_dim "
            f"{q_shape[2] / max(heads, 1):g}; the kernel is built for head_dim {ATTENTION_HEAD_DIM} only")
    if any(d != torch.float16 for d in dtypes):
        raise _abi.SpyreKernelError(f"causal_attention: float16 only, got {tuple(dtypes)}")
    if (batch is not None and batch != q_shape[0]) or (seq is not None and seq != q_shape[1]):
        raise _abi.SpyreKernelError(
            f"causal_attention: batch {batch} x seq {seq} does not match q shape {q_shape}")


def causal_attention(q: StickTensor, k: StickTensor, v: StickTensor, batch: int, seq: int,
                     heads: int, scale: float, out: Optional[StickTensor] = None,
                     scores: Optional[torch.Tensor] = None) -> StickTensor:
    """Causal scaled-dot-product attention over packed [batch, seq, heads*128] q / k / v images.

    One fused kernel (scores stay on the SM).  With ``fused_attention`` off, three launches
    for all heads together: scores = q k^T (tcgen05 GEMM reading the heads out of the packed
    images), masked softmax in place, out = probs v written straight into the packed output
    image; `scores` is scratch of heads*batch*seq*seq fp16 elements for that path."""
    hd = ATTENTION_HEAD_DIM
    check_attention_args(q.shape, k.shape, v.shape, heads, (q.dtype, k.dtype, v.dtype),
                         out.shape if out is not None else None, batch, seq)
    dev = q.image.device
    rows = batch * seq
    out = out or empty((batch, seq, heads * hd), torch.float16, dev)
    if fused_attention:
        rc = _abi.lib().ts_attention_causal_f16(q.ptr(), k.ptr(), v.ptr(), out.ptr(), batch, seq,
                                                heads, hd, float(scale), _stream())
        _abi.check(rc, "ts_attention_causal_f16")
        return out
    if scores is None:
        scores = torch.empty(heads * rows * seq, dtype=torch.float16, device=dev)
    packed_stick, packed_head = rows * 64, 2 * rows * 64          # q / k / v / out images
    sc_stick, sc_head = heads * rows * 64, rows * 64              # scores as [heads*batch*seq, seq]
    lib = _abi.lib()
    rc = lib.ts_gemm_f16_ex(q.ptr(), packed_stick, packed_head, k.ptr(), packed_stick, packed_head,
                            None, scores.data_ptr(), sc_stick, sc_head, heads, batch, seq, seq, hd,
                            1, 1, _stream())
    _abi.check(rc, "ts_gemm_f16_ex (q k^T)")
    rc = lib.ts_softmax_rows_causal(scores.data_ptr(), scores.data_ptr(), heads * rows, seq, seq,
                                    float(scale), _stream())
    _abi.check(rc, "ts_softmax_rows_causal")
    rc = lib.ts_gemm_f16_ex(scores.data_ptr(), sc_stick, sc_head, v.ptr(), packed_stick, packed_head,
                            None, out.ptr(), packed_stick, packed_head, heads, batch, seq, hd, seq,
                            0, 1, _stream())
    _abi.check(rc, "ts_gemm_f16_ex (probs v)")
    return out
