"""Lowerings the spyre backend adds to Inductor for the duration of one of its compilations
(reference: torch_spyre/_inductor/lowering.py:25-153, which registers its lowerings process-wide
at import time).

* Ops that have a dedicated kernel stay whole: ``_softmax``, ``_log_softmax``, ``native_layer_norm``
  (and ``mish`` / ``softplus``) become fallback kernels that call the eager spyre op, where
  Inductor would otherwise want them decomposed into several pointwise and reduction kernels.
* ``silu`` and ``rsub.Scalar``, which the spyre decomposition table keeps whole for the pattern
  rewrites, are lowered to pointwise loop bodies so that they fuse with their neighbours.
* ``mm`` / ``bmm`` / ``addmm`` keep Inductor's own lowering: an extern kernel call with ``out=``,
  served by the eager ``mm.out`` / ``bmm.out`` / ``addmm.out`` registrations.

Everything registered here is removed again when the compilation ends, so Inductor's behaviour for
other devices in the same process is left as it was."""
from __future__ import annotations

import contextlib

import torch
import torch._inductor.lowering as L
from torch._inductor.virtualized import ops

aten = torch.ops.aten

KEPT_WHOLE = (aten._softmax.default, aten._log_softmax.default, aten.native_layer_norm.default,
              aten.mish.default, aten.softplus.default)


def _silu(x):
    fn = L.make_pointwise(lambda v: ops.mul(v, ops.sigmoid(v)))
    return fn(x)


def _rsub_scalar(x, other, alpha=1):
    def inner(v):
        scaled = v if alpha == 1 else ops.mul(v, ops.constant(float(alpha), torch.float16))
        return ops.sub(ops.constant(float(other), torch.float16), scaled)

    return L.make_pointwise(inner)(x)


POINTWISE = {aten.silu.default: _silu, aten.rsub.Scalar: _rsub_scalar}


@contextlib.contextmanager
def spyre_lowerings():
    saved_lowerings = dict(L.lowerings)
    saved_fallbacks = set(L.fallbacks)
    try:
        for op in KEPT_WHOLE:
            L.lowerings.pop(op, None)
            L.make_fallback(op, override_decomp=True, warn=False)
        for op, fn in POINTWISE.items():
            L.lowerings.pop(op, None)
            L.register_lowering(op, type_promotion_kind=None)(fn)
        yield
    finally:
        L.lowerings.clear()
        L.lowerings.update(saved_lowerings)
        L.fallbacks.clear()
        L.fallbacks.update(saved_fallbacks)
