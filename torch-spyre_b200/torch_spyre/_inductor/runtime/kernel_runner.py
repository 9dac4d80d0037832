"""Runners: objects with ``run(*tensors)`` that the compiled graph calls.

The reference's runner hands a compiled graph file to ``_C.launch_kernel``
(torch_spyre/_inductor/runtime/kernel_runner.py:30-40); here the runner holds a fused program
and launches ``ts_pointwise_chain`` on the current stream."""
from __future__ import annotations

import math
from typing import List

import torch

from ... import stick_ops as K
from . import KernelSpec, UnimplementedOp


class SpyreUnimplementedRunner:
    def __init__(self, name: str, op: str):
        self.name, self.op = name, op

    def run(self, *args, **kw):
        raise RuntimeError(f"Invoked {self.name} which contains unimplemented operation {self.op}")


class SpyreFusedKernelRunner:
    """One fused pointwise(+row reduction) group."""

    def __init__(self, name: str, spec: KernelSpec):
        self.name, self.spec = name, spec
        info = spec.op_info
        self.shape = tuple(spec.dimensions)
        self.insns = info["insns"]
        self.n_outputs = info["n_outputs"]
        self.reduce = info["reduce"]
        self.reduce_scale = info["reduce_scale"]
        self.keepdim = info["keepdim"]
        self._plans = {}      # input shapes -> marshalled constant arguments of the launch

    def run(self, *tensors: torch.Tensor) -> List[torch.Tensor]:
        """run(*inputs) allocates and returns the results; run(*inputs, *outputs[, reduced output])
        writes into the given buffers, outputs last: the convention of a generated wrapper
        (torch_spyre/_inductor/spyre_kernel.py:362-369 of the reference)."""
        from ... import ops

        info = self.spec.op_info
        n_in = info["n_inputs"]
        inputs, given = tensors[:n_in], tensors[n_in:]
        like = inputs[0] if inputs else given[0]
        n_results = self.n_outputs + (1 if self.reduce else 0)
        if given and len(given) != n_results:
            raise RuntimeError(f"{self.name}: expected {n_in} inputs and {n_results} outputs, got {len(tensors)} tensors")
        shapes = info.get("input_shapes") or [None] * n_in
        fast = self._run_marshalled(inputs, given, shapes, like)
        if fast is not None:
            return fast
        with ops._with_device(like):
            # an operand is the buffer viewed with the shape its index expression walks
            sticks = [ops._st(t if s is None or tuple(t.shape) == tuple(s) else t.reshape(tuple(s)))
                      for t, s in zip(inputs, shapes)]
            chain = K.Chain()
            chain.inputs = sticks
            for op, a, b in self.insns:
                chain.emit(op, a, b)
            lead = list(self.shape[:-1])
            rshape = lead + [1] if self.keepdim else (lead or [1])
            if given:
                outs = [self._as_image(t, self.shape) for t in given[:self.n_outputs]]
                red = self._as_image(given[-1], rshape) if self.reduce else None
            else:
                outs = [torch.empty(self.shape, dtype=torch.float16, device=like.device)
                        for _ in range(self.n_outputs)]
                red = torch.empty(rshape, dtype=torch.float16, device=like.device) if self.reduce else None
            K.run_chain(chain, self.shape, n_outputs=self.n_outputs, reduce=self.reduce,
                        reduce_scale=self.reduce_scale, keepdim=self.keepdim,
                        outputs=[ops._st(o) for o in outs],
                        red_out=ops._st(red) if red is not None else None)
        return list(outs) + ([red] if red is not None else [])

    def _run_marshalled(self, inputs, given, shapes, like):
        """The common case without any per-call building: every tensor is its own stick image and
        already has the shape the program walks it with, so a launch is the cached constant
        arguments plus the tensors' addresses.  Returns None when a tensor needs the general path
        (a view to materialise, a reshape)."""
        from ... import _C, ops

        eff = []          # the shape each operand is walked with
        for t, s in zip(inputs, shapes):
            mine = tuple(t.shape) if t.dim() else (1,)
            want = mine if s is None else (tuple(s) if len(s) else (1,))
            # a different shape over the same bytes: equal innermost extents (leading dims merge freely)
            if t.numel() == 0 or not _C.is_canonical(t) or t.numel() != math.prod(want) or \
                    (want != mine and want[-1] != mine[-1]):
                return None
            eff.append(want)
        lead = list(self.shape[:-1])
        rshape = lead + [1] if self.keepdim else (lead or [1])
        if given:
            def holds(buffer, shape):      # the buffer's own image is the image of `shape`
                mine = tuple(buffer.shape) if buffer.dim() else (1,)
                return _C.is_canonical(buffer) and buffer.numel() == math.prod(shape) and \
                    (mine == tuple(shape) or mine[-1] == tuple(shape)[-1])

            if not all(holds(t, self.shape) for t in given[:self.n_outputs]):
                return None
            if self.reduce and not holds(given[-1], tuple(rshape)):
                return None
        key = tuple(eff)
        plan = self._plans.get(key)
        if plan is None:
            out_shape = self.shape if len(self.shape) else (1,)
            shape4 = ([1] * (4 - len(out_shape)) + list(out_shape)) if len(out_shape) <= 4 \
                else K.broadcast_shape4(out_shape, out_shape)
            in_shapes = []
            for shape in eff:
                in_shapes += K.broadcast_shape4(out_shape, shape)
            chain = K.Chain()
            for op, a, b in self.insns:
                chain.emit(op, a, b)
            insns = (K.PwInsn * len(chain.insns))(*chain.insns)
            red_inner = (lead[-1] if lead else 1) if (self.reduce is not None and not self.keepdim) else 1
            plan = (insns, len(chain.insns), K._abi.i64(in_shapes), len(inputs), K._abi.i64(shape4),
                    K.RED[self.reduce], float(self.reduce_scale), int(self.keepdim), red_inner)
            self._plans[key] = plan
        insns, n_insns, in_shapes, n_in, shape4, red_code, red_scale, keepdim, red_inner = plan
        with ops._with_device(like):
            if given:
                outs = list(given[:self.n_outputs])
                red = given[-1] if self.reduce else None
            else:
                outs = [torch.empty(self.shape, dtype=torch.float16, device=like.device) for _ in range(self.n_outputs)]
                red = torch.empty(rshape, dtype=torch.float16, device=like.device) if self.reduce else None
            rc = K._abi.lib().ts_pointwise_chain(
                insns, n_insns, K._abi.ptrs([t.data_ptr() for t in inputs]), in_shapes, n_in,
                K._abi.ptrs([t.data_ptr() for t in outs]), len(outs), shape4, red_code, red_scale,
                red.data_ptr() if red is not None else None, keepdim, red_inner, K._stream())
            if rc != 0:
                K._abi.check(rc, "ts_pointwise_chain")
        return list(outs) + ([red] if red is not None else [])

    @staticmethod
    def _as_image(buffer: torch.Tensor, shape) -> torch.Tensor:
        """An output buffer the wrapper allocated, viewed with the kernel's iteration shape.  The
        kernel writes the stick image of that shape, so the buffer's own image must be the same
        bytes: equal innermost extents (leading dims merge freely)."""
        from ... import _C

        t = buffer if tuple(buffer.shape) == tuple(shape) else buffer.view(tuple(shape))
        if not _C.is_canonical(t):
            raise RuntimeError(f"output buffer of shape {tuple(buffer.shape)} cannot hold the stick image of {tuple(shape)}")
        return t


def launch_kernel(spec, args):
    """Dispatcher behind ``_C.launch_kernel(spec, args)``: the last `n` tensors are outputs in
    the reference's convention; here a spec is run through its runner and the results returned."""
    if isinstance(spec, UnimplementedOp):
        raise RuntimeError(f"unimplemented operation {spec.op}")
    return SpyreFusedKernelRunner("launch_kernel", spec).run(*args)
