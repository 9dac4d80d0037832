"""Runners: objects with ``run(*tensors)`` that the compiled graph calls.

The reference's runner hands a compiled graph file to ``_C.launch_kernel``
(torch_spyre/_inductor/runtime/kernel_runner.py:30-40); here the runner holds a fused program
and launches ``ts_pointwise_chain`` on the current stream."""
from __future__ import annotations

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

    def run(self, *inputs: torch.Tensor) -> List[torch.Tensor]:
        from ... import ops

        like = inputs[0]
        with torch.cuda.device(like.device.index or 0):
            sticks = [ops._st(t) for t in inputs]
            chain = K.Chain()
            chain.inputs = sticks
            for op, a, b in self.insns:
                chain.emit(op, a, b)
            outs = [torch.empty(self.shape, dtype=torch.float16, device=like.device)
                    for _ in range(self.n_outputs)]
            red = None
            if self.reduce:
                lead = list(self.shape[:-1])
                rshape = lead + [1] if self.keepdim else (lead or [1])
                red = torch.empty(rshape, dtype=torch.float16, device=like.device)
            K.run_chain(chain, self.shape, n_outputs=self.n_outputs, reduce=self.reduce,
                        reduce_scale=self.reduce_scale, keepdim=self.keepdim,
                        outputs=[ops._st(o) for o in outs],
                        red_out=ops._st(red) if red is not None else None)
        return outs + ([red] if red is not None else [])


def launch_kernel(spec, args):
    """Dispatcher behind ``_C.launch_kernel(spec, args)``: the last `n` tensors are outputs in
    the reference's convention; here a spec is run through its runner and the results returned."""
    if isinstance(spec, UnimplementedOp):
        raise RuntimeError(f"unimplemented operation {spec.op}")
    return SpyreFusedKernelRunner("launch_kernel", spec).run(*args)
