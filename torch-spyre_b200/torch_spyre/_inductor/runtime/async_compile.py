"""``SpyreAsyncCompile``: turns a KernelSpec into a runner.

The reference writes a SuperDSC JSON file and shells out to its backend compiler
(torch_spyre/_inductor/runtime/async_compile.py:45-88).  The CUDA kernels are compiled ahead
of time, so "compiling" a spec is resolving it to a launcher; nothing runs in a subprocess."""
from __future__ import annotations

from . import KernelSpec, UnimplementedOp
from .kernel_runner import SpyreFusedKernelRunner, SpyreUnimplementedRunner


# When a list is installed here, every spec handed to sdsc() is appended to it (the compiler uses
# this to know which kernels a generated wrapper defined).
capture = None


class SpyreAsyncCompile:
    def __init__(self) -> None:
        pass

    def sdsc(self, kernel_name: str, ks):
        if capture is not None:
            capture.append(ks)
        if isinstance(ks, UnimplementedOp):
            print(f"WARNING: Compiling unimplemented {ks.op} to runtime exception")
            return SpyreUnimplementedRunner(kernel_name, ks.op)
        if isinstance(ks, KernelSpec) and ks.op.startswith("fused_pointwise"):
            return SpyreFusedKernelRunner(kernel_name, ks)
        return SpyreUnimplementedRunner(kernel_name, getattr(ks, "op", str(ks)))

    def wait(self, scope) -> None:
        pass
