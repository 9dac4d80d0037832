"""Wrapper codegen class registered for the spyre device (reference: SpyrePythonWrapperCodegen,
torch_spyre/_inductor/wrapper.py:29-99).  The generated module imports the runtime's spec classes
and creates the ``async_compile`` object whose ``sdsc`` turns a KernelSpec into a runner."""
from __future__ import annotations

from torch._inductor.codegen.wrapper import PythonWrapperCodegen, SubgraphPythonWrapperCodegen
from torch._inductor.sizevars import SizeVarAllocator
from torch._inductor.virtualized import V


def noop_simplify_loops_impl(self, index_vars, sizes, index_formulas):
    """Keeps every loop dim as the graph has it.  Inductor would merge dims that are contiguous in
    its row-major picture of memory, but a spyre tensor is a stick image: which logical dim is the
    innermost one decides where an element lives, so [8192, 8192] and [67108864] are different
    layouts (same reason as the reference's wrapper.py:88-99)."""
    return sizes, lambda x: x, lambda x: x


class SpyrePythonWrapperCodegen(PythonWrapperCodegen):
    def __init__(self):
        super().__init__()
        V.graph.sizevars._simplify_loops_impl = noop_simplify_loops_impl.__get__(V.graph.sizevars, SizeVarAllocator)

    @staticmethod
    def create(is_subgraph=False, subgraph_name=None, parent_wrapper=None, partition_signatures=None):
        if is_subgraph:
            return SubgraphPythonWrapperCodegen(subgraph_name, parent_wrapper, partition_signatures)
        return SpyrePythonWrapperCodegen()

    def write_header(self) -> None:
        super().write_header()
        self.imports.splice(
            """
            import torch_spyre
            from torch_spyre._inductor.runtime import ConstantArg, TensorArg, KernelSpec, UnimplementedOp
            from torch_spyre._inductor.runtime.async_compile import SpyreAsyncCompile
            """,
            strip=True,
        )
        self.header.writeline("del async_compile")
        self.header.writeline("async_compile = SpyreAsyncCompile()")
