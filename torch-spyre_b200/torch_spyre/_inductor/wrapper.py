"""Wrapper codegen class registered for the spyre device
(reference: SpyrePythonWrapperCodegen, torch_spyre/_inductor/wrapper.py:29-99)."""
from torch._inductor.codegen.wrapper import PythonWrapperCodegen


class SpyrePythonWrapperCodegen(PythonWrapperCodegen):
    @staticmethod
    def create(is_subgraph=False, subgraph_name=None, parent_wrapper=None, partition_signatures=None):
        return SpyrePythonWrapperCodegen()

    def write_header(self) -> None:
        super().write_header()
        self.imports.splice(
            """
            from torch_spyre._inductor.runtime import ConstantArg, TensorArg, KernelSpec, UnimplementedOp
            from torch_spyre._inductor.runtime.async_compile import SpyreAsyncCompile
            async_compile = SpyreAsyncCompile()
            """,
            strip=True,
        )
