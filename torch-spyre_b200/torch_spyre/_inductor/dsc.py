"""Scheduling class registered for the spyre device with Inductor.

The reference registers ``SuperDSCScheduling`` (a SIMDScheduling that emits one SuperDSC kernel per
node, torch_spyre/_inductor/dsc.py:28-63: ``define_kernel`` writes
``async_compile.sdsc(name, KernelSpec(...))`` into the wrapper and ``call_kernel`` writes
``name.run(args)``).  The same two lines are written here; what differs is the unit: Inductor's
scheduler is allowed to fuse pointwise nodes with each other and into a reduction over the
innermost dim (``can_fuse_*`` below; the reference's heuristics refuse every fusion,
torch_spyre/_inductor/choices.py:58-83), and the fused node becomes one program of the CUDA library
(``SpyreKernel``)."""
from __future__ import annotations

from torch._inductor.scheduler import BaseScheduling, BaseSchedulerNode, FusedSchedulerNode, SchedulerNode
from torch._inductor.utils import IndentedBuffer, get_fused_kernel_name, get_kernel_metadata
from torch._inductor.virtualized import V

from . import Unsupported
from .spyre_kernel import SpyreKernel


def _sizes(node: BaseSchedulerNode):
    """(pointwise sizes, reduction sizes) of a scheduler node as tuples of ints, or None."""
    try:
        _, (iters, reds) = node.group
        return tuple(int(s) for s in iters), tuple(int(s) for s in reds)
    except Exception:
        return None


def _is_scale_epilogue(node: SchedulerNode) -> bool:
    allowed = {"load", "constant", "to_dtype", "mul", "truediv", "store"}
    if len(node._body.subblocks):
        return False
    for n in node._body.root_block.graph.nodes:
        if n.op == "call_method" and n.target not in allowed:
            return False
        if n.op == "call_module" and n.target != "get_index":
            return False
    return True


class SuperDSCScheduling(BaseScheduling):
    dsc_type: str = "sdsc"

    def __init__(self, scheduler=None):
        super().__init__(scheduler)

    # -- fusion ---------------------------------------------------------------------------
    def group_fn(self, sizes):
        return tuple(tuple(V.graph.sizevars.simplify(s) for s in size) for size in sizes)

    def can_fuse_vertical(self, node1: BaseSchedulerNode, node2: BaseSchedulerNode) -> bool:
        """Producer node1 into consumer node2: pointwise into pointwise over the same iteration
        space, or pointwise into a reduction over the innermost dim of that space."""
        s1, s2 = _sizes(node1), _sizes(node2)
        if s1 is None or s2 is None or node1.is_template() or node2.is_template():
            return False
        if node1.is_reduction():
            # a sum followed by a scaling of its result by constants (what mean lowers to)
            return (not node2.is_reduction() and s2 == (s1[0], ()) and isinstance(node2, SchedulerNode)
                    and _is_scale_epilogue(node2))
        if any(isinstance(n, SchedulerNode) and len(n._body.subblocks) for n in list(node1.get_nodes()) + list(node2.get_nodes())):
            return False
        if not node2.is_reduction():
            return s1 == s2
        return len(s2[1]) == 1 and s1[1] == () and s1[0] == s2[0] + s2[1]

    def can_fuse_horizontal(self, node1: BaseSchedulerNode, node2: BaseSchedulerNode) -> bool:
        # two kernels that merely share an input gain nothing from sharing a launch here
        return False

    # -- code generation ------------------------------------------------------------------
    def define_kernel(self, src_code: str, node_schedule, summary) -> str:
        """Writes ``name = async_compile.sdsc('name', KernelSpec(...))`` into the wrapper header."""
        wrapper = V.graph.wrapper_code
        if src_code in wrapper.src_to_kernel:
            return wrapper.src_to_kernel[src_code]
        fused_name = get_fused_kernel_name(node_schedule, "original_aten")
        kernel_name = "_".join([self.dsc_type, fused_name, wrapper.next_kernel_suffix()])
        wrapper.src_to_kernel[src_code] = kernel_name
        buf = IndentedBuffer()
        buf.writeline(f"async_compile.{self.dsc_type}('{kernel_name}',")
        with buf.indent():
            buf.splice(src_code)
        buf.writeline(")")
        origins, detailed_origins = get_kernel_metadata(node_schedule, wrapper)
        layouts = IndentedBuffer()
        layouts.writeline(f"{wrapper.comment} Argument Layouts:")
        for i, acc in enumerate(summary.inputs + summary.outputs + ([summary.reduction_out] if summary.reduction_out else [])):
            buffer = V.graph.try_get_buffer(acc.name)
            if buffer is not None:
                layouts.writeline(f"{wrapper.comment}   {i}: {buffer.get_layout()} viewed as {list(acc.shape)}")
        wrapper.define_kernel(kernel_name, buf.getvalue(), f"{origins}\n{detailed_origins}\n{layouts.getvalue().rstrip()}")
        return kernel_name

    @staticmethod
    def spec_source(spec) -> str:
        buf = IndentedBuffer()
        buf.writeline("KernelSpec(")
        with buf.indent():
            buf.writeline(f"op={spec.op!r},")
            buf.writeline(f"is_reduction={spec.is_reduction!r},")
            buf.writeline(f"dimensions={spec.dimensions!r},")
            buf.writeline(f"scales={spec.scales!r},")
            buf.writeline(f"op_info={spec.op_info!r},")
            buf.writeline("args=[")
            with buf.indent():
                for arg in spec.args:
                    buf.writeline(f"{arg!r},")
            buf.writeline("]")
        buf.writeline(")")
        return buf.getvalue()

    def codegen_node(self, node: BaseSchedulerNode) -> None:
        nodes = [n for n in node.get_nodes() if isinstance(n, SchedulerNode)]
        if len(nodes) != len(list(node.get_nodes())):
            raise Unsupported(f"scheduler node {type(node).__name__} with members that are not loop nodes")
        fused_names = OrderedNames(n.get_name() for n in nodes)

        def removable(buffer_name: str) -> bool:
            # an intermediate that no later kernel and no graph output reads is never stored
            return bool(isinstance(node, FusedSchedulerNode) and
                        V.graph.scheduler.can_buffer_be_removed_through_fusion(buffer_name, fused_names.as_set()))

        kernel = SpyreKernel(nodes, removable)
        summary = kernel.summarize()
        if kernel.scaled_from is not None and not removable(kernel.scaled_from):
            raise Unsupported("an unscaled reduction result that is also needed outside its kernel")
        for name in list(kernel.values) + ([kernel.scaled_from] if kernel.scaled_from else []):
            if removable(name):
                V.graph.removed_buffers.add(name)
        for n in nodes:
            n.mark_run()      # allocates the node's output buffers in the wrapper
        kernel_name = self.define_kernel(self.spec_source(summary.spec), nodes, summary)
        wrapper = V.graph.wrapper_code
        call_args = [a.name for a in summary.inputs] + [a.name for a in summary.outputs]
        if summary.reduction_out is not None:
            call_args.append(summary.reduction_out.name)
        wrapper.writeline(f"{kernel_name}.run({', '.join(call_args)})")
        self.free_buffers_in_scheduler()

    def codegen_template(self, template_node, epilogue_nodes, prologue_nodes=None, **kwargs):
        raise Unsupported("Inductor templates on spyre")

    def codegen_sync(self) -> None:
        pass

    def flush(self) -> None:
        pass

    def ready_to_flush(self) -> bool:
        return False

    def get_backend_features(self, device):
        return {}

    def benchmark_fused_nodes(self, nodes):
        raise Unsupported("benchmarking fused nodes on spyre")


class OrderedNames(list):
    def as_set(self):
        from torch.utils._ordered_set import OrderedSet

        return OrderedSet(self)
