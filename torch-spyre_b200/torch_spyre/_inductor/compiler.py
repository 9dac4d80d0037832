"""Compiles an aten FX graph whose tensors live on ``spyre`` into a list of kernel launches.

Entry: ``SpyreAotAutograd`` (same hook as the reference, torch_spyre/_inductor/fake_ops.py:
243-255): when any example input is on spyre, the forward / inference compiler that AOT
autograd would hand to Inductor's Triton path is replaced by ``compile_graph`` below.  The
reference's pipeline at this point is lowering -> one SpyreKernel per node -> SuperDSC JSON ->
dxp_standalone -> launch_kernel (torch_spyre/_inductor/dsc.py:42-63,
runtime/async_compile.py:45-88, runtime/kernel_runner.py:30-40); here groups of pointwise
nodes (plus a trailing row reduction) become one ``KernelSpec`` each, resolved by
``SpyreAsyncCompile.sdsc`` to a launcher of the pre-built CUDA kernels, and every other aten
node is executed by the eager spyre kernels.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Sequence

import torch
from torch.fx import GraphModule, Node

from . import fusion
from .runtime import ConstantArg, KernelSpec, TensorArg
from .runtime.async_compile import SpyreAsyncCompile

aten = torch.ops.aten


def _outside_users(owner: Dict[Node, fusion.Group], g: fusion.Group):
    inside = set(g.nodes)

    def fn(n: Node) -> bool:
        for u in n.users:
            if u not in inside and u is not g.reduction:
                return True
            if u is g.reduction and n is not g.nodes[-1]:
                return True
        return False

    return fn


def spec_from_program(name: str, prog: fusion.Program) -> KernelSpec:
    args: List[Any] = []
    for i, n in enumerate(prog.inputs):
        args.append(TensorArg(True, i, torch.float16))
    n_out = len(prog.outputs) + (1 if prog.reduce else 0)
    for i in range(n_out):
        args.append(TensorArg(False, len(prog.inputs) + i, torch.float16))
    scales = [[1 if s != 1 else -1 for s in (fusion.node_shape(n) or ())] for n in prog.inputs]
    op_info = {
        "insns": prog.insns, "n_inputs": len(prog.inputs), "n_outputs": len(prog.outputs),
        "input_shapes": [fusion.node_shape(n) for n in prog.inputs],
        "reduce": prog.reduce, "reduce_scale": prog.reduce_scale, "keepdim": prog.keepdim,
    }
    return KernelSpec(op="fused_pointwise" + ("_rowreduce" if prog.reduce else ""),
                      is_reduction=prog.reduce is not None, dimensions=list(prog.shape), args=args,
                      scales=scales, op_info=op_info)


class CompiledGraph:
    """Executable plan: fused launches and eager aten calls in graph order."""

    def __init__(self, gm: GraphModule):
        self.gm = gm
        self.steps: List[Callable[[Dict[Node, Any]], None]] = []
        self.kernel_specs: List[KernelSpec] = []
        self.fused_nodes = 0
        self.placeholders: List[Node] = [n for n in gm.graph.nodes if n.op == "placeholder"]
        self.output_node: Node = next(n for n in gm.graph.nodes if n.op == "output")
        self._build()

    def _build(self) -> None:
        graph = self.gm.graph
        groups, owner = fusion.build_groups(graph)
        programs: Dict[int, fusion.Program] = {}
        async_compile = SpyreAsyncCompile()
        emitted: Dict[int, bool] = {}
        for gi, g in enumerate(groups):
            if len(g.nodes) == 1 and g.reduction is None:
                continue  # a lone op gains nothing over its eager kernel
            try:
                programs[id(g)] = fusion.linearise(g, _outside_users(owner, g))
            except (fusion.CannotFuse, Exception):
                continue
        for n in graph.nodes:
            if n.op in ("placeholder", "output"):
                continue
            g = owner.get(n)
            prog = programs.get(id(g)) if g is not None else None
            if prog is not None:
                last = g.reduction if g.reduction is not None else g.nodes[-1]
                if n is last and not emitted.get(id(g)):
                    emitted[id(g)] = True
                    name = f"spyre_fused_{len(self.kernel_specs)}"
                    spec = spec_from_program(name, prog)
                    self.kernel_specs.append(spec)
                    runner = async_compile.sdsc(name, spec)
                    self.fused_nodes += len(g.nodes) + (1 if g.reduction is not None else 0)
                    self.steps.append(self._fused_step(prog, runner))
                continue
            if n.op == "get_attr":
                self.steps.append(self._attr_step(n))
            elif n.op == "call_function":
                self.steps.append(self._call_step(n))
            else:
                raise RuntimeError(f"unsupported FX node {n.op}")

    def _attr_step(self, n: Node):
        value = getattr(self.gm, n.target)

        def step(env):
            env[n] = value

        return step

    @staticmethod
    def _call_step(n: Node):
        def step(env):
            args = torch.fx.node.map_arg(n.args, lambda a: env[a])
            kwargs = torch.fx.node.map_arg(n.kwargs, lambda a: env[a])
            env[n] = n.target(*args, **kwargs)

        return step

    @staticmethod
    def _fused_step(prog: fusion.Program, runner):
        out_nodes = list(prog.outputs) + ([prog.reduce_node] if prog.reduce else [])

        def step(env):
            results = runner.run(*[env[i] for i in prog.inputs])
            for node, value in zip(out_nodes, results):
                env[node] = value

        return step

    def __call__(self, args: Sequence[Any]):
        env: Dict[Node, Any] = {}
        for p, a in zip(self.placeholders, args):
            env[p] = a
        if isinstance(args, list):
            args.clear()
        for step in self.steps:
            step(env)
        return torch.fx.node.map_arg(self.output_node.args[0], lambda a: env[a])


def compile_graph(gm: GraphModule, example_inputs) -> Callable:
    from . import patterns

    patterns.rewrite_aten_graph(gm)
    compiled = CompiledGraph(gm)

    def run(args):
        return compiled(args)

    run._boxed_call = True
    run.compiled_graph = compiled
    last_compiled.append(compiled)
    del last_compiled[:-4]
    return run


# the most recent compiled graphs, for tests and debugging
last_compiled: List[CompiledGraph] = []


def spyre_decompositions():
    """Decompositions applied while tracing for spyre: everything the eager kernels do not
    implement directly is broken down; ops with a dedicated kernel are kept whole."""
    from torch._decomp import core_aten_decompositions

    table = dict(core_aten_decompositions())
    keep = [aten._softmax.default, aten._log_softmax.default, aten.native_layer_norm.default,
            aten.silu.default, aten.gelu.default, aten.mish.default, aten.addmm.default,
            aten.mean.dim, aten.amax.default, aten.amin.default, aten.rsub.Scalar, aten.softplus.default,
            aten.reciprocal.default, aten.rsqrt.default, aten.sigmoid.default, aten.tanh.default,
            aten.relu.default, aten.maximum.default, aten.minimum.default, aten.clone.default]
    for op in keep:
        table.pop(op, None)
    return table


def install_aot_hook() -> None:
    """Replaces dynamo's AotAutograd factory the way the reference does
    (torch_spyre/_inductor/__init__.py:88-90)."""
    import torch._dynamo.backends.common as common

    if getattr(common, "_spyre_hook_installed", False):
        return
    base = common.AotAutograd

    class SpyreAotAutograd(base):
        def __call__(self, gm: GraphModule, example_inputs, **kwargs):
            on_spyre = any(isinstance(t, torch.Tensor) and t.device.type == "spyre"
                           for t in example_inputs)
            if on_spyre:
                from . import patterns

                patterns.rewrite_dynamo_graph(gm)
                self.kwargs = dict(self.kwargs)
                self.kwargs["fw_compiler"] = compile_graph
                self.kwargs["inference_compiler"] = compile_graph
                self.kwargs.pop("bw_compiler", None)
                self.kwargs["decompositions"] = spyre_decompositions()
                self.kwargs.pop("partition_fn", None)
                self.kwargs.pop("cudagraphs", None)
            return super().__call__(gm, example_inputs, **kwargs)

    def factory(**kwargs):
        return SpyreAotAutograd(**kwargs)

    common.SpyreAotAutograd = SpyreAotAutograd
    common.aot_autograd = factory
    try:
        import torch._inductor.compile_fx as compile_fx

        if hasattr(compile_fx, "aot_autograd"):
            compile_fx.aot_autograd = factory
    except Exception:
        pass
    common._spyre_hook_installed = True
