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


class _Unit:
    """One schedulable piece of the plan: a fused group or a single FX node."""

    __slots__ = ("produces", "needs", "make_step", "first")

    def __init__(self, produces, needs, make_step, first):
        self.produces, self.needs, self.make_step, self.first = produces, needs, make_step, first


def _arg_reader(a, slot: Dict[Node, int]):
    """Compiles one FX argument into (is_constant, value-or-reader): nodes become slot reads,
    lists / tuples of nodes become readers that rebuild the container, the rest is constant."""
    if isinstance(a, Node):
        i = slot[a]
        return False, (lambda env: env[i])
    if isinstance(a, (list, tuple)):
        parts = [_arg_reader(x, slot) for x in a]
        if all(c for c, _ in parts):
            return True, a
        kind = type(a)
        return False, (lambda env: kind(v if c else v(env) for c, v in parts))
    if isinstance(a, dict):
        parts = {k: _arg_reader(v, slot) for k, v in a.items()}
        if all(c for c, _ in parts.values()):
            return True, a
        return False, (lambda env: {k: (v if c else v(env)) for k, (c, v) in parts.items()})
    if isinstance(a, slice):
        parts = [_arg_reader(x, slot) for x in (a.start, a.stop, a.step)]
        if all(c for c, _ in parts):
            return True, a
        return False, (lambda env: slice(*[(v if c else v(env)) for c, v in parts]))
    return True, a


class CompiledGraph:
    """Executable plan: fused launches and eager aten calls, in an order that respects every
    data dependency.  Values live in a flat slot list; each step's arguments are compiled once
    into slot reads, and a value's slot is cleared after its last reader so that its memory goes
    back to the allocator while the graph is still running."""

    route = "plan"

    def __init__(self, gm: GraphModule):
        self.gm = gm
        self.steps: List[Callable[[list], None]] = []
        self.kernel_specs: List[KernelSpec] = []
        self.fused_nodes = 0
        self.placeholders: List[Node] = [n for n in gm.graph.nodes if n.op == "placeholder"]
        self.output_node: Node = next(n for n in gm.graph.nodes if n.op == "output")
        self.slot: Dict[Node, int] = {n: i for i, n in enumerate(gm.graph.nodes)}
        self._build()

    # -- planning ------------------------------------------------------------------------
    def _units(self) -> List[_Unit]:
        graph = self.gm.graph
        order = {n: i for i, n in enumerate(graph.nodes)}
        groups, owner = fusion.build_groups(graph)
        programs: Dict[int, fusion.Program] = {}
        for g in groups:
            if len(g.nodes) == 1 and g.reduction is None:
                continue  # a lone op gains nothing over its eager kernel
            try:
                programs[id(g)] = fusion.linearise(g, _outside_users(owner, g))
            except (fusion.CannotFuse, Exception):
                continue
        units: List[_Unit] = []
        seen: Dict[int, bool] = {}
        for n in graph.nodes:
            if n.op in ("placeholder", "output"):
                continue
            g = owner.get(n)
            prog = programs.get(id(g)) if g is not None else None
            if prog is not None:
                if not seen.get(id(g)):
                    seen[id(g)] = True
                    members = list(g.nodes) + ([g.reduction] if g.reduction is not None else [])
                    units.append(_Unit(members, list(prog.inputs),
                                       (lambda prog=prog, members=members: self._fused_step(prog, len(members))),
                                       order[members[0]]))
                continue
            if n.op == "get_attr":
                units.append(_Unit([n], [], (lambda n=n: self._attr_step(n)), order[n]))
            elif n.op == "call_function":
                units.append(_Unit([n], list(n.all_input_nodes), (lambda n=n: self._call_step(n)), order[n]))
            else:
                raise RuntimeError(f"unsupported FX node {n.op}")
        return units

    @staticmethod
    def _schedule(units: List[_Unit], ready: Sequence[Node]) -> List[_Unit]:
        """Stable topological order: at every point the unit that comes first in the graph among
        those whose inputs exist.  A fused group needs the inputs of all its members at once, so
        it may have to run later than its first member and earlier than an outside reader of
        one of its stored values."""
        have = set(ready)
        pending = sorted(units, key=lambda u: u.first)
        out: List[_Unit] = []
        while pending:
            for i, u in enumerate(pending):
                if all(d in have for d in u.needs):
                    out.append(pending.pop(i))
                    have.update(u.produces)
                    break
            else:
                raise fusion.CannotFuse("fused groups depend on each other")
        return out

    def _build(self) -> None:
        try:
            plan = self._schedule(self._units(), self.placeholders)
        except fusion.CannotFuse:
            # cannot happen while build_groups keeps groups acyclic; run unfused if it ever does
            saved = fusion.is_pointwise
            fusion.is_pointwise = lambda n: False
            try:
                plan = self._schedule(self._units(), self.placeholders)
            finally:
                fusion.is_pointwise = saved
        for u in plan:
            self.steps.append(u.make_step())
        self._plan_frees(plan)

    def _plan_frees(self, plan: List[_Unit]) -> None:
        """After each step, clear the slots whose last reader that step was."""
        keep = set()
        torch.fx.node.map_arg(self.output_node.args[0], lambda a: keep.add(a) or a)
        last_reader: Dict[Node, int] = {}
        for i, u in enumerate(plan):
            for d in u.needs:
                last_reader[d] = i
            for p in u.produces:
                last_reader.setdefault(p, i)
        frees: List[List[int]] = [[] for _ in plan]
        for node, i in last_reader.items():
            if node not in keep:
                frees[i].append(self.slot[node])
        self.frees = [tuple(f) for f in frees]

    # -- steps ---------------------------------------------------------------------------
    def _attr_step(self, n: Node):
        value = getattr(self.gm, n.target)
        i = self.slot[n]

        def step(env):
            env[i] = value

        return step

    def _call_step(self, n: Node):
        target, i = n.target, self.slot[n]
        args = [_arg_reader(a, self.slot) for a in n.args]
        kwargs = {k: _arg_reader(v, self.slot) for k, v in n.kwargs.items()}
        if not kwargs and all(not c for c, _ in args) and len(args) <= 3:
            readers = [v for _, v in args]
            if len(readers) == 1:
                r0 = readers[0]

                def step(env):
                    env[i] = target(r0(env))
            elif len(readers) == 2:
                r0, r1 = readers

                def step(env):
                    env[i] = target(r0(env), r1(env))
            else:
                def step(env):
                    env[i] = target(*[r(env) for r in readers])
            return step

        def step(env):
            env[i] = target(*[(v if c else v(env)) for c, v in args],
                            **{k: (v if c else v(env)) for k, (c, v) in kwargs.items()})

        return step

    def _fused_step(self, prog: fusion.Program, n_members: int):
        name = f"spyre_fused_{len(self.kernel_specs)}"
        spec = spec_from_program(name, prog)
        self.kernel_specs.append(spec)
        runner = SpyreAsyncCompile().sdsc(name, spec)
        self.fused_nodes += n_members
        out_slots = [self.slot[n] for n in list(prog.outputs) + ([prog.reduce_node] if prog.reduce else [])]
        in_slots = [self.slot[n] for n in prog.inputs]

        def step(env):
            results = runner.run(*[env[i] for i in in_slots])
            for i, value in zip(out_slots, results):
                env[i] = value

        return step

    def __call__(self, args: Sequence[Any]):
        env: list = [None] * len(self.slot)
        for p, a in zip(self.placeholders, args):
            env[self.slot[p]] = a
        if isinstance(args, list):
            args.clear()
        for step, free in zip(self.steps, self.frees):
            step(env)
            for i in free:
                env[i] = None
        slot = self.slot
        return torch.fx.node.map_arg(self.output_node.args[0], lambda a: env[slot[a]])


# "inductor": lower through Inductor itself (scheduler fusion, generated wrapper calling
# async_compile.sdsc / runner.run), falling back to the FX-level plan below when Inductor meets
# something the spyre scheduling cannot express; "plan": always the FX-level plan.
backend_mode = "inductor"
# what the last compilations used, newest last ("inductor" / "plan: <why>"), for tests
last_routes: List[str] = []


def compile_graph(gm: GraphModule, example_inputs) -> Callable:
    from . import patterns

    patterns.rewrite_aten_graph(gm)
    if backend_mode == "inductor":
        try:
            run = compile_with_inductor(gm, example_inputs)
            last_routes.append("inductor")
            del last_routes[:-8]
            return run
        except Exception as e:  # Unsupported from the scheduling, or an Inductor lowering that has no spyre form
            last_routes.append(f"plan: {type(e).__name__}: {str(e)[:200]}")
            del last_routes[:-8]
    return compile_with_plan(gm, example_inputs)


def compile_with_inductor(gm: GraphModule, example_inputs) -> Callable:
    """The aten graph goes through stock Inductor: lowering, its scheduler's fusion, then
    SuperDSCScheduling / SpyrePythonWrapperCodegen (registered for the device) write the wrapper."""
    import copy

    import torch._inductor.config as inductor_config
    from torch._inductor.compile_fx import compile_fx_inner
    from torch._inductor.virtualized import V

    from .choices import SpyreHeuristics

    patches = {"split_reductions": False, "keep_output_stride": False, "benchmark_harness": False,
               "permute_fusion": False, "fx_graph_cache": False, "implicit_fallbacks": True,
               "triton.cudagraphs": False, "size_asserts": False, "nan_asserts": False}
    gm_copy = copy.deepcopy(gm)     # Inductor edits the graph it is given; the plan fallback wants the original
    from .lowering import spyre_lowerings

    from .runtime import async_compile

    specs: List[KernelSpec] = []
    saved_capture, async_compile.capture = async_compile.capture, specs
    try:
        with inductor_config.patch(patches), V.set_choices_handler(SpyreHeuristics()), spyre_lowerings():
            run = compile_fx_inner(gm_copy, example_inputs)
    finally:
        async_compile.capture = saved_capture
    last_compiled.append(InductorCompiled(gm, specs))
    del last_compiled[:-4]
    return run


class InductorCompiled:
    """What a compilation through Inductor left behind, for tests and debugging: the aten graph it
    was given and the specs of the kernels its wrapper defined."""

    route = "inductor"

    def __init__(self, gm: GraphModule, kernel_specs: List[KernelSpec]):
        self.gm, self.kernel_specs = gm, kernel_specs


def compile_with_plan(gm: GraphModule, example_inputs) -> Callable:
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
