"""CPU tests of the compile-time half of the spyre torch.compile backend: grouping of
pointwise nodes, linearisation into accumulator-machine programs, and that the programs mean
what the graph means (checked with a host emulator of the instruction set)."""
import pytest
import torch
import torch.nn.functional as F
from torch.fx.experimental.proxy_tensor import make_fx

import torch_spyre  # noqa: F401
from torch_spyre._inductor import compiler, fusion


def trace(fn, *inputs):
    gm = make_fx(fn, decomposition_table=compiler.spyre_decompositions(), tracing_mode="fake")(*inputs)
    return gm


def programs_of(gm):
    groups, owner = fusion.build_groups(gm.graph)
    progs = []
    for g in groups:
        progs.append((g, fusion.linearise(g, compiler._outside_users(owner, g))))
    return progs


def run_and_compare(fn, *inputs, expect_groups=1):
    gm = trace(fn, *inputs)
    progs = programs_of(gm)
    if expect_groups is not None:
        assert len(progs) == expect_groups
    placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
    values = dict(zip(placeholders, inputs))
    want = fn(*inputs)
    want = want if isinstance(want, (tuple, list)) else (want,)
    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    outs = out_node.args[0]
    outs = outs if isinstance(outs, (tuple, list)) else (outs,)
    for g, prog in progs:
        values.update(fusion.emulate(prog, values))
    for node, ref in zip(outs, want):
        torch.testing.assert_close(values[node].float(), ref.float(), rtol=1e-2, atol=2e-3)
    return progs


def x(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).half()


def test_config2_is_one_program():
    a, b = (torch.rand(256) * 2 - 1).half(), (torch.rand(256) * 2 - 1).half()
    progs = run_and_compare(lambda t, a, b: torch.exp(t * a + b).sum(-1), x(64, 256), a, b)
    (_, prog), = progs
    assert [i[0] for i in prog.insns] == ["LOAD", "MUL", "ADD", "EXP"]
    assert prog.reduce == "sum" and not prog.keepdim and len(prog.inputs) == 3 and not prog.outputs


def test_alias_operands_and_reuse():
    run_and_compare(lambda t: t * t * t, x(67, 256))
    run_and_compare(lambda t: t + t + t, x(67, 256))
    run_and_compare(lambda t: (t + 1) * (t + 1), x(8, 64))
    run_and_compare(lambda t, u: (t - u) / (t * t + 2.0), x(8, 64), x(8, 64, seed=1))
    run_and_compare(lambda t, u: (t - u) / (u * u + 2.0), x(8, 64), x(8, 64, seed=1))


def test_scalar_first_operands_and_where():
    run_and_compare(lambda t: 2.0 - t, x(8, 64))
    run_and_compare(lambda t: 1.0 / (1.0 + torch.exp(-t)), x(8, 64))
    run_and_compare(lambda t, u: torch.where(t >= u, t, u * 2), x(8, 64), x(8, 64, seed=1))


def test_softplus_block():
    def softplus(t):
        z = t * 1.0
        return torch.where(z > 20.0, t, torch.log(1.0 + torch.exp(z)) / 1.0)

    run_and_compare(softplus, x(64, 128))


def test_two_outputs_and_mean():
    progs = run_and_compare(lambda t, u: (torch.relu(t + u), torch.tanh(t + u).mean(-1, keepdim=True)),
                            x(16, 128), x(16, 128, seed=1), expect_groups=None)
    reducing = [p for _, p in progs if p.reduce]
    assert len(reducing) == 1
    prog = reducing[0]
    assert prog.reduce == "sum" and prog.keepdim and abs(prog.reduce_scale - 1 / 128) < 1e-9


def test_x_minus_rowmax_makes_two_kernels():
    gm = trace(lambda t: t - t.amax(-1, keepdim=True), x(128, 256))
    groups, owner = fusion.build_groups(gm.graph)
    assert len(groups) == 1 and len(groups[0].nodes) == 1   # the subtraction; amax stays eager


def test_non_pointwise_nodes_split_groups():
    def fn(t, w):
        h = torch.relu(t + 1.0)
        y = h @ w
        return torch.sigmoid(y) * 2.0

    gm = trace(fn, x(32, 64), x(64, 64, seed=1))
    groups, _ = fusion.build_groups(gm.graph)
    assert len(groups) == 2 and [len(g.nodes) for g in groups] == [2, 2]


def test_slot_pressure_is_reported():
    def fn(t):
        a, b, c, d, e = t + 1, t + 2, t + 3, t + 4, t + 5
        return ((a * b) * (c * d)) * e + a + b + c + d + e

    gm = trace(fn, x(8, 64))
    groups, owner = fusion.build_groups(gm.graph)
    with pytest.raises(fusion.CannotFuse):
        for g in groups:
            fusion.linearise(g, compiler._outside_users(owner, g))


class _EmulatingCompile:
    """Stand-in for SpyreAsyncCompile on a machine without the device: runs a fused program
    with the host emulator of the instruction set."""

    def sdsc(self, name, spec):
        info = spec.op_info

        class Runner:
            def run(self, *tensors):
                nodes = [object() for _ in tensors]
                outs = [object() for _ in range(info["n_outputs"])]
                red = object() if info["reduce"] else None
                prog = fusion.Program(info["insns"], nodes, outs, tuple(spec.dimensions), info["reduce"],
                                      info["reduce_scale"], info["keepdim"], red)
                got = fusion.emulate(prog, dict(zip(nodes, tensors)))
                return [got[o] for o in outs] + ([got[red]] if red is not None else [])

        return Runner()

    def wait(self, scope):
        pass


def run_compiled(monkeypatch, fn, *inputs):
    monkeypatch.setattr(compiler, "SpyreAsyncCompile", _EmulatingCompile)
    gm = trace(fn, *inputs)
    cg = compiler.CompiledGraph(gm)
    got = cg(list(inputs))
    want = fn(*inputs)
    got = got if isinstance(got, (tuple, list)) else (got,)
    want = want if isinstance(want, (tuple, list)) else (want,)
    for g, w in zip(got, want):
        torch.testing.assert_close(g.float(), w.float(), rtol=1e-2, atol=2e-3)
    return cg


def test_outside_reader_between_members_of_a_group(monkeypatch):
    """exp feeds a matmul and a later add: [exp, add] fuse, and the fused launch has to be
    scheduled before the matmul that reads exp's stored result."""
    def fn(t, w):
        p1 = torch.exp(t)
        q = p1 @ w
        p2 = p1 + 1.0
        return q, p2

    cg = run_compiled(monkeypatch, fn, x(32, 64) * 0.1, x(64, 64, seed=1) * 0.1)
    assert cg.fused_nodes == 2 and len(cg.kernel_specs) == 1


def test_outside_reader_between_group_and_its_reduction(monkeypatch):
    def fn(t, w):
        e = torch.exp(t * 0.5)
        q = e @ w
        return q, e.sum(-1)

    cg = run_compiled(monkeypatch, fn, x(32, 64) * 0.1, x(64, 64, seed=1) * 0.1)
    assert len(cg.kernel_specs) == 1 and cg.kernel_specs[0].is_reduction


def test_group_waits_for_a_late_input(monkeypatch):
    """The second member's other operand is produced by a matmul that comes after the first
    member: the fused launch has to wait for it."""
    def fn(t, w):
        a = torch.tanh(t)
        m = t @ w
        return (a + m) * 2.0

    run_compiled(monkeypatch, fn, x(32, 64) * 0.1, x(64, 64, seed=1) * 0.1)


def test_intermediates_are_released_after_their_last_reader(monkeypatch):
    def fn(t, w):
        h = torch.relu(t + 1.0)
        y = h @ w
        return torch.sigmoid(y) * 2.0

    cg = run_compiled(monkeypatch, fn, x(32, 64), x(64, 64, seed=1))
    freed = {i for f in cg.frees for i in f}
    out_nodes = set()
    torch.fx.node.map_arg(cg.output_node.args[0], lambda a: out_nodes.add(a) or a)
    assert all(cg.slot[n] not in freed for n in out_nodes)
    assert len(freed) >= 3      # inputs and both intermediates
