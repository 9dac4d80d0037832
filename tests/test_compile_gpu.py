"""GPU tests of torch.compile on the spyre device: the cases of the reference's
tests/_inductor/test_inductor_ops.py and test_building_blocks.py, compiled vs torch CPU eager
(rtol 1e-2 / atol 1e-3), plus the fused benchmark graph."""
import pytest
import torch
import torch.nn.functional as F

import torch_spyre  # noqa: F401
from oracle import math_ref
from oracle.math_ref import assert_close
from torch_spyre._inductor import compiler

pytestmark = pytest.mark.gpu
DEV = "spyre"
SEED = 0xAFFE


@pytest.fixture(autouse=True)
def _fresh(cuda):
    torch._dynamo.reset()
    yield


def rnd(*shape, seed=SEED, positive=False):
    t = torch.randn(*shape, generator=torch.Generator().manual_seed(seed))
    if positive:
        t = t.abs() + 0.1
    return t.half()


def check(fn, *cpu_inputs, atol=1e-3):
    want = fn(*cpu_inputs)
    got = torch.compile(fn)(*[t.to(DEV) for t in cpu_inputs])
    if isinstance(want, (tuple, list)):
        for g, w in zip(got, want):
            assert_close(g.cpu(), w, atol=atol)
    else:
        assert_close(got.cpu().reshape(want.shape), want, atol=atol)
    return compiler.last_compiled[-1]


@pytest.mark.parametrize("shape", [(64,), (256,), (67, 256)])
@pytest.mark.parametrize("op", ["abs", "exp", "reciprocal", "relu", "tanh", "sqrt", "rsqrt", "log"])
def test_unary(op, shape):
    check(getattr(torch, op), rnd(*shape, positive=op in ("sqrt", "rsqrt", "log", "reciprocal")))


@pytest.mark.parametrize("op", [torch.add, torch.mul, torch.sub, torch.div])
def test_binary(op):
    check(op, rnd(67, 256, positive=True), rnd(67, 256, seed=1, positive=True))


def test_broadcast_alias_where_reductions():
    check(lambda a, b: a + b, rnd(256), rnd(67, 256, seed=1))
    check(lambda x: x + x + x, rnd(67, 256))
    check(lambda x: x * x * x, rnd(67, 256))
    check(lambda x, y: torch.where(x >= y, x, y), rnd(67, 256), rnd(67, 256, seed=1))
    check(lambda x: torch.sum(x, 0), rnd(67, 256), atol=2e-2)
    check(lambda x: torch.amax(x, 0), rnd(67, 256))
    check(lambda x: x - torch.amax(x, 1, keepdim=True), rnd(128, 256))
    check(lambda x: x - torch.amax(x, 0, keepdim=True), rnd(128, 256))


def test_mm_and_linear_graph():
    check(lambda a, b: a @ b, rnd(67, 256), (rnd(256, 128, seed=1) * 0.1).half())
    w, bias = (rnd(192, 256, seed=2) * 0.1).half(), rnd(192, seed=3)
    check(lambda x, w, b: torch.relu(F.linear(x, w, b)) * 2.0, rnd(67, 256), w, bias)


@pytest.mark.parametrize("dim", [0, 1, -1])
def test_softmax(dim):
    check(lambda x: torch.softmax(x, dim), rnd(512, 1024))


def test_softplus_and_attention_blocks():
    def softplus(x):
        z = x * 1.0
        return torch.where(z > 20.0, x, torch.log(1.0 + torch.exp(z)) / 1.0)

    plan = check(softplus, rnd(64, 128))
    assert len(plan.kernel_specs) == 1          # the whole block is one kernel

    def attention(q, k, v):
        s = (q @ k.t()) * (128 ** -0.5)
        return torch.softmax(s, -1) @ v

    check(attention, rnd(256, 128), rnd(256, 128, seed=1), rnd(256, 128, seed=2))


def test_layer_norm_graph():
    w, b = rnd(256, seed=1), rnd(256, seed=2)
    check(lambda x, w, b: F.layer_norm(x, (256,), w, b) + 1.0, rnd(67, 256), w, b)


def test_config2_compiles_to_one_fused_kernel():
    x, a, b = math_ref.fused_inputs(256, 2048)
    plan = check(lambda x, a, b: torch.exp(x * a + b).sum(-1), x, a, b)
    assert len(plan.kernel_specs) == 1 and plan.fused_nodes == 4
    spec = plan.kernel_specs[0]
    assert spec.is_reduction and spec.dimensions == [256, 2048]
    assert [i[0] for i in spec.op_info["insns"]] == ["LOAD", "MUL", "ADD", "EXP"]
