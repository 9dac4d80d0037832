"""GPU parity: pointwise chains, reductions, softmax and norms against torch CPU eager
(rtol 1e-2, atol 1e-3: tests/test_modules.py:39-40 of the reference), through the C ABI."""
import pytest
import torch
import torch.nn.functional as F

from oracle import math_ref
from oracle.math_ref import assert_close
from torch_spyre import stick_ops as K
from torch_spyre.stick_ops import Chain

pytestmark = pytest.mark.gpu
SEED = 0xAFFE  # tests/_inductor/test_inductor_ops.py:50 of the reference


def up(t: torch.Tensor, cuda) -> K.StickTensor:
    return K.to_sticks(t.to(cuda))


def down(st: K.StickTensor) -> torch.Tensor:
    return K.from_sticks(st).cpu()


def randn(*shape, seed=SEED):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).half()


UNARY = {
    "ABS": torch.abs, "NEG": torch.neg, "EXP": torch.exp, "RELU": torch.relu,
    "TANH": torch.tanh, "SIGMOID": torch.sigmoid, "SILU": F.silu, "GELU": F.gelu,
    "GELU_TANH": lambda x: F.gelu(x, approximate="tanh"), "SQUARE": lambda x: x * x,
    "SIN": torch.sin, "COS": torch.cos, "ERF": torch.erf, "FLOOR": torch.floor,
    "CEIL": torch.ceil, "SIGN": torch.sign, "EXPM1": torch.expm1, "SOFTPLUS": F.softplus,
    "MISH": F.mish,
}
UNARY_POS = {"LOG": torch.log, "SQRT": torch.sqrt, "RSQRT": torch.rsqrt,
             "RECIP": torch.reciprocal, "LOG1P": torch.log1p}


@pytest.mark.parametrize("shape", [(64,), (256,), (67, 256), (3, 5), (4, 7, 130)])
@pytest.mark.parametrize("op", sorted(UNARY) + sorted(UNARY_POS))
def test_unary(op, shape, cuda):
    x = randn(*shape)
    if op in UNARY_POS:
        x = x.abs() + 0.1
    fn = UNARY.get(op) or UNARY_POS[op]
    c = Chain()
    c.emit("LOAD", c.tensor(up(x, cuda))).emit(op).store(0)
    (y,), _ = K.run_chain(c, shape)
    assert_close(down(y), fn(x))


BINARY = {"ADD": torch.add, "SUB": torch.sub, "MUL": torch.mul, "DIV": torch.div,
          "MAX": torch.maximum, "MIN": torch.minimum,
          "RSUB": lambda a, b: b - a, "RDIV": lambda a, b: b / a}


@pytest.mark.parametrize("op", sorted(BINARY))
@pytest.mark.parametrize("shapes", [((67, 256), (67, 256)), ((67, 256), (256,)), ((67, 256), (67, 1)),
                                    ((4, 5, 130), (5, 1)), ((4, 5, 130), (4, 1, 130)),
                                    ((2, 3, 4, 70), (3, 1, 70)), ((3, 64), (1,))])
def test_binary_broadcast(op, shapes, cuda):
    a, b = randn(*shapes[0]), randn(*shapes[1], seed=SEED + 1)
    if op in ("DIV", "RDIV"):
        a, b = a.abs() + 0.5, b.abs() + 0.5
    c = Chain()
    c.emit("LOAD", c.tensor(up(a, cuda))).emit(op, c.tensor(up(b, cuda))).store(0)
    (y,), _ = K.run_chain(c, shapes[0])
    assert_close(down(y), BINARY[op](a, b))


def test_scalar_immediates_and_pow(cuda):
    x = randn(67, 256).abs() + 0.1
    c = Chain()
    c.emit("LOAD", c.tensor(up(x, cuda))).emit("ADD", c.imm(2.0)).emit("MUL", c.imm(0.5)) \
        .emit("POW", c.imm(3.0)).store(0)
    (y,), _ = K.run_chain(c, x.shape)
    assert_close(down(y), torch.pow((x + 2.0) * 0.5, 3.0))


def test_compare_and_where(cuda):
    x, y = randn(128, 256), randn(128, 256, seed=1)
    y[::3] = x[::3]
    sx, sy = up(x, cuda), up(y, cuda)
    for op, fn in [("EQ", torch.eq), ("NE", torch.ne), ("GE", torch.ge), ("GT", torch.gt),
                   ("LE", torch.le), ("LT", torch.lt)]:
        c = Chain()
        c.emit("LOAD", c.tensor(sx)).emit(op, c.tensor(sy)).store(0)
        (m,), _ = K.run_chain(c, x.shape)
        assert torch.equal(down(m).bool(), fn(x, y))
    # where(x >= y, x, y * 2)
    c = Chain()
    c.emit("LOAD", c.tensor(sy)).emit("MUL", c.imm(2.0)).save(0)
    c.emit("LOAD", c.tensor(sx)).emit("GE", c.tensor(sy)).emit("WHERE", c.tensor(sx), c.saved(0)).store(0)
    (w,), _ = K.run_chain(c, x.shape)
    assert_close(down(w), torch.where(x >= y, x, y * 2))


def test_alias_operands_and_two_outputs(cuda):
    x = randn(67, 256)
    sx = up(x, cuda)
    c = Chain()
    c.emit("LOAD", c.tensor(sx)).emit("MUL", c.tensor(sx)).store(0).emit("MUL", c.tensor(sx)).store(1)
    (y2, y3), _ = K.run_chain(c, x.shape, n_outputs=2)
    assert len(c.inputs) == 1
    assert_close(down(y2), x * x)
    assert_close(down(y3), x * x * x)


def test_softplus_building_block(cuda):
    # tests/_inductor/test_building_blocks.py:38-65 of the reference: where(x*b > t, x, log(1+exp(x*b))/b)
    x = randn(64, 128) * 8
    beta, thr = 1.0, 20.0
    # op by op in fp16, as eager does (exp overflows to inf above ~11.09, exactly as here)
    want = torch.where(x * beta > thr, x, torch.log(1 + torch.exp(x * beta)) / beta)
    c = Chain()
    sx = up(x, cuda)
    c.emit("LOAD", c.tensor(sx)).emit("MUL", c.imm(beta)).save(0)
    c.emit("EXP").emit("ADD", c.imm(1.0)).emit("LOG").emit("DIV", c.imm(beta)).save(1)
    c.emit("LOAD", c.saved(0)).emit("GT", c.imm(thr)).emit("WHERE", c.tensor(sx), c.saved(1)).store(0)
    (y,), _ = K.run_chain(c, x.shape)
    torch.testing.assert_close(down(y), want, rtol=1e-2, atol=1e-3, equal_nan=True)


@pytest.mark.parametrize("shape", [(3, 64), (67, 256), (128, 4096), (5, 70), (4, 6, 200), (1, 8192), (300,)])
@pytest.mark.parametrize("op", ["sum", "max", "min"])
@pytest.mark.parametrize("keepdim", [False, True])
def test_row_reductions(op, shape, keepdim, cuda):
    x = randn(*shape)
    c = Chain()
    c.emit("LOAD", c.tensor(up(x, cuda)))
    _, r = K.run_chain(c, shape, n_outputs=0, reduce=op, keepdim=keepdim)
    if op == "sum":
        want = x.sum(-1, keepdim=keepdim)
    else:
        want = getattr(x, op)(-1, keepdim=keepdim).values
    got = down(r).reshape(want.shape)
    assert_close(got, want, rtol=1e-2, atol=2e-2 if op == "sum" else 1e-3)
    # pad lanes of the reduced image must be zero
    img = r.image.cpu().view(-1, 64)
    if not keepdim and len(shape) >= 2:
        last = shape[-2]
        if last % 64:
            assert (img.view(-1, x[..., 0].numel() // last, 64)[-1, :, last % 64:] == 0).all()
    if keepdim:
        assert (img[:, 1:] == 0).all()


def test_mean_via_scale(cuda):
    x = randn(67, 256)
    c = Chain()
    c.emit("LOAD", c.tensor(up(x, cuda)))
    _, r = K.run_chain(c, x.shape, n_outputs=0, reduce="sum", reduce_scale=1.0 / 256)
    assert_close(down(r), x.mean(-1))


@pytest.mark.parametrize("rows,cols", [(64, 256), (128, 8192), (67, 200)])
def test_fused_config2_small(rows, cols, cuda):
    x, a, b = math_ref.fused_inputs(rows, cols)
    c = Chain()
    c.emit("LOAD", c.tensor(up(x, cuda))).emit("MUL", c.tensor(up(a, cuda))) \
        .emit("ADD", c.tensor(up(b, cuda))).emit("EXP")
    _, r = K.run_chain(c, x.shape, n_outputs=0, reduce="sum")
    want = math_ref.fused_ref(x, a, b)
    assert_close(down(r), want)


def test_x_minus_rowmax(cuda):
    # tests/_inductor/test_inductor_ops.py:163-168 of the reference (dim 1)
    x = randn(128, 256)
    sx = up(x, cuda)
    c = Chain()
    c.emit("LOAD", c.tensor(sx))
    _, m = K.run_chain(c, x.shape, n_outputs=0, reduce="max", keepdim=True)
    c2 = Chain()
    c2.emit("LOAD", c2.tensor(sx)).emit("SUB", c2.tensor(m)).store(0)
    (y,), _ = K.run_chain(c2, x.shape)
    assert_close(down(y), x - x.max(1, keepdim=True).values)


@pytest.mark.parametrize("shape", [(3, 64), (512, 1024), (1024, 256), (256, 4096), (5, 70), (7, 8192),
                                   (4, 9, 130), (64,)])
@pytest.mark.parametrize("log", [False, True])
def test_softmax_last_dim(shape, log, cuda):
    x = randn(*shape)
    y = K.softmax(up(x, cuda), -1, log)
    want = F.log_softmax(x, -1) if log else torch.softmax(x, -1)
    assert_close(down(y), want)
    if shape[-1] % 64:
        img = y.image.cpu().view(-1, y.rows, 64)
        assert (img[-1, :, shape[-1] % 64:] == 0).all()


def test_softmax_config1(cuda):
    x = math_ref.softmax_inputs()
    y = K.softmax(up(x, cuda), -1)
    assert_close(down(y), torch.softmax(x, -1))


@pytest.mark.parametrize("shape,dim", [((512, 1024), 0), ((67, 256), 0), ((4, 9, 130), 1), ((4, 9, 130), 0),
                                       ((2, 3, 5, 64), 2)])
def test_softmax_other_dims(shape, dim, cuda):
    x = randn(*shape)
    assert_close(down(K.softmax(up(x, cuda), dim)), torch.softmax(x, dim))
    assert_close(down(K.softmax(up(x, cuda), dim, True)), F.log_softmax(x, dim))


@pytest.mark.parametrize("shape,dim", [((67, 256), 0), ((512, 1024), 0), ((4, 9, 130), 1), ((4, 9, 130), 0),
                                       ((20000, 64), 0), ((2, 3, 5, 64), 2)])
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_reduce_other_dims(shape, dim, op, cuda):
    x = randn(*shape)
    if shape[0] == 20000:
        x = x * 0.1
    r = K.reduce_mid(up(x, cuda), dim, op)
    want = x.sum(dim) if op == "sum" else getattr(x, op)(dim).values
    assert_close(down(r), want, atol=2e-2 if op == "sum" else 1e-3)
    k = K.reduce_mid(up(x, cuda), dim, op, keepdim=True)
    assert_close(down(k), want.unsqueeze(dim), atol=2e-2 if op == "sum" else 1e-3)


@pytest.mark.parametrize("shape", [(3, 64), (67, 256), (16, 4096), (5, 70), (4, 9, 130), (2, 8192)])
def test_layer_norm(shape, cuda):
    x = randn(*shape) * 2 + 0.5
    w, b = randn(shape[-1], seed=1), randn(shape[-1], seed=2)
    sx = up(x, cuda)
    y = K.layernorm_rows(sx, up(w, cuda), up(b, cuda), 1e-5)
    assert_close(down(y), F.layer_norm(x, (shape[-1],), w, b, 1e-5))
    y = K.layernorm_rows(sx, None, None, 1e-5)
    assert_close(down(y), F.layer_norm(x, (shape[-1],), None, None, 1e-5))


@pytest.mark.parametrize("shape", [(3, 64), (16, 4096), (5, 70), (4, 9, 130)])
def test_rms_norm(shape, cuda):
    x = randn(*shape) * 2
    w = randn(shape[-1], seed=1) * 0.1 + 1
    eps = 1e-5
    xf = x.float()
    normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps))
    want_module = w * normed.half()          # RMSNorm module order: round, then fp16 multiply
    y = K.rmsnorm_rows(up(x, cuda), up(w, cuda), eps, True)
    assert_close(down(y), want_module)
    y = K.rmsnorm_rows(up(x, cuda), up(w, cuda), eps, False)
    assert_close(down(y), F.rms_norm(x, (shape[-1],), w, eps))


def test_back_to_back_launches_keep_stream_order(cuda):
    """The streaming kernels are launched so that a kernel may be placed on the SMs while the one
    before it on the stream is still finishing; it must nevertheless see everything that one
    wrote.  A ping-pong of dependent launches (pointwise -> pointwise -> row sum -> softmax of the
    pointwise result), each reading what the previous one wrote into reused buffers, is enqueued
    without any synchronisation and compared bit for bit with the same sequence run with a
    device synchronisation after every launch."""
    rows, cols = 4096, 4096
    x = randn(rows, cols)
    b = randn(cols, seed=SEED + 1)

    def sequence(sync):
        bufs = [K.empty((rows, cols), device=cuda), K.empty((rows, cols), device=cuda)]
        cur = up(x, cuda)
        sb = up(b, cuda)
        sums = []
        for i in range(6):
            c = Chain()
            c.emit("LOAD", c.tensor(cur)).emit("MUL", c.imm(0.5)).emit("ADD", c.tensor(sb)).store(0)
            (cur,), _ = K.run_chain(c, (rows, cols), outputs=[bufs[i & 1]])
            if sync:
                torch.cuda.synchronize()
            c2 = Chain()
            c2.emit("LOAD", c2.tensor(cur)).emit("ABS")
            _, r = K.run_chain(c2, (rows, cols), n_outputs=0, reduce="sum", reduce_scale=1.0 / cols)
            if sync:
                torch.cuda.synchronize()
            sums.append(r)
        y = K.softmax(cur, -1)
        torch.cuda.synchronize()
        return [down(s) for s in sums] + [down(y), down(cur)]

    want = sequence(True)
    for _ in range(5):
        got = sequence(False)
        for g, w in zip(got, want):
            assert torch.equal(g.view(torch.int16), w.view(torch.int16))
    # and the arithmetic itself, once
    ref = x
    for _ in range(6):
        ref = ref * 0.5 + b
    assert_close(want[-1], ref)
