"""GPU parity of the decoder-layer building blocks and of the whole layer (eager and through
torch.compile) against the CPU oracle, at sizes the oracle finishes in seconds."""
import math

import pytest
import torch

import torch_spyre  # noqa: F401
from examples.llama_layer import LlamaStyleLayer
from oracle import llama_ref as L
from oracle.math_ref import assert_close
from torch_spyre import _abi

pytestmark = pytest.mark.gpu
DEV = "spyre"


@pytest.fixture(autouse=True)
def _need_gpu(cuda):
    torch._dynamo.reset()
    yield


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).half()


@pytest.mark.parametrize("b,s,heads", [(1, 64, 1), (2, 256, 4), (1, 200, 2), (3, 130, 2)])
def test_rotary(b, s, heads):
    x = rnd(b, s, heads * 128)
    cos, sin = L.rope_tables(s, 128)
    got = torch.ops.spyre.rotary(x.to(DEV), cos.to(DEV), sin.to(DEV), heads).cpu()
    assert_close(got, torch.ops.spyre.rotary(x, cos, sin, heads))


@pytest.mark.parametrize("b,s,heads", [(1, 64, 1), (2, 256, 4), (1, 200, 2), (2, 320, 3),
                                       (1, 128, 1), (1, 384, 2), (3, 1024, 5), (1, 2048, 2),
                                       # odd tile counts with enough (batch, head) slices for several rounds of
                                       # the one-tile kernel's work order, a left-over slice on the spare CTA,
                                       # and a long odd sequence
                                       (4, 640, 20), (2, 896, 40), (1, 384, 50), (1, 2176, 3)])
def test_causal_attention(b, s, heads):
    q, k, v = rnd(b, s, heads * 128, seed=1), rnd(b, s, heads * 128, seed=2), rnd(b, s, heads * 128, seed=3)
    scale = 1 / math.sqrt(128)
    got = torch.ops.spyre.causal_attention(q.to(DEV), k.to(DEV), v.to(DEV), heads, scale).cpu()
    torch.cuda.synchronize()
    assert _abi.lib().ts_gemm_error_state() == 0
    assert _abi.lib().ts_attention_error_state() == 0
    qh, kh, vh = (t.view(b, s, heads, 128).transpose(1, 2).float() for t in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale)
    assert_close(got, ref.transpose(1, 2).reshape(b, s, -1).half(), atol=2e-3)


@pytest.mark.parametrize("s", [512, 640])     # an even and an odd number of tiles: the two kernels
def test_fused_attention_peaked_scores(s):
    """Scores large enough that the running maximum changes from key tile to key tile and the
    softmax is nearly one-hot.  The one-kernel path keeps scores in fp32, so it must meet the
    oracle's tolerance; the three-launch path (fp16 scores in memory) is only required to be
    no closer to the fp32 reference than that rounding allows."""
    from torch_spyre import stick_ops as K

    b, heads = 2, 3
    q, k, v = rnd(b, s, heads * 128, seed=4, scale=3.0), rnd(b, s, heads * 128, seed=5, scale=3.0), \
        rnd(b, s, heads * 128, seed=6)
    scale = 1 / math.sqrt(128)
    args = [t.to(DEV) for t in (q, k, v)]
    fused = torch.ops.spyre.causal_attention(*args, heads, scale).cpu()
    K.fused_attention = False
    try:
        unfused = torch.ops.spyre.causal_attention(*args, heads, scale).cpu()
    finally:
        K.fused_attention = True
    assert _abi.lib().ts_attention_error_state() == 0
    qh, kh, vh = (t.view(b, s, heads, 128).transpose(1, 2).float() for t in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale)
    ref = ref.transpose(1, 2).reshape(b, s, -1)
    assert_close(fused, ref.half(), atol=2e-3)
    assert (fused.float() - ref).abs().max() <= (unfused.float() - ref).abs().max() + 1e-3


def test_attention_rejects_unsupported_shapes():
    lib = _abi.lib()
    buf = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    p = buf.data_ptr()
    assert lib.ts_attention_causal_f16(p, p, p, p, 1, 128, 1, 64, 0.1, None) == _abi.TS_ERR_UNSUPPORTED
    assert lib.ts_attention_causal_f16(p, None, p, p, 1, 128, 1, 128, 0.1, None) == _abi.TS_ERR_INVALID
    assert lib.ts_attention_causal_f16(p + 2, p, p, p, 1, 128, 1, 128, 0.1, None) == _abi.TS_ERR_ALIGNMENT
    assert lib.ts_attention_causal_f16(p, p, p, p, 0, 128, 1, 128, 0.1, None) == 0


def test_rms_norm_op():
    x, w = rnd(4, 100, 512) * 2, (1 + rnd(512, seed=1) * 0.02)
    assert_close(torch.ops.spyre.rms_norm(x.to(DEV), w.to(DEV), 1e-5).cpu(), L.rms_norm(x, w, 1e-5))


@pytest.mark.parametrize("compiled", [False, True])
def test_decoder_layer(compiled):
    cfg = L.LayerConfig(d_model=512, heads=4, ffn=1024)
    w = L.make_weights(cfg)
    b, s = 2, 256
    x = rnd(b, s, cfg.d_model, seed=5)
    cos, sin = L.rope_tables(s, cfg.head_dim)
    layer = LlamaStyleLayer({k: v.to(DEV) for k, v in w.items()}, cfg.heads, cfg.eps, cos.to(DEV), sin.to(DEV))
    fn = torch.compile(layer) if compiled else layer
    got = fn(x.to(DEV)).cpu()
    want = L.layer_forward(x, w, cfg)
    # a whole layer accumulates a few fp16 roundings per stage: same rtol, atol for |y| ~ 1
    torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=5e-3)
    if compiled:
        from torch_spyre._inductor import compiler
        plan = compiler.last_compiled[-1]
        names = [str(n.target) for n in plan.gm.graph.nodes if n.op == "call_function"]
        # the gate / up pair with its silu and multiply is one GEMM; both residuals ride in GEMMs
        assert sum("spyre.swiglu_linear" in t for t in names) == 1
        assert sum("aten.addmm" in t for t in names) == 2
        assert not any("aten.silu" in t for t in names)
