"""The graph rewrites that map stock decoder-layer code onto the fused spyre ops, checked on CPU:
the rewritten graphs must contain the fused nodes and compute what the original graphs compute
(every spyre custom op has a plain-torch definition off the device)."""
import pytest
import torch

import torch_spyre  # noqa: F401  (registers the spyre custom ops)
from torch_spyre._inductor import patterns

transformers = pytest.importorskip("transformers")


def _layer_and_inputs(batch=2, seq=64, heads=2, hidden=256, inter=384):
    from transformers.models.llama.modeling_llama import (LlamaConfig, LlamaDecoderLayer,
                                                          LlamaRotaryEmbedding)
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads,
                      num_key_value_heads=heads, num_hidden_layers=1, max_position_embeddings=512,
                      rms_norm_eps=1e-5, attn_implementation="sdpa")
    layer = LlamaDecoderLayer(cfg, 0).eval()
    x = torch.randn(batch, seq, hidden)
    pos = torch.arange(seq)[None].expand(batch, -1)
    cos, sin = LlamaRotaryEmbedding(cfg)(x, pos)
    return layer, x, cos, sin, pos


def _targets(gm):
    return [str(n.target) for n in gm.graph.nodes if n.op == "call_function"]


def test_rewrites_on_decoder_layer_graphs():
    from torch._functorch.aot_autograd import aot_module_simplified

    layer, x, cos, sin, pos = _layer_and_inputs()
    seen = {}

    def fw_compiler(gm, example_inputs):
        seen["before"] = _targets(gm)
        seen["count"] = patterns.rewrite_aten_graph(gm)
        seen["after"] = _targets(gm)
        return gm.forward

    def backend(gm, example_inputs):
        seen["sdpa"] = patterns.rewrite_dynamo_graph(gm)
        return aot_module_simplified(gm, example_inputs, fw_compiler=fw_compiler)

    def f(x, cos, sin):
        out = layer(x, position_embeddings=(cos, sin), attention_mask=None, position_ids=pos)
        return out[0] if isinstance(out, tuple) else out

    # the fp32 layer keeps the RMS-norm casts out of the graph, so trace a half-precision copy
    layer.half()
    xh, ch, sh = x.half(), cos.half(), sin.half()
    with torch.no_grad():
        want = f(xh, ch, sh)
        got = torch.compile(f, backend=backend)(xh, ch, sh)
    assert seen["sdpa"] == 1
    assert seen["count"] == 7        # two RMS norms, rotary on q and on k, two residual matmuls, SwiGLU
    after = seen["after"]
    assert sum("spyre.rms_norm" in t for t in after) == 2
    assert sum("spyre.rotary" in t for t in after) == 2
    assert sum("spyre.sdpa_causal" in t for t in after) == 1
    assert sum("aten.addmm" in t for t in after) == 2     # o_proj and down_proj take their residuals
    assert sum("spyre.swiglu_linear" in t for t in after) == 1 and not any("aten.silu" in t for t in after)
    assert not any("aten.cat" in t or "aten.pow" in t or "aten.rsqrt" in t for t in after)
    torch.testing.assert_close(got, want, rtol=1e-2, atol=2e-3)


def test_rms_norm_pattern_needs_exclusive_intermediates():
    """If an intermediate of the idiom is used elsewhere the rewrite must leave the graph alone."""
    from torch.fx.experimental.proxy_tensor import make_fx

    def f(x, w):
        x32 = x.float()
        r = torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + 1e-5)
        return w * (x32 * r).half(), r

    gm = make_fx(f)(torch.randn(4, 64).half(), torch.ones(64).half())
    assert patterns.rewrite_aten_graph(gm) == 0


def test_gate_up_interleave_and_its_cache():
    from torch_spyre._inductor import customops as C

    wg, wu = torch.randn(128, 64).half(), torch.randn(128, 64).half()
    w = C.interleave_gate_up(wg, wu)
    assert w.shape == (256, 64)
    assert torch.equal(w[0:64], wg[0:64]) and torch.equal(w[64:128], wu[0:64])
    assert torch.equal(w[128:192], wg[64:128]) and torch.equal(w[192:256], wu[64:128])
    first = C._cached_gate_up(wg, wu)
    assert C._cached_gate_up(wg, wu) is first
    wg.add_(1)                                   # written to: the cached copy is stale
    assert C._cached_gate_up(wg, wu) is not first
    other = torch.randn(128, 64).half()          # a different tensor, wherever it lives
    assert torch.equal(C._cached_gate_up(other, wu)[0:64], other[0:64])
    x = torch.randn(5, 64).half()
    want = torch.nn.functional.silu(x @ wg.t()) * (x @ wu.t())
    torch.testing.assert_close(torch.ops.spyre.swiglu_linear(x, wg, wu), want)


def _sdpa_rewrites(q, k, v):
    seen = {}

    def backend(gm, example_inputs):
        seen["count"] = patterns.rewrite_dynamo_graph(gm)
        return gm.forward

    f = lambda q, k, v: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)  # noqa: E731
    torch._dynamo.reset()
    torch.compile(f, backend=backend)(q, k, v)
    return seen["count"]


def test_sdpa_rewrite_only_for_what_the_fused_kernel_takes():
    """head_dim 128, fp16, q / k / v of one shape: anything else keeps the stock SDPA."""
    h = lambda *s: torch.randn(*s).half()  # noqa: E731
    assert _sdpa_rewrites(h(1, 2, 16, 128), h(1, 2, 16, 128), h(1, 2, 16, 128)) == 1
    assert _sdpa_rewrites(h(1, 2, 16, 64), h(1, 2, 16, 64), h(1, 2, 16, 64)) == 0        # head_dim 64
    assert _sdpa_rewrites(torch.randn(1, 2, 16, 128), torch.randn(1, 2, 16, 128),
                          torch.randn(1, 2, 16, 128)) == 0                                # fp32
    assert _sdpa_rewrites(h(1, 2, 16, 128), h(1, 2, 24, 128), h(1, 2, 24, 128)) == 0     # longer keys


def test_attention_wrapper_refuses_before_any_launch():
    """The host wrapper validates shapes and head size itself; these calls must raise without
    reaching the kernel library (the stand-in images are CPU tensors and are never read)."""
    from torch_spyre import _abi, stick_ops as K

    def st(*shape, dtype=torch.float16):
        return K.StickTensor(torch.empty(0, dtype=dtype), tuple(shape), dtype)

    with pytest.raises(_abi.SpyreKernelError, match="head_dim"):
        K.causal_attention(st(1, 128, 128), st(1, 128, 128), st(1, 128, 128), 1, 128, 2, 0.1)   # head_dim 64
    with pytest.raises(_abi.SpyreKernelError, match="one shape"):
        K.causal_attention(st(1, 128, 256), st(1, 256, 256), st(1, 256, 256), 1, 128, 2, 0.1)
    with pytest.raises(_abi.SpyreKernelError, match="out shape"):
        K.causal_attention(st(1, 128, 256), st(1, 128, 256), st(1, 128, 256), 1, 128, 2, 0.1,
                           out=st(1, 128, 128))
    with pytest.raises(_abi.SpyreKernelError, match="float16"):
        K.causal_attention(st(1, 128, 256, dtype=torch.bfloat16), st(1, 128, 256), st(1, 128, 256),
                           1, 128, 2, 0.1)
    with pytest.raises(_abi.SpyreKernelError, match="does not match"):
        K.causal_attention(st(1, 128, 256), st(1, 128, 256), st(1, 128, 256), 2, 128, 2, 0.1)
    K.check_attention_args((2, 128, 256), (2, 128, 256), (2, 128, 256), 2, (torch.float16,) * 3)


def test_device_only_custom_ops_refuse_host_tensors():
    """swap / slice / exx2 / layernormscale / layernormnorm are registered for the spyre device
    only, as in the reference (torch_spyre/_inductor/customops.py:38,56,102,116,133)."""
    x = torch.arange(8.0).half()
    for call in (lambda: torch.ops.spyre.swap(x), lambda: torch.ops.spyre.slice(x.reshape(-1, 1)),
                 lambda: torch.ops.spyre.exx2(x.reshape(2, 4), 0.25, False),
                 lambda: torch.ops.spyre.layernormscale(x.reshape(4, 2), 1e-5)):
        with pytest.raises(NotImplementedError):
            call()
    assert torch.equal(torch.ops.spyre.compact(x.reshape(-1, 1)), x)       # compact has no device restriction


def test_fp32_softmax_idiom_becomes_the_fp16_softmax():
    """softmax(x, dim, dtype=float32).to(float16) on an fp16 tensor (how attention code keeps the
    reduction in fp32) is one fp16 softmax for the device, whose kernel computes in fp32 and rounds
    once; an fp32 softmax with any other user is left alone."""
    from torch.fx.experimental.proxy_tensor import make_fx

    from torch_spyre._inductor import patterns

    def wanted(x):
        return torch.softmax(x, -1, dtype=torch.float32).to(torch.float16) * 2

    gm = make_fx(wanted)(torch.randn(4, 8).half())
    assert patterns.rewrite_aten_graph(gm) == 1
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert torch.ops.aten._to_copy.default not in targets
    sm = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is torch.ops.aten._softmax.default]
    assert len(sm) == 1 and sm[0].meta["val"].dtype == torch.float16
    x = torch.randn(64, 200).half()
    torch.testing.assert_close(gm(x), wanted(x), rtol=1e-3, atol=1e-5)

    def shared(x):
        s = torch.softmax(x, -1, dtype=torch.float32)
        return s.to(torch.float16), s.sum()

    gm2 = make_fx(shared)(torch.randn(4, 8).half())
    assert patterns.rewrite_aten_graph(gm2) == 0
