"""The decoder layer the reference's own test builds (transformers' LlamaDecoderLayer,
tests/test_modules.py:178-211 of the reference, skipped there) moved to the spyre device and
run through torch.compile, unmodified: the graph rewrites route its RMS norms, rotary embedding
and causal attention onto the fused kernels.  Oracle: the same module on CPU."""
import pytest
import torch

import torch_spyre  # noqa: F401
from oracle.math_ref import assert_close
from torch_spyre import _abi
from torch_spyre._inductor import compiler

transformers = pytest.importorskip("transformers")
pytestmark = pytest.mark.gpu
DEV = "spyre"


@pytest.fixture(autouse=True)
def _need_gpu(cuda):
    torch._dynamo.reset()
    yield


def _build(batch, seq, heads, inter):
    from transformers.models.llama.modeling_llama import (LlamaConfig, LlamaDecoderLayer,
                                                          LlamaRotaryEmbedding)
    torch.manual_seed(0)
    hidden = heads * 128
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads,
                      num_key_value_heads=heads, num_hidden_layers=1, max_position_embeddings=1024,
                      rms_norm_eps=1e-5, attn_implementation="sdpa")
    layer = LlamaDecoderLayer(cfg, 0).half().eval()
    x = torch.randn(batch, seq, hidden).half()
    pos = torch.arange(seq)[None].expand(batch, -1)
    cos, sin = LlamaRotaryEmbedding(cfg)(x, pos)
    return layer, x, cos.half(), sin.half(), pos


@pytest.mark.parametrize("batch,seq,heads,inter", [(2, 256, 2, 384), (1, 200, 3, 512)])
def test_hf_decoder_layer_compiled_on_spyre(batch, seq, heads, inter):
    layer, x, cos, sin, pos = _build(batch, seq, heads, inter)

    def run(mod, x, cos, sin):
        out = mod(x, position_embeddings=(cos, sin), attention_mask=None, position_ids=pos)
        return out[0] if isinstance(out, tuple) else out

    with torch.no_grad():
        want = run(layer, x, cos, sin)
        dev_layer = layer.to(DEV)
        fn = torch.compile(lambda a, c, s: run(dev_layer, a, c, s))
        got = fn(x.to(DEV), cos.to(DEV), sin.to(DEV)).cpu()
    torch.cuda.synchronize()
    assert _abi.lib().ts_gemm_error_state() == 0 and _abi.lib().ts_attention_error_state() == 0
    graph = compiler.last_compiled[-1]
    names = [str(n.target) for n in graph.gm.graph.nodes if n.op == "call_function"]
    assert sum("spyre.rms_norm" in t for t in names) == 2
    assert sum("spyre.rotary" in t for t in names) == 2
    assert sum("spyre.sdpa_causal" in t for t in names) == 1
    assert_close(got, want, atol=4e-3)
