"""CPU: the plain-torch decoder-layer oracle against transformers' LlamaDecoderLayer (the class
the reference's own test names), and the custom ops' host definitions against the oracle."""
import math

import pytest
import torch

import torch_spyre  # noqa: F401
from oracle import llama_ref as L


def test_oracle_matches_transformers_decoder_layer():
    tf = pytest.importorskip("transformers")
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding

    cfg = L.LayerConfig(d_model=512, heads=4, ffn=1024)
    w = L.make_weights(cfg)
    b, s = 2, 64
    x = torch.randn(b, s, cfg.d_model, generator=torch.Generator().manual_seed(1)).half()
    hc = tf.LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=4,
                        intermediate_size=1024, rms_norm_eps=cfg.eps, num_hidden_layers=1,
                        max_position_embeddings=128, attn_implementation="eager")
    layer = LlamaDecoderLayer(hc, 0).half()
    missing = layer.load_state_dict({
        "self_attn.q_proj.weight": w["q"], "self_attn.k_proj.weight": w["k"],
        "self_attn.v_proj.weight": w["v"], "self_attn.o_proj.weight": w["o"],
        "mlp.gate_proj.weight": w["gate"], "mlp.up_proj.weight": w["up"],
        "mlp.down_proj.weight": w["down"], "input_layernorm.weight": w["norm1"],
        "post_attention_layernorm.weight": w["norm2"]}, strict=False)
    assert not missing.missing_keys
    pos = torch.arange(s)[None].expand(b, -1)
    pe = LlamaRotaryEmbedding(hc)(x, pos)
    mask = torch.full((s, s), float("-inf")).triu(1)[None, None].half()
    with torch.no_grad():
        out = layer(x, attention_mask=mask, position_ids=pos, position_embeddings=pe)
    out = out[0] if isinstance(out, tuple) else out
    torch.testing.assert_close(L.layer_forward(x, w, cfg), out, rtol=1e-2, atol=1e-3)


def test_custom_ops_host_definitions_match_oracle():
    cfg = L.LayerConfig(d_model=256, heads=2, ffn=512)
    g = torch.Generator().manual_seed(2)
    b, s = 2, 48
    x = torch.randn(b, s, cfg.d_model, generator=g).half()
    wt = (1 + torch.randn(cfg.d_model, generator=g) * 0.02).half()
    torch.testing.assert_close(torch.ops.spyre.rms_norm(x, wt, 1e-5), L.rms_norm(x, wt, 1e-5))
    cos, sin = L.rope_tables(s, cfg.head_dim)
    xh = x.view(b, s, cfg.heads, cfg.head_dim).transpose(1, 2)
    want = (xh * cos[None, None] + L.rotate_half(xh) * sin[None, None]).transpose(1, 2).reshape(b, s, -1)
    torch.testing.assert_close(torch.ops.spyre.rotary(x, cos, sin, cfg.heads), want)
    q, k, v = (torch.randn(b, s, cfg.d_model, generator=g).half() for _ in range(3))
    scale = 1 / math.sqrt(cfg.head_dim)
    qh, kh, vh = (t.view(b, s, cfg.heads, cfg.head_dim).transpose(1, 2) for t in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(qh.float(), kh.float(), vh.float(),
                                                           is_causal=True, scale=scale)
    got = torch.ops.spyre.causal_attention(q, k, v, cfg.heads, scale)
    torch.testing.assert_close(got.float(), ref.transpose(1, 2).reshape(b, s, -1), rtol=1e-2, atol=2e-3)
