"""CPU oracle for the Llama-style decoder layer of the benchmark (d_model 4096, 32 heads of
128, SwiGLU FFN 11008, RMSNorm, rotary, causal attention), written in plain torch from that
description.  TEST INFRASTRUCTURE ONLY.

It is pinned against the decoder layer class the reference's own (skipped) test names,
transformers' LlamaDecoderLayer (tests/test_modules.py:28-33,179-211 of the reference), by
tests/test_llama_oracle_cpu.py: same weights, same input, same output within fp16 tolerance.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class LayerConfig:
    d_model: int = 4096
    heads: int = 32
    ffn: int = 11008
    eps: float = 1e-5
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads


def make_weights(cfg: LayerConfig, seed: int = 0, dtype=torch.float16):
    """Random init N(0, 0.02) for the projections, ones (+ N(0,0.02)) for the norm weights."""
    g = torch.Generator().manual_seed(seed)
    d, f = cfg.d_model, cfg.ffn

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(dtype)

    return {
        "q": w(d, d), "k": w(d, d), "v": w(d, d), "o": w(d, d),
        "gate": w(f, d), "up": w(f, d), "down": w(d, f),
        "norm1": (1.0 + torch.randn(d, generator=g) * 0.02).to(dtype),
        "norm2": (1.0 + torch.randn(d, generator=g) * 0.02).to(dtype),
    }


def rope_tables(seq: int, head_dim: int, theta: float = 10000.0, dtype=torch.float16):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.arange(seq, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rms_norm(x, weight, eps):
    xf = x.float()
    return weight * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def layer_forward(x: torch.Tensor, w: dict, cfg: LayerConfig) -> torch.Tensor:
    """Every op in x.dtype, rounding after each one (what eager does)."""
    b, s, d = x.shape
    hd, nh = cfg.head_dim, cfg.heads
    # the tables are fp16 values whatever the compute dtype: they are inputs of the layer
    cos, sin = (t.to(x.dtype) for t in rope_tables(s, hd, cfg.rope_theta, torch.float16))
    h = rms_norm(x, w["norm1"], cfg.eps)
    q = F.linear(h, w["q"]).view(b, s, nh, hd).transpose(1, 2)
    k = F.linear(h, w["k"]).view(b, s, nh, hd).transpose(1, 2)
    v = F.linear(h, w["v"]).view(b, s, nh, hd).transpose(1, 2)
    c, sn = cos[None, None], sin[None, None]
    q = q * c + rotate_half(q) * sn
    k = k * c + rotate_half(k) * sn
    scores = torch.matmul(q, k.transpose(2, 3)) * (1.0 / math.sqrt(hd))
    mask = torch.full((s, s), float("-inf"), dtype=torch.float32).triu(1)
    probs = torch.softmax(scores.float() + mask, dim=-1).to(x.dtype)
    attn = torch.matmul(probs, v).transpose(1, 2).reshape(b, s, d)
    x = x + F.linear(attn, w["o"])
    h = rms_norm(x, w["norm2"], cfg.eps)
    return x + F.linear(F.silu(F.linear(h, w["gate"])) * F.linear(h, w["up"]), w["down"])


def layer_forward_fp32(x: torch.Tensor, w: dict, cfg: LayerConfig) -> torch.Tensor:
    """The same layer on the same fp16 inputs, evaluated in fp32 throughout: the yardstick two
    fp16 evaluations are measured against when they round in different places."""
    return layer_forward(x.float(), {k: v.float() for k, v in w.items()}, cfg)


def make_model_weights(cfg: LayerConfig, vocab: int, n_layers: int, seed: int = 0) -> dict:
    """Seeded weights of a small model: embedding, `n_layers` layers, final norm, output projection."""
    g = torch.Generator().manual_seed(1000 + seed)
    return {"embed": (torch.randn(vocab, cfg.d_model, generator=g)).half(),
            "layers": [make_weights(cfg, seed=seed + 1 + i) for i in range(n_layers)],
            "final_norm": (torch.randn(cfg.d_model, generator=g) * 0.02 + 1.0).half(),
            "lm_head": (torch.randn(vocab, cfg.d_model, generator=g) * 0.02).half()}


def model_forward(ids: torch.Tensor, mw: dict, cfg: LayerConfig, dtype=torch.float16) -> torch.Tensor:
    """Token ids [batch, seq] -> logits [batch, seq, vocab]; every op in `dtype`, rounding after each."""
    conv = (lambda t: t.to(dtype))
    x = F.embedding(ids, conv(mw["embed"]))
    for w in mw["layers"]:
        x = layer_forward(x, {k: conv(v) for k, v in w.items()}, cfg)
    x = rms_norm(x, conv(mw["final_norm"]), cfg.eps)
    return F.linear(x, conv(mw["lm_head"]))


def attention_forward(q, k, v, heads: int, scale: float):
    """Causal attention on packed [batch, seq, heads*head_dim] tensors, every op in q.dtype."""
    b, s, width = q.shape
    hd = width // heads
    qh, kh, vh = (t.view(b, s, heads, hd).transpose(1, 2) for t in (q, k, v))
    scores = torch.matmul(qh, kh.transpose(2, 3)) * scale
    mask = torch.full((s, s), float("-inf"), dtype=torch.float32).triu(1)
    probs = torch.softmax(scores.float() + mask, dim=-1).to(q.dtype)
    return torch.matmul(probs, vh).transpose(1, 2).reshape(b, s, width)


def layer_flops(batch: int, seq: int, cfg: LayerConfig, causal: bool = True) -> float:
    d, f, hd, nh = cfg.d_model, cfg.ffn, cfg.head_dim, cfg.heads
    tokens = batch * seq
    proj = 2.0 * tokens * d * d * 4
    ffn = 2.0 * tokens * d * f * 3
    attn = 2.0 * 2.0 * batch * nh * seq * seq * hd * (0.5 if causal else 1.0)
    return proj + ffn + attn
