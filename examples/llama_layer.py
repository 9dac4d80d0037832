"""A Llama-style decoder layer written as user code for the spyre device.

The reference ships examples/softmax.py in the same spirit (examples/softmax.py:17-44); its own
Llama test is skipped (tests/test_modules.py:178-211).  The layer uses ordinary torch calls
(F.linear, F.silu, +, *) and the fused custom ops the backend provides for the pieces a
decoder layer is made of (torch.ops.spyre.rms_norm / rotary / causal_attention); compiled with
torch.compile, the pointwise glue (SwiGLU gate, residual adds) is fused by the spyre backend.
Tensors keep the packed [batch, seq, heads*head_dim] form throughout, which is the form the
attention kernels read heads out of, so no transpose is ever materialised.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

import torch_spyre  # noqa: F401  (registers the device, ops and custom ops)


class LlamaStyleLayer(torch.nn.Module):
    def __init__(self, weights: dict, heads: int, eps: float, cos: torch.Tensor, sin: torch.Tensor):
        super().__init__()
        for name, value in weights.items():
            self.register_buffer("w_" + name, value)
        self.register_buffer("cos", cos)
        self.register_buffer("sin", sin)
        self.heads, self.eps = heads, eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        heads = self.heads
        scale = 1.0 / math.sqrt(x.shape[-1] // heads)
        h = torch.ops.spyre.rms_norm(x, self.w_norm1, self.eps)
        q = torch.ops.spyre.rotary(F.linear(h, self.w_q), self.cos, self.sin, heads)
        k = torch.ops.spyre.rotary(F.linear(h, self.w_k), self.cos, self.sin, heads)
        v = F.linear(h, self.w_v)
        attn = torch.ops.spyre.causal_attention(q, k, v, heads, scale)
        x = x + F.linear(attn, self.w_o)
        h = torch.ops.spyre.rms_norm(x, self.w_norm2, self.eps)
        return x + F.linear(F.silu(F.linear(h, self.w_gate)) * F.linear(h, self.w_up), self.w_down)
