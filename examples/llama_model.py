"""A small Llama-style model as user code for the spyre device: token embedding, a stack of
decoder layers (examples/llama_layer.py), a final RMS norm and the output projection.

The reference's module tests climb the same ladder, nn.Linear up to a decoder layer
(tests/test_modules.py:133-211); this is the next rung: a whole forward pass, from token ids on
the device to logits, through torch.compile or eagerly.
"""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.nn.functional as F

import torch_spyre  # noqa: F401  (registers the device, ops and custom ops)

from .llama_layer import LlamaStyleLayer


class LlamaStyleModel(torch.nn.Module):
    def __init__(self, embed: torch.Tensor, layers: List[Dict[str, torch.Tensor]], final_norm: torch.Tensor,
                 lm_head: torch.Tensor, heads: int, eps: float, cos: torch.Tensor, sin: torch.Tensor):
        super().__init__()
        self.register_buffer("embed", embed)            # [vocab, d_model]
        self.register_buffer("final_norm", final_norm)  # [d_model]
        self.register_buffer("lm_head", lm_head)        # [vocab, d_model]
        self.layers = torch.nn.ModuleList(LlamaStyleLayer(w, heads, eps, cos, sin) for w in layers)
        self.eps = eps

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        x = F.embedding(ids, self.embed)
        for layer in self.layers:
            x = layer(x)
        x = torch.ops.spyre.rms_norm(x, self.final_norm, self.eps)
        return F.linear(x, self.lm_head)
