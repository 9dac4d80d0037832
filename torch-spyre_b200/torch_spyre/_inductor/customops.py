"""``torch.ops.spyre.*`` custom ops with the reference's schemas
(torch_spyre/_inductor/customops.py:22-154).

compact / swap / slice move a 1-D tensor between the dense form and the "one value per
stick" form; here both forms are ordinary tensors (shape [n] and [n, 1] have exactly those
two stick images), so they are reshapes.  layer_norm runs the fused kernel; exx2 /
layernormscale / layernormnorm are the three stages the reference decomposes it into
(torch_spyre/_inductor/decompositions.py:26-36), kept so that graphs naming them still run."""
from typing import Optional, Sequence

import torch


@torch.library.custom_op("spyre::compact", mutates_args=())
def compact(input: torch.Tensor) -> torch.Tensor:
    return input.reshape(-1).clone()


@compact.register_fake
def _(input):
    return input.new_empty(input.numel())


@torch.library.custom_op("spyre::swap", mutates_args=())
def swap(input: torch.Tensor) -> torch.Tensor:
    return input.reshape(-1, 1).clone()


@swap.register_fake
def _(input):
    return input.new_empty(input.numel(), 1)


@torch.library.custom_op("spyre::slice", mutates_args=())
def slice(input: torch.Tensor) -> torch.Tensor:
    return input.reshape(-1).clone()


@slice.register_fake
def _(input):
    return input.new_empty(input.numel())


@torch.library.custom_op("spyre::layer_norm", mutates_args=())
def layer_norm(x: torch.Tensor, normalized_shape: Sequence[int], weight: Optional[torch.Tensor] = None,
               bias: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    if len(normalized_shape) != 1:
        from . import Unsupported

        raise Unsupported(f"spyre.layernorm: unsupported reduction shape {normalized_shape}")
    return torch.native_layer_norm(x, list(normalized_shape), weight, bias, eps)[0]


@layer_norm.register_fake
def _(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    return x.new_empty(x.size())


@torch.library.custom_op("spyre::exx2", mutates_args=())
def exx2(x: torch.Tensor, exx2Scale: float, useZeroMean: bool) -> torch.Tensor:
    """Per row: [mean, mean of squares] scaled by exx2Scale * n, as a [rows..., 2] tensor."""
    n = x.shape[-1]
    mean = x.mean(-1, keepdim=True) * (exx2Scale * n)
    sq = (x * x).mean(-1, keepdim=True) * (exx2Scale * n)
    if useZeroMean:
        mean = mean * 0.0
    return torch.cat([mean, sq], dim=-1)


@exx2.register_fake
def _(x, exx2Scale, useZeroMean):
    return x.new_empty(list(x.shape[:-1]) + [2])


@torch.library.custom_op("spyre::layernormscale", mutates_args=())
def layernormscale(x: torch.Tensor, eps: float) -> torch.Tensor:
    """From [mean, E[x^2]] to [mean, rsqrt(var + eps)]."""
    mean, sq = x[..., 0:1], x[..., 1:2]
    return torch.cat([mean, torch.rsqrt(sq - mean * mean + eps)], dim=-1)


@layernormscale.register_fake
def _(x, eps):
    return x.new_empty(x.size())


@torch.library.custom_op("spyre::layernormnorm", mutates_args=())
def layernormnorm(x: torch.Tensor, mean: torch.Tensor, norm_mean: torch.Tensor,
                  weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = (x - norm_mean[..., 0:1]) * norm_mean[..., 1:2]
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


@layernormnorm.register_fake
def _(x, mean, norm_mean, weight=None, bias=None):
    return x.new_empty(x.size())
