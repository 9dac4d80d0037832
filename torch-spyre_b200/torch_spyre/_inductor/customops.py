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


@torch.library.custom_op("spyre::swap", mutates_args=(), device_types="spyre")
def swap(input: torch.Tensor) -> torch.Tensor:
    return input.reshape(-1, 1).clone()


@swap.register_fake
def _(input):
    return input.new_empty(input.numel(), 1)


@torch.library.custom_op("spyre::slice", mutates_args=(), device_types="spyre")
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


@torch.library.custom_op("spyre::exx2", mutates_args=(), device_types="spyre")
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


@torch.library.custom_op("spyre::layernormscale", mutates_args=(), device_types="spyre")
def layernormscale(x: torch.Tensor, eps: float) -> torch.Tensor:
    """From [mean, E[x^2]] to [mean, rsqrt(var + eps)]."""
    mean, sq = x[..., 0:1], x[..., 1:2]
    return torch.cat([mean, torch.rsqrt(sq - mean * mean + eps)], dim=-1)


@layernormscale.register_fake
def _(x, eps):
    return x.new_empty(x.size())


@torch.library.custom_op("spyre::layernormnorm", mutates_args=(), device_types="spyre")
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


# ---- fused building blocks of a decoder layer -------------------------------------------
# On spyre tensors these run the fused kernels; on any other device they are defined by the
# plain torch formula, so a graph naming them means the same thing everywhere.

def _on_spyre(t: torch.Tensor) -> bool:
    return t.device.type == "spyre"


@torch.library.custom_op("spyre::rms_norm", mutates_args=())
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if _on_spyre(x):
        from .. import ops

        return ops.rms_norm(x, weight, eps, round_before_weight=True)
    xf = x.float()
    normed = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * normed.to(x.dtype)


@rms_norm.register_fake
def _(x, weight, eps):
    return x.new_empty(x.size())


@torch.library.custom_op("spyre::rotary", mutates_args=())
def rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, heads: int) -> torch.Tensor:
    """x: [batch, seq, heads*head_dim]; cos, sin: [seq, head_dim]."""
    b, s, width = x.shape
    hd = width // heads
    if _on_spyre(x):
        from .. import ops, stick_ops as K

        out = torch.empty_like(x)
        with torch.cuda.device(x.device.index or 0):
            K.rotary(ops._st(x), ops._st(cos), ops._st(sin), b, s, heads, hd, out=ops._st(out))
        return out
    xh = x.view(b, s, heads, hd)
    rot = torch.cat((-xh[..., hd // 2:], xh[..., : hd // 2]), dim=-1)
    c, sn = cos.view(1, s, 1, hd), sin.view(1, s, 1, hd)
    return (xh * c + rot * sn).reshape(b, s, width)


@rotary.register_fake
def _(x, cos, sin, heads):
    return x.new_empty(x.size())


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[2N, K] weight whose rows alternate between w_gate and w_up in blocks of 64: the operand of
    the fused SwiGLU GEMM, whose 256-column tiles then hold matching gate / up stick pairs."""
    n, k = w_gate.shape
    return torch.stack((w_gate.reshape(n // 64, 64, k), w_up.reshape(n // 64, 64, k)), dim=1).reshape(2 * n, k)


_gate_up_cache: dict = {}


def invalidate_gate_up_cache() -> None:
    """Forget every interleaved gate / up weight (after weights were changed through ``.data``)."""
    _gate_up_cache.clear()


def _cached_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """The interleaved weight for this pair of weight tensors, rebuilt whenever either tensor is a
    different object, lives elsewhere or has been written to (an address alone could be a new
    tensor in recycled memory).  Entries die with their weights (weak references) and at most 16
    are kept.  A write through a detached alias (``w.data.copy_(...)``) changes neither the address
    nor the parameter's version counter and is therefore not seen: call
    ``invalidate_gate_up_cache()`` after such a write."""
    import weakref

    key = (id(w_gate), id(w_up))
    stamp = (w_gate.data_ptr(), w_up.data_ptr(), w_gate._version, w_up._version, tuple(w_gate.shape))
    hit = _gate_up_cache.get(key)
    if hit is not None and hit[0]() is w_gate and hit[1]() is w_up and hit[2] == stamp:
        return hit[3]
    if len(_gate_up_cache) >= 16:
        _gate_up_cache.clear()
    w = interleave_gate_up(w_gate, w_up)
    _gate_up_cache[key] = (weakref.ref(w_gate), weakref.ref(w_up), stamp, w)
    return w


@torch.library.custom_op("spyre::swiglu_linear", mutates_args=())
def swiglu_linear(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """silu(x @ w_gate^T) * (x @ w_up^T); x: [..., K], weights [N, K]."""
    if _on_spyre(x) and w_gate.shape[0] % 64 == 0:
        from .. import ops, stick_ops as K

        w = _cached_gate_up(w_gate, w_up)
        out = torch.empty(tuple(x.shape[:-1]) + (w_gate.shape[0],), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device.index or 0):
            K.swiglu_matmul(ops._st(x), ops._st(w), out=ops._st(out))
        return out
    return torch.nn.functional.silu(torch.nn.functional.linear(x, w_gate)) * torch.nn.functional.linear(x, w_up)


@swiglu_linear.register_fake
def _(x, w_gate, w_up):
    return x.new_empty(tuple(x.shape[:-1]) + (w_gate.shape[0],))


def _fused_attention_fits(q, k, v, head_dim: int) -> bool:
    """The fused kernel takes head_dim 128, fp16 and q / k / v of one shape; any other causal
    attention keeps torch's own formula (which decomposes into ops the device does have)."""
    return (head_dim == 128 and tuple(k.shape) == tuple(q.shape) and tuple(v.shape) == tuple(q.shape)
            and q.dtype == k.dtype == v.dtype == torch.float16)


@torch.library.custom_op("spyre::sdpa_causal", mutates_args=())
def sdpa_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale) on [batch, heads, seq,
    head_dim] tensors.  On spyre the heads are attended in the packed [batch, seq, heads*head_dim]
    form: when q / k / v are the usual transposed views of projection outputs, that form is the
    projection output itself and nothing is copied."""
    b, h, s, d = q.shape
    if _on_spyre(q) and _fused_attention_fits(q, k, v, d):
        packed = [t.transpose(1, 2).reshape(b, s, h * d) for t in (q, k, v)]
        out = torch.ops.spyre.causal_attention(packed[0], packed[1], packed[2], h, scale)
        return out.view(b, s, h, d).transpose(1, 2)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale)


@sdpa_causal.register_fake
def _(q, k, v, scale):
    b, h, s, d = q.shape
    return q.new_empty((b, s, h, d)).transpose(1, 2)


@torch.library.custom_op("spyre::causal_attention", mutates_args=())
def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int,
                     scale: float) -> torch.Tensor:
    """Causal softmax(q k^T * scale) v per head; q, k, v: [batch, seq, heads*head_dim]."""
    b, s, width = q.shape
    hd = width // heads
    if _on_spyre(q):
        from .. import ops, stick_ops as K

        # raises for any head size other than 128, unequal shapes or another dtype
        K.check_attention_args(q.shape, k.shape, v.shape, heads, (q.dtype, k.dtype, v.dtype))
        out = torch.empty_like(q)
        with torch.cuda.device(q.device.index or 0):
            K.causal_attention(ops._st(q), ops._st(k), ops._st(v), b, s, heads, scale, out=ops._st(out))
        return out
    qh, kh, vh = (t.view(b, s, heads, hd).transpose(1, 2) for t in (q, k, v))
    scores = torch.matmul(qh, kh.transpose(2, 3)) * scale
    mask = torch.full((s, s), float("-inf"), dtype=torch.float32).triu(1)
    probs = torch.softmax(scores.float() + mask, dim=-1).to(q.dtype)
    return torch.matmul(probs, vh).transpose(1, 2).reshape(b, s, width)


@causal_attention.register_fake
def _(q, k, v, heads, scale):
    return q.new_empty(q.size())
