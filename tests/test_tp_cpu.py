"""Partitioning of the decoder layer's weights for tensor parallelism, checked on CPU: the shards
cover the weights exactly, split on stick boundaries, and the sharded arithmetic (column-parallel
projections, row-parallel projections summed over ranks) equals the unsharded layer."""
import pytest
import torch
import torch.nn.functional as F

from oracle import llama_ref as L
from torch_spyre import tensor_parallel as TP


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_cover_the_weights_on_stick_boundaries(world):
    cfg = L.LayerConfig(d_model=1024, heads=8, ffn=11008 // 4)        # 2752 = 43 sticks: uneven over 2, 4, 8 ranks
    w = L.make_weights(cfg)
    shards = [TP.shard_layer_weights(w, cfg.heads, r, world) for r in range(world)]
    for name in ("q", "k", "v", "gate", "up"):
        assert torch.equal(torch.cat([s[name] for s in shards], 0), w[name])
    for name in ("o", "down"):
        assert torch.equal(torch.cat([s[name] for s in shards], 1), w[name])
    for s in shards:
        assert s["gate"].shape[0] % 64 == 0 and s["down"].shape[1] == s["gate"].shape[0]
        assert s["q"].shape[0] == cfg.d_model // world and s["o"].shape[1] == cfg.d_model // world
    assert sum(TP.shard_bounds(11008, r, 8)[1] - TP.shard_bounds(11008, r, 8)[0] for r in range(8)) == 11008
    assert all((TP.shard_bounds(11008, r, 8)[0] % 64, TP.shard_bounds(11008, r, 8)[1] % 64) == (0, 0) for r in range(8))
    with pytest.raises(ValueError):
        TP.shard_layer_weights(w, cfg.heads, 0, 3)


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_arithmetic_equals_the_unsharded_layer(world):
    """The data flow of TPDecoderLayer in plain torch, fp32: per-rank column-parallel projections
    and attention on the rank's heads, row-parallel projections summed over the ranks."""
    cfg = L.LayerConfig(d_model=256, heads=4, ffn=512)
    w = {k: v.float() for k, v in L.make_weights(cfg).items()}
    b, s = 2, 32
    x = torch.randn(b, s, cfg.d_model, generator=torch.Generator().manual_seed(0))
    want = L.layer_forward(x, w, cfg)
    hd = cfg.head_dim
    cos, sin = (t.float() for t in L.rope_tables(s, hd))
    shards = [TP.shard_layer_weights(w, cfg.heads, r, world) for r in range(world)]
    h = L.rms_norm(x, w["norm1"], cfg.eps)
    partial = []
    for sh in shards:
        nh = cfg.heads // world
        q, k, v = (F.linear(h, sh[n]).view(b, s, nh, hd).transpose(1, 2) for n in ("q", "k", "v"))
        q = q * cos[None, None] + L.rotate_half(q) * sin[None, None]
        k = k * cos[None, None] + L.rotate_half(k) * sin[None, None]
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, nh * hd)
        partial.append(F.linear(a, sh["o"]))
    x2 = x + sum(partial)
    h2 = L.rms_norm(x2, w["norm2"], cfg.eps)
    y = x2 + sum(F.linear(F.silu(F.linear(h2, sh["gate"])) * F.linear(h2, sh["up"]), sh["down"]) for sh in shards)
    torch.testing.assert_close(y, want, rtol=1e-4, atol=1e-4)
