"""Tensor-parallel linears for the decoder layer, one process per GPU.

The reference is single-device (torch_spyre/__init__.py:87-89 hard-codes one device); its model
ladder ends at a sharded-size Llama decoder layer (tests/test_modules.py:133-211).  Here a layer
can be split over the GPUs of one box the Megatron way, with the activations sharded by rows
(tokens) between the blocks:

    x_shard [M/R, d] -> RMSNorm -> all-gather [M, d]
        -> column-parallel q, k, v  (each rank: its heads)      [M, d/R]
        -> rotary, causal attention on the rank's heads
        -> row-parallel o_proj, reduce-scatter in the GEMM epilogue, + residual -> [M/R, d]
    -> RMSNorm -> all-gather -> column-parallel SwiGLU gate/up [M, f/R]
        -> row-parallel down_proj, reduce-scatter in the GEMM epilogue, + residual -> [M/R, d]

The two reduce-scatters are not separate collectives: ``ts_gemm_f16_scatter_store`` stores every
tile of the rank's partial product into the rank's own slot in the owning rank's memory over NVLink
(plain 16-byte stores covering whole sticks) while the rest of the GEMM is still running, so per
layer 2 x [M, d] fp16 cross NVLink under the matmuls; the owner then sums its slots locally in
fp32 (``ts_sum_slots_f16``, which also adds the residual).  (``ts_gemm_f16_scatter_add``, fp16
reductions straight into one buffer per owner, is the same idea without the slots; reductions cross
NVLink far below link rate, which made the layer slower on 8 GPUs than on 4.)  The all-gathers are peer copies of each rank's
row block into every rank's full image (the copy engines, one 2-D copy per peer).  Buffers that
peers write live in symmetric memory (``torch.distributed._symmetric_memory``); ordering between
ranks is its device-side barrier on the current stream.  No TMA copy ever names a peer's memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import stick_ops as K
from .sharding import shard_rows
from .stick_ops import StickTensor

STICK = 64


# ---- partitioning (no device needed) ------------------------------------------------------------

def shard_bounds(total: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of this rank's block of `total` features: whole sticks (64 features) when the
    total is a whole number of sticks, so that every shard is a valid K for the GEMM and a valid
    stick-aligned N; the first ranks take the extra sticks when they do not divide evenly."""
    if total % STICK == 0:
        lo, hi = shard_rows(total // STICK, rank, world)
        return lo * STICK, hi * STICK
    return shard_rows(total, rank, world)


def shard_columns(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Column-parallel shard of a linear weight [N, K]: this rank's block of output features."""
    lo, hi = shard_bounds(w.shape[0], rank, world)
    return w[lo:hi].contiguous()


def shard_reduction(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Row-parallel shard of a linear weight [N, K]: this rank's block of the reduction dim."""
    lo, hi = shard_bounds(w.shape[1], rank, world)
    return w[:, lo:hi].contiguous()


def shard_layer_weights(w: Dict[str, torch.Tensor], heads: int, rank: int, world: int) -> Dict[str, torch.Tensor]:
    """The decoder layer's weights for one rank: q / k / v by whole heads, gate / up by output
    features, o / down by the matching blocks of their reduction dim, norms replicated."""
    if heads % world:
        raise ValueError(f"{heads} heads cannot be split over {world} ranks")
    hd = w["q"].shape[0] // heads
    lo, hi = (heads // world) * rank * hd, (heads // world) * (rank + 1) * hd
    out = {k: w[k][lo:hi].contiguous() for k in ("q", "k", "v")}
    out["o"] = w["o"][:, lo:hi].contiguous()
    out["gate"], out["up"] = shard_columns(w["gate"], rank, world), shard_columns(w["up"], rank, world)
    out["down"] = shard_reduction(w["down"], rank, world)
    if out["gate"].shape[0] % STICK or out["gate"].shape[0] == 0:
        raise ValueError(f"FFN width {w['gate'].shape[0]} does not split into whole sticks over {world} ranks")
    out["norm1"], out["norm2"] = w["norm1"], w["norm2"]
    return out


# ---- symmetric buffers ----------------------------------------------------------------------------

@dataclass
class PeerBuffer:
    """An fp16 buffer every rank allocates identically, with the device addresses of all ranks'
    copies."""
    local: torch.Tensor          # flat CUDA fp16 tensor (this rank's copy)
    ptrs: List[int]              # device address of each rank's copy, index = rank
    handle: object


class TPGroup:
    def __init__(self, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.dist, self.symm_mem = dist, symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("one box: at most 8 ranks")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._sync: Optional[PeerBuffer] = None

    def buffer(self, numel: int) -> PeerBuffer:
        t = self.symm_mem.empty(numel, dtype=torch.float16, device=self.device)
        hdl = self.symm_mem.rendezvous(t, self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        if ptrs[self.rank] != t.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe the local buffer")
        buf = PeerBuffer(t, ptrs, hdl)
        if self._sync is None:
            self._sync = buf
        return buf

    def barrier(self) -> None:
        """All ranks' work enqueued so far on their current streams is complete, and visible to
        peers, before any rank's later work starts (symmetric memory's device-side barrier)."""
        if self._sync is None:
            self.buffer(STICK)
        self._sync.handle.barrier()


# ---- the sharded ops ------------------------------------------------------------------------------

def all_gather_rows(tp: TPGroup, shard: StickTensor, full: PeerBuffer, rows_total: int,
                    entry_barrier: bool = True) -> StickTensor:
    """Every rank's [rows, cols] block copied into every rank's image of [rows_total, cols].  In the
    stick image a row block is one contiguous piece per stick column: a 2-D copy per peer.
    `entry_barrier=False` when the caller knows that every rank has passed a barrier since it last
    read `full` (its old contents are then dead everywhere)."""
    rows, cols = shard.rows, shard.cols
    sticks = -(-cols // STICK)
    width, spitch, dpitch = rows * 128, rows * 128, rows_total * 128
    off = tp.rank * rows * 128
    stream = torch.cuda.current_stream().cuda_stream
    if entry_barrier:
        tp.barrier()      # every rank is done reading the previous contents of `full`
    for peer in range(tp.world):
        rc = K._abi.lib().ts_peer_copy_2d(full.ptrs[peer] + off, dpitch, shard.ptr(), spitch, width, sticks, stream)
        K._abi.check(rc, f"ts_peer_copy_2d to rank {peer}")
    tp.barrier()          # every block has landed everywhere
    return StickTensor(full.local[: sticks * rows_total * STICK], (rows_total, cols))


def row_parallel_linear(tp: TPGroup, a: StickTensor, w_local: StickTensor, slots: PeerBuffer,
                        residual_shard: Optional[StickTensor], entry_barrier: bool = True) -> StickTensor:
    """a: [M, K/R] (this rank's slice of the reduction dim), w_local: [N, K/R].  Returns this rank's
    [M/R, N] block of a @ w^T summed over the ranks (+ residual_shard).  `slots` holds, on every rank,
    one [M/R, N] image per writing rank: the GEMM stores each block of rows of its partial product
    into its own slot on the owning rank (whole sticks over NVLink, under the rest of the GEMM), and
    after the barrier the owner adds its slots up locally in fp32."""
    M, N = a.rows, w_local.shape[0]
    rows = M // tp.world
    n = (-(-N // STICK)) * rows * STICK                 # elements of one slot
    if slots.local.numel() < tp.world * n:
        raise ValueError("slot buffer too small for one image per rank")
    if entry_barrier:     # (not needed when every rank has passed a barrier since it last summed `slots`)
        tp.barrier()      # every owner has finished adding up the slots of the previous call
    mine = [slots.ptrs[owner] + tp.rank * n * 2 for owner in range(tp.world)]
    K.matmul_scatter_store(a, w_local, mine, b_kmajor=True)
    tp.barrier()          # every rank's stores have landed
    return K.sum_slots(slots.local, tp.world, (rows, N), residual_shard)


class TPDecoderLayer:
    """The Llama-style decoder layer of the benchmark, sharded over the ranks of `tp`.  Takes and
    returns this rank's block of rows of the [batch * seq, d_model] activations."""

    def __init__(self, tp: TPGroup, weights: Dict[str, torch.Tensor], heads: int, eps: float,
                 cos: torch.Tensor, sin: torch.Tensor, batch: int, seq: int, buffers=None):
        """`buffers`: the (gathered activations, o-projection slots, down-projection slots) peer
        buffers of another layer of the same shape, to share them.  That is safe for layers run
        one after the other: a layer's first write into a peer's buffer comes after its first
        barrier, which completes only when every rank has finished the layer before."""
        from ._inductor.customops import interleave_gate_up

        self.tp, self.eps, self.batch, self.seq = tp, eps, batch, seq
        self.heads_local = heads // tp.world
        w = shard_layer_weights(weights, heads, tp.rank, tp.world)
        w["gate_up"] = interleave_gate_up(w.pop("gate"), w.pop("up"))
        self.w = {k: K.copy_host_to_sticks(v.contiguous()) for k, v in w.items()}
        self.cos, self.sin = K.copy_host_to_sticks(cos.contiguous()), K.copy_host_to_sticks(sin.contiguous())
        self.d = weights["q"].shape[1]
        self.M = batch * seq
        if self.M % tp.world or (self.M // tp.world) % 32:
            raise ValueError("rows per rank must be a multiple of 32")
        self.rows = self.M // tp.world
        if buffers is None:
            # gathered activations [M, d]; one [rows, d] image per writing rank for each of the two
            # row-parallel linears
            buffers = (tp.buffer(self.M * self.d), tp.buffer(tp.world * self.rows * self.d),
                       tp.buffer(tp.world * self.rows * self.d))
        self.buffers = buffers
        self.full, self.out_a, self.out_b = buffers
        self.nvlink_bytes_per_call = 0

    def __call__(self, x_shard: StickTensor) -> StickTensor:
        tp, w = self.tp, self.w
        R = tp.world
        # Four barriers per layer: one after each gather and one after each scatter.  The entry
        # barriers of the helpers are not needed here: between a rank's last read of `full` (or its
        # sum over a slot buffer) and the next write into it by any peer lies at least one of those
        # four, and a barrier completes only when every rank's earlier work on its stream has.
        h = K.rmsnorm_rows(x_shard, w["norm1"], self.eps)
        hf = all_gather_rows(tp, h, self.full, self.M, entry_barrier=False)
        q = K.matmul(hf, w["q"], b_kmajor=True)
        k = K.matmul(hf, w["k"], b_kmajor=True)
        v = K.matmul(hf, w["v"], b_kmajor=True)
        width = self.heads_local * 128
        shape3 = (self.batch, self.seq, width)
        q = K.rotary(StickTensor(q.image, shape3), self.cos, self.sin, self.batch, self.seq, self.heads_local)
        k = K.rotary(StickTensor(k.image, shape3), self.cos, self.sin, self.batch, self.seq, self.heads_local)
        attn = K.causal_attention(q, k, StickTensor(v.image, shape3), self.batch, self.seq, self.heads_local,
                                  128 ** -0.5)
        x2 = row_parallel_linear(tp, StickTensor(attn.image, (self.M, width)), w["o"], self.out_a, x_shard,
                                 entry_barrier=False)
        h2 = K.rmsnorm_rows(x2, w["norm2"], self.eps)
        hf2 = all_gather_rows(tp, h2, self.full, self.M, entry_barrier=False)
        act = K.swiglu_matmul(hf2, w["gate_up"])
        y = row_parallel_linear(tp, act, w["down"], self.out_b, x2, entry_barrier=False)
        # bytes this rank sent to peers: two gathers of its block and two scatters of its partial product
        self.nvlink_bytes_per_call = 2 * (R - 1) * self.rows * self.d * 2 + 2 * (R - 1) * self.rows * self.d * 2
        return y


class TPLlamaModel:
    """Token ids to logits over the ranks of `tp`: the next rung above the sharded decoder layer
    (the reference's module ladder, tests/test_modules.py:133-211, stops at one layer on one
    device).  The activations stay sharded by rows from the embedding to the logits: every rank
    looks up its own block of tokens (the table, the final norm and the output projection are
    replicated), runs the stack of TPDecoderLayer, which share one set of peer buffers, and
    returns the logits of its rows."""

    def __init__(self, tp: TPGroup, weights: Dict, heads: int, eps: float, cos: torch.Tensor,
                 sin: torch.Tensor, batch: int, seq: int):
        self.tp, self.eps = tp, eps
        self.embed = K.copy_host_to_sticks(weights["embed"].contiguous())
        self.final_norm = K.copy_host_to_sticks(weights["final_norm"].contiguous())
        self.lm_head = K.copy_host_to_sticks(weights["lm_head"].contiguous())
        self.layers: List[TPDecoderLayer] = []
        for w in weights["layers"]:
            shared = self.layers[0].buffers if self.layers else None
            self.layers.append(TPDecoderLayer(tp, w, heads, eps, cos, sin, batch, seq, buffers=shared))
        self.rows = self.layers[0].rows if self.layers else batch * seq // tp.world

    def __call__(self, ids_shard: torch.Tensor) -> StickTensor:
        """`ids_shard`: this rank's block of the flattened [batch * seq] token ids (int32 or int64,
        on this rank's GPU).  Returns the [rows, vocab] logits of those tokens."""
        if ids_shard.numel() != self.rows:
            raise ValueError(f"expected {self.rows} token ids, got {ids_shard.numel()}")
        x = K.embedding_rows(self.embed, ids_shard)
        for layer in self.layers:
            x = layer(x)
        x = K.rmsnorm_rows(x, self.final_norm, self.eps)
        return K.matmul(x, self.lm_head, b_kmajor=True)
