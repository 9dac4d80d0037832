"""CPU tests of the multi-process path bench.py uses at N > 1: world_size-2 gloo ranks shard
the rows of a workload, no collective touches the data, and the timing reduction is a MAX."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torch_spyre.sharding import shard_rows


def test_shard_rows_covers_everything_once():
    for total, world in [(8192, 1), (8192, 2), (8192, 8), (67, 4), (5, 8), (32, 8), (64, 3)]:
        spans = [shard_rows(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a0 <= a1
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(67, 256, generator=g).half()          # every rank builds the same global input
    a = (torch.rand(256, generator=g) * 2 - 1).half()
    lo, hi = shard_rows(x.shape[0], rank, world)
    y_local = torch.exp(x[lo:hi] * a).sum(-1)              # the rank's own rows only: no exchange
    # timing reduction as in bench.py: the slowest rank defines the step time
    t = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.barrier()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    torch.save({"lo": lo, "hi": hi, "y": y_local, "t": float(t)}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_without_exchange(tmp_path):
    world, port = 2, _free_port()
    mp.start_processes(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, start_method="spawn")
    parts = [torch.load(os.path.join(tmp_path, f"r{r}.pt")) for r in range(world)]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(67, 256, generator=g).half()
    a = (torch.rand(256, generator=g) * 2 - 1).half()
    want = torch.exp(x * a).sum(-1)
    got = torch.cat([p["y"] for p in parts])
    assert torch.equal(got, want)
    assert [p["t"] for p in parts] == [2.0, 2.0]
    assert parts[0]["hi"] == parts[1]["lo"]
