"""Batch / row sharding across the GPUs of one node.

The reference is single-device (torch_spyre/__init__.py:87-89 hard-codes a device count of
one); here every workload of the hot path is independent along its leading dim, so N ranks
(one process per GPU) each take a contiguous block of leading indices and no collective
touches the data.  Shard on the host side, before the relayout: each GPU then holds the stick
image of its own slice."""
from __future__ import annotations

from typing import Tuple


def shard_rows(total: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of `rank`'s block when `total` leading indices are split over `world`
    ranks as evenly as possible (the first `total % world` ranks get one more)."""
    if world < 1 or not (0 <= rank < world) or total < 0:
        raise ValueError(f"bad shard request: total={total} rank={rank} world={world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)
