"""Inductor heuristics for the spyre device (reference: SpyreHeuristics,
torch_spyre/_inductor/choices.py:22-83).  The reference switches every fusion off, so each op is a
kernel of its own and each intermediate a round trip through device memory; here fusion stays on
(the scheduling class says which pairs it can turn into one program) and what is switched off is
what the kernels do themselves: reductions are neither split in two stages nor made cooperative."""
from __future__ import annotations

import torch
from torch._inductor.choices import InductorChoices


class SpyreHeuristics(InductorChoices):
    @staticmethod
    def should_use_cooperative_reduction(features) -> bool:
        return False

    @staticmethod
    def should_use_persistent_reduction(features, cooperative_reduction: bool) -> bool:
        return True

    @staticmethod
    def want_no_x_dim(features) -> bool:
        return False

    @staticmethod
    def reduction_split_factor(device: torch.device, reduction_numel_hint: int, numel_hint: int,
                               inner_reduction: bool) -> int:
        """A row reduction is one launch whatever its length: the kernel spreads a row over a CTA."""
        return 1
