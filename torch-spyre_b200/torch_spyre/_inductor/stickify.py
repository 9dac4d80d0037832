"""Layout description of a spyre tensor on the Inductor side: ``SpyreDCI`` ("device compute
info": which dim is the stick dim, in which order the dims are laid out) and ``SpyreFixedLayout``,
a ``FixedLayout`` that carries one (reference: torch_spyre/_inductor/stickify.py:28-135).

Every tensor the CUDA kernels see is in the generic stick layout (identity dim order, the innermost
dim is the stick dim), so nothing has to be propagated through the graph; the classes exist so that
code written against the reference's names keeps working, and ``spyre_strides`` is what the layout
oracle is pinned against."""
from __future__ import annotations

import dataclasses
import enum
from typing import List, Union

import torch
from torch._inductor.ir import FixedLayout

from . import Unsupported

BYTES_IN_STICK = 128


class StickFormat(enum.Enum):
    DENSE = 1
    SPARSE = 2
    SPARSE_MULTI = 3


def elems_per_stick(dtype: torch.dtype) -> int:
    return BYTES_IN_STICK // dtype.itemsize


@dataclasses.dataclass
class SpyreDCI:
    """dim_order follows the PyTorch convention: dim_order[-1] has the smallest stride and
    dim_order[-num_stick_dims:] are the stick dims."""

    dim_order: List[int]
    num_stick_dims: int = 1
    format: StickFormat = StickFormat.DENSE

    def __post_init__(self):
        assert self.num_stick_dims == 1, "currently limited to one stick dimension"

    @staticmethod
    def generic_stick_dci(t: torch.Tensor) -> "SpyreDCI":
        return SpyreDCI(list(range(len(t.size()))))

    def get_stick_dims(self) -> List[int]:
        return self.dim_order[-self.num_stick_dims:]

    def is_stick_dim(self, dim: Union[int, List[int]]) -> bool:
        dims = [dim] if isinstance(dim, int) else list(dim)
        return any(d in self.get_stick_dims() for d in dims)

    def is_stick_reduction(self, axis: List[int]) -> bool:
        stick = [d in self.get_stick_dims() for d in axis]
        if any(stick) and not all(stick):
            raise Unsupported(f"reduction on both stick and non-stick dimensions {axis}")
        return any(stick)

    def spyre_strides(self, size, dtype: torch.dtype) -> list:
        cur = 1 if self.format == StickFormat.DENSE else elems_per_stick(dtype)
        strides = [-1] * len(size)
        for d in reversed(self.dim_order):
            strides[d] = cur
            cur = cur * size[d]
        return strides

    def spyre_layout(self, device: torch.device, size, dtype: torch.dtype) -> "SpyreFixedLayout":
        return SpyreFixedLayout(device, dtype, list(size), self.spyre_strides(size, dtype), self)


class SpyreFixedLayout(FixedLayout):
    dci: SpyreDCI

    def __init__(self, device, dtype, size, stride, dci: SpyreDCI) -> None:
        super().__init__(device, dtype, size, stride)
        self.dci = dci

    def __str__(self) -> str:
        index = "" if self.device.index is None else f":{self.device.index}"
        return (f"{type(self).__name__}('{self.device.type}{index}', {self.dtype}, size={self.size}, "
                f"stride={self.stride}, dci={self.dci})")

    def get_allocation_size(self):
        return self.size

    __repr__ = __str__
