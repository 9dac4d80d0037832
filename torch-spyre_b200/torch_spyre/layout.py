"""Host-side SpyreTensorLayout: the stick-tiled device layout of a tensor.

Mirrors the class the reference exposes through pybind
(torch_spyre/csrc/spyre_tensor_impl.h:29-93, bound in torch_spyre/csrc/module.cpp:
180-203): same three constructors, same read/write fields, same ``__str__``, same
nested ``StickFormat`` enum.  The arithmetic is done by ``ts_layout_init`` in the
kernel library so that Python and C++ callers share one implementation.
"""
from __future__ import annotations

import enum
from typing import List, Sequence

import torch

from . import _abi

BYTES_IN_STICK = 128


def elems_per_stick(dtype: torch.dtype) -> int:
    return BYTES_IN_STICK // dtype.itemsize


class SpyreTensorLayout:
    class StickFormat(enum.IntEnum):
        Dense = 0
        Sparse = 1
        SparseMulti = 2

    device_size: List[int]
    device_strides: List[int]
    dim_map: List[int]
    num_stick_dims: int
    format: "SpyreTensorLayout.StickFormat"

    def __init__(self, *args):
        """SpyreTensorLayout(host_size, dtype)
        SpyreTensorLayout(host_size, dtype, dim_order, format=Dense)
        SpyreTensorLayout(device_size, device_strides, dim_map, num_stick_dims, format)"""
        if len(args) == 5:
            size, strides, dmap, nstick, fmt = args
            self.device_size = [int(v) for v in size]
            self.device_strides = [int(v) for v in strides]
            self.dim_map = [int(v) for v in dmap]
            self.num_stick_dims = int(nstick)
            self.format = SpyreTensorLayout.StickFormat(fmt)
            self.elem_bytes = 2
            return
        if len(args) not in (2, 3, 4) or not isinstance(args[1], torch.dtype):
            raise TypeError("SpyreTensorLayout(host_size, dtype[, dim_order[, format]]) or "
                            "(device_size, device_strides, dim_map, num_stick_dims, format)")
        host_size = [int(v) for v in args[0]]
        dtype = args[1]
        dim_order = [int(v) for v in args[2]] if len(args) >= 3 else None
        fmt = args[3] if len(args) == 4 else SpyreTensorLayout.StickFormat.Dense
        rank = len(host_size)
        if rank < 1 or rank + 1 > _abi.TS_MAX_DIMS:
            raise ValueError(f"Unsupported tensor rank: {rank}")
        size = (_abi.ctypes.c_int64 * (rank + 1))()
        strides = (_abi.ctypes.c_int64 * (rank + 1))()
        dmap = (_abi.ctypes.c_int32 * (rank + 1))()
        n = _abi.lib().ts_layout_init(_abi.i64(host_size), rank, dtype.itemsize,
                                      _abi.i32(dim_order) if dim_order is not None else None,
                                      size, strides, dmap)
        if n < 0:
            _abi.check(n, "ts_layout_init")
        self.device_size = list(size)
        self.device_strides = list(strides)
        self.dim_map = list(dmap)
        self.num_stick_dims = 1
        self.format = SpyreTensorLayout.StickFormat(fmt)
        self.elem_bytes = dtype.itemsize

    def numel(self) -> int:
        n = 1
        for s in self.device_size:
            n *= s
        return n

    def __str__(self) -> str:
        return (f"SpyreTensorLayout(device_size={self.device_size}, "
                f"device_strides={self.device_strides}, dim_map ={self.dim_map}, "
                f"num_stick_dims={self.num_stick_dims}, format=\"{self.format.name}\")")

    __repr__ = __str__

    def __eq__(self, other) -> bool:
        return (isinstance(other, SpyreTensorLayout) and self.device_size == other.device_size
                and self.device_strides == other.device_strides and self.dim_map == other.dim_map
                and self.num_stick_dims == other.num_stick_dims and self.format == other.format)


def storage_nbytes(host_size: Sequence[int], dtype: torch.dtype) -> int:
    """Bytes of a device allocation for this host shape: whole sticks
    (torch_spyre/csrc/spyre_mem.cpp:598-611).  A 0-dim tensor is laid out as [1]
    (spyre_mem.cpp:625-631)."""
    hs = list(host_size) if len(host_size) else [1]
    if any(s == 0 for s in hs):
        return 0
    return SpyreTensorLayout(hs, dtype).numel() * dtype.itemsize
