"""CPU oracle for the stick-tiled tensor layout and the host<->device relayout.

TEST INFRASTRUCTURE ONLY.  Nothing on the product path may import this module;
only the test-suite, the smoke check and the benchmark's CPU-baseline leg do.

It restates, in numpy, two pieces of the reference:

* ``SpyreTensorLayout::init`` (torch_spyre/csrc/spyre_tensor_impl.cpp:39-74):
  host size + element size (+ dim_order) -> device_size / device_strides /
  dim_map, one stick = 128 bytes, stick dim stored twice (outermost as the
  stick count, innermost as the position inside the stick).
* the element walk that ``get_device_stride_info`` describes for the
  host<->device copy (torch_spyre/csrc/spyre_mem.cpp:213-244): every host index
  is decomposed along the device dims that ``dim_map`` assigns to its host dim
  and lands at the sum of ``index * device_stride``.  The per-rank dim order of
  the copy path (``get_device_layout``, spyre_mem.cpp:70-91) is available as
  ``legacy_copy_layout``.

Parity status: the layout metadata is pinned by the reference's golden vectors
(tests/tensor/test_tensor_layout.py:27-94, tests/test_spyre.py:171-176).  The
device byte image is pinned by no reference test (only round trips are), so the
image is defined here as: the layout above, pad lanes zero, element bits
unchanged.  "parity unpinned" for the image itself.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

import numpy as np

BYTES_IN_STICK = 128  # spyre_tensor_impl.cpp:27

DENSE, SPARSE, SPARSE_MULTI = 0, 1, 2
_FORMAT_NAMES = {DENSE: "Dense", SPARSE: "Sparse", SPARSE_MULTI: "SparseMulti"}


@dataclass
class Layout:
    device_size: List[int]
    device_strides: List[int]
    dim_map: List[int]
    num_stick_dims: int = 1
    format: int = DENSE
    elem_bytes: int = 2

    def numel_device(self) -> int:
        n = 1
        for s in self.device_size:
            n *= s
        return n

    def __str__(self) -> str:  # spyre_tensor_impl.cpp:76-111
        return (
            f"SpyreTensorLayout(device_size={list(self.device_size)}, "
            f"device_strides={list(self.device_strides)}, "
            f"dim_map ={list(self.dim_map)}, "
            f"num_stick_dims={self.num_stick_dims}, "
            f'format="{_FORMAT_NAMES[self.format]}")'
        )


def generic_stick_layout(
    host_size: Sequence[int],
    elem_bytes: int = 2,
    dim_order: Sequence[int] | None = None,
    fmt: int = DENSE,
) -> Layout:
    """spyre_tensor_impl.cpp:29-74."""
    host_dims = len(host_size)
    if dim_order is None:
        dim_order = list(range(host_dims))
    device_dims = host_dims + 1
    elems = BYTES_IN_STICK // elem_bytes
    size = [0] * device_dims
    dmap = [0] * device_dims
    stick_dim = dim_order[host_dims - 1]
    dmap[0] = stick_dim
    dmap[device_dims - 1] = stick_dim
    size[0] = (host_size[stick_dim] + elems - 1) // elems
    size[device_dims - 1] = elems
    for i in range(1, device_dims - 1):
        dmap[i] = dim_order[i - 1]
        size[i] = host_size[dim_order[i - 1]]
    strides = [0] * device_dims
    cur = elems
    strides[device_dims - 1] = 1
    for i in range(device_dims - 2, -1, -1):
        strides[i] = cur
        cur *= size[i]
    return Layout(size, strides, dmap, 1, fmt, elem_bytes)


def legacy_copy_layout(host_size: Sequence[int], elem_bytes: int = 2) -> Layout:
    """The per-rank device dim order the reference's copy path uses
    (get_device_layout, spyre_mem.cpp:70-91, listed there innermost first),
    expressed as a Layout (outermost first).  The reference only handles an
    inner dim that is a stick multiple or shorter than one stick
    (spyre_mem.cpp:104-109); here the stick count is the ceiling, which agrees
    with it on both of those cases."""
    rank = len(host_size)
    inner_first = {1: [0, 0], 2: [1, 0, 1], 3: [2, 0, 2, 1], 4: [3, 2, 1, 3, 0]}
    if rank not in inner_first:
        raise ValueError(f"Unsupported tensor rank: {rank}")  # spyre_mem.cpp:85-88
    order = inner_first[rank]
    elems = BYTES_IN_STICK // elem_bytes
    stick_dim = order[0]
    dmap = list(reversed(order))
    size = []
    for pos, d in enumerate(dmap):
        if d == stick_dim:
            last = pos == len(dmap) - 1
            size.append(elems if last else (host_size[d] + elems - 1) // elems)
        else:
            size.append(host_size[d])
    strides = [0] * len(size)
    cur = 1
    for i in range(len(size) - 1, -1, -1):
        strides[i] = cur
        cur *= size[i]
    return Layout(size, strides, dmap, 1, DENSE, elem_bytes)


def storage_nbytes(host_size: Sequence[int], elem_bytes: int = 2) -> int:
    """Bytes a device allocation of this host shape occupies: whole sticks
    (spyre_mem.cpp:598-611; a 2-element fp16 tensor is 128 bytes,
    tests/test_spyre.py:171-176).  A 0-dim tensor is treated as [1]
    (spyre_mem.cpp:625-631)."""
    hs = list(host_size) if len(host_size) else [1]
    lay = generic_stick_layout(hs, elem_bytes)
    return lay.numel_device() * elem_bytes


def device_offsets(host_size: Sequence[int], lay: Layout) -> np.ndarray:
    """Device element offset of every host index, shape == host_size.

    Host dim h owns the device dims d with dim_map[d] == h; its index is split
    over them in mixed radix, outermost device dim most significant
    (spyre_mem.cpp:213-244 builds exactly these per-dim (size, stride) pairs).
    """
    rank = len(host_size)
    off = np.zeros(tuple(host_size), dtype=np.int64)
    for h in range(rank):
        devs = [d for d in range(len(lay.dim_map)) if lay.dim_map[d] == h]
        idx = np.arange(host_size[h], dtype=np.int64)
        contrib = np.zeros(host_size[h], dtype=np.int64)
        rem = idx
        for d in reversed(devs):  # innermost first
            if d == devs[0]:
                q = rem
            else:
                q = rem % lay.device_size[d]
                rem = rem // lay.device_size[d]
            contrib += q * lay.device_strides[d]
        shape = [1] * rank
        shape[h] = host_size[h]
        off = off + contrib.reshape(shape)
    return off


def to_sticks(host: np.ndarray, lay: Layout) -> np.ndarray:
    """Host tensor (any strides, viewed as an unsigned integer of the element
    width) -> flat device image with zero padding."""
    image = np.zeros(lay.numel_device(), dtype=host.dtype)
    if host.size:
        image[device_offsets(host.shape, lay).reshape(-1)] = host.reshape(-1)
    return image


def from_sticks(image: np.ndarray, lay: Layout, host_size: Sequence[int]) -> np.ndarray:
    """Flat device image -> contiguous host tensor."""
    if int(np.prod(host_size)) == 0:
        return np.zeros(tuple(host_size), dtype=image.dtype)
    return image[device_offsets(host_size, lay)]


def to_sticks_generic_fast(host: np.ndarray, elem_bytes: int = 2) -> np.ndarray:
    """Same image as to_sticks(host, generic_stick_layout(host.shape)), built by
    pad -> reshape -> move the stick count outermost; used at full benchmark
    sizes where the index-array form above would need too much memory."""
    elems = BYTES_IN_STICK // elem_bytes
    inner = host.shape[-1]
    n_sticks = (inner + elems - 1) // elems
    pad = n_sticks * elems - inner
    if pad:
        width = [(0, 0)] * (host.ndim - 1) + [(0, pad)]
        host = np.pad(host, width)
    tiled = host.reshape(host.shape[:-1] + (n_sticks, elems))
    return np.ascontiguousarray(np.moveaxis(tiled, -2, 0)).reshape(-1)


def from_sticks_generic_fast(image: np.ndarray, host_size: Sequence[int], elem_bytes: int = 2) -> np.ndarray:
    elems = BYTES_IN_STICK // elem_bytes
    inner = host_size[-1]
    n_sticks = (inner + elems - 1) // elems
    tiled = image.reshape((n_sticks,) + tuple(host_size[:-1]) + (elems,))
    full = np.moveaxis(tiled, 0, -2).reshape(tuple(host_size[:-1]) + (n_sticks * elems,))
    return np.ascontiguousarray(full[..., :inner])
