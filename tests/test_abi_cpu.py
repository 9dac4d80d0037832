"""CPU tests: the C-ABI library loads, exports every declared symbol, and its
host-side logic (layout init, argument validation) behaves; no kernel runs."""
import ctypes
import json
import os
import re

import pytest
import torch

from torch_spyre import _abi, storage_nbytes
from torch_spyre.layout import SpyreTensorLayout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _declared_functions():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        text = open(os.path.join(inc, fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(ts_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    declared = _declared_functions()
    assert len(declared) >= 10
    handle = ctypes.CDLL(_abi.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), name
    # and the Python binding table covers the header
    assert sorted(_abi.SIGNATURES) == declared


def test_abi_version_and_status_text():
    lib = _abi.lib()
    assert lib.ts_abi_version() >= 1
    assert lib.ts_status_string(0) == b"ok"
    assert b"invalid" in lib.ts_status_string(-1)


def test_layout_reference_vectors():
    with open(os.path.join(GOLD, "layout_reference_vectors.json")) as f:
        gold = json.load(f)
    for v in gold["layouts"]:
        args = [v["host_size"], torch.float16] + ([v["dim_order"]] if v["dim_order"] else [])
        stl = SpyreTensorLayout(*args)
        assert stl.device_size == v["device_size"]
        assert stl.device_strides == v["device_strides"]
        assert stl.dim_map == v["dim_map"]
        assert stl.format == SpyreTensorLayout.StickFormat.Dense
        assert stl.num_stick_dims == 1
    assert str(SpyreTensorLayout(gold["str"]["host_size"], torch.float16)) == gold["str"]["text"]
    for v in gold["storage_nbytes"]:
        assert storage_nbytes(v["host_size"], torch.float16) == v["nbytes"]


def test_explicit_and_sparse_constructors():
    # tests/tensor/test_tensor_layout.py:64-87 of the reference
    x = SpyreTensorLayout([512, 256], torch.float16)
    y = SpyreTensorLayout([4, 512, 64], [32768, 64, 1], [1, 0, 1], 1,
                          SpyreTensorLayout.StickFormat.Dense)
    assert x == y
    s = SpyreTensorLayout([4, 512, 64], [32768, 64, 1], [1, 0, 1], 1,
                          SpyreTensorLayout.StickFormat.Sparse)
    assert s.format == SpyreTensorLayout.StickFormat.Sparse


def test_other_dtypes_stick_lengths():
    assert SpyreTensorLayout([64, 64], torch.float32).device_size == [2, 64, 32]
    assert SpyreTensorLayout([64, 64], torch.int8).device_size == [1, 64, 128]


def test_relayout_argument_validation_without_gpu():
    lib = _abi.lib()
    size, strides = _abi.i64([4, 64]), _abi.i64([64, 1])
    ds, dst, dm = _abi.i64([1, 4, 64]), _abi.i64([256, 64, 1]), _abi.i32([1, 0, 1])
    # null data pointers
    assert lib.ts_relayout_to_sticks(None, None, 2, size, strides, 2, ds, dst, dm, 3, None) == -1
    # bad element size, bad rank, bad dim_map
    assert lib.ts_relayout_to_sticks(16, 16, 3, size, strides, 2, ds, dst, dm, 3, None) == -1
    assert lib.ts_relayout_to_sticks(16, 16, 2, size, strides, 9, ds, dst, dm, 3, None) == -1
    assert lib.ts_relayout_to_sticks(16, 16, 2, size, strides, 2, ds, dst, _abi.i32([5, 0, 1]), 3,
                                     None) == -1
    # device layout smaller than the host tensor
    assert lib.ts_relayout_to_sticks(16, 16, 2, _abi.i64([4, 200]), strides, 2, ds, dst, dm, 3,
                                     None) == -1
    # empty tensors are a no-op
    assert lib.ts_relayout_from_sticks(None, None, 2, _abi.i64([0, 64]), strides, 2,
                                       _abi.i64([1, 0, 64]), dst, dm, 3, None) == 0


def test_host_span_bytes():
    lib = _abi.lib()
    assert lib.ts_host_span_bytes(2, _abi.i64([4, 64]), _abi.i64([64, 1]), 2) == 512
    assert lib.ts_host_span_bytes(2, _abi.i64([4, 64]), _abi.i64([1, 4]), 2) == 512
    assert lib.ts_host_span_bytes(2, _abi.i64([4, 64]), _abi.i64([128, 1]), 2) == (3 * 128 + 64) * 2
    assert lib.ts_host_span_bytes(2, _abi.i64([4, 64]), _abi.i64([-64, 1]), 2) == -1


def test_pointwise_argument_validation_without_gpu():
    lib = _abi.lib()
    ins = (_abi.PwInsn * 1)(_abi.PwInsn(0, 1, 0, 0, 0, 0.0, 0.0))
    shape = _abi.i64([1, 1, 4, 64])
    assert lib.ts_pointwise_chain(None, 1, None, None, 0, None, 0, shape, 0, 1.0, None, 0, 1,
                                  None) == -1
    # tensor operand index out of range
    assert lib.ts_pointwise_chain(ins, 1, None, None, 0, _abi.ptrs([16]), 1, shape, 0, 1.0, None,
                                  0, 1, None) == -1
    # input shape that is neither equal nor 1
    assert lib.ts_pointwise_chain(ins, 1, _abi.ptrs([16]), _abi.i64([1, 1, 3, 64]), 1,
                                  _abi.ptrs([16]), 1, shape, 0, 1.0, None, 0, 1, None) == -1
    # misaligned pointer
    assert lib.ts_pointwise_chain(ins, 1, _abi.ptrs([8]), _abi.i64([1, 1, 4, 64]), 1,
                                  _abi.ptrs([16]), 1, shape, 0, 1.0, None, 0, 1, None) == -4


def test_row_ops_validation_without_gpu():
    lib = _abi.lib()
    assert lib.ts_softmax_rows(None, None, 4, 64, 0, None) == -1
    assert lib.ts_softmax_rows(16, 16, 4, 1 << 20, 0, None) == -5
    assert lib.ts_softmax_rows(None, None, 0, 64, 0, None) == 0
    assert lib.ts_reduce_mid(16, 16, 4, 4, 63, 1, 1.0, None, None) == -1
    assert lib.ts_reduce_mid_scratch_bytes(1, 1 << 20, 64) > 0
    assert lib.ts_reduce_mid_scratch_bytes(4096, 16, 4096) == 0


@pytest.mark.parametrize("threads", [1, 2, 5, 8])
def test_helper_thread_copy_of_the_pageable_path(threads):
    """The team of helper threads that stages pageable host tensors (csrc/relayout.cu): every byte
    arrives, nothing beyond the span is written, for sizes around the slice and page boundaries
    and for more threads than pages; bad arguments are refused."""
    import numpy as np

    lib = _abi.lib()
    rng = np.random.default_rng(threads)
    for n in (0, 1, 4095, 4096, 4097, 70_000, (8 << 20) + 13, 33 << 20):
        src = rng.integers(0, 256, size=n + 64, dtype=np.uint8)
        dst = np.full(n + 64, 0xEE, dtype=np.uint8)
        rc = lib.ts_host_copy_selftest(dst.ctypes.data, src.ctypes.data, n, threads)
        assert rc == _abi.TS_OK
        assert np.array_equal(dst[:n], src[:n])
        assert (dst[n:] == 0xEE).all()
    buf = np.zeros(16, dtype=np.uint8)
    assert lib.ts_host_copy_selftest(buf.ctypes.data, buf.ctypes.data, -1, 2) == _abi.TS_ERR_INVALID
    assert lib.ts_host_copy_selftest(buf.ctypes.data, buf.ctypes.data, 8, 0) == _abi.TS_ERR_INVALID
    assert lib.ts_host_copy_selftest(None, buf.ctypes.data, 8, 2) == _abi.TS_ERR_INVALID
