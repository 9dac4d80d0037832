"""ctypes loader for the C restatement of the stick relayout (relayout_oracle.c).

TEST INFRASTRUCTURE ONLY: used by tests, the smoke check and the benchmark's
CPU-baseline leg.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Sequence

import numpy as np

from .layout import Layout

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "librelayout_oracle.so")
_lib = None


def build() -> str:
    subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        sig = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
               ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64), ctypes.c_int,
               ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64),
               ctypes.POINTER(ctypes.c_int32), ctypes.c_int, ctypes.c_int]
        for fn in (_lib.oracle_to_sticks, _lib.oracle_from_sticks):
            fn.argtypes = sig
            fn.restype = ctypes.c_int
    return _lib


def _i64(v: Sequence[int]):
    return (ctypes.c_int64 * max(len(v), 1))(*v)


def _i32(v: Sequence[int]):
    return (ctypes.c_int32 * max(len(v), 1))(*v)


def to_sticks(host: np.ndarray, lay: Layout, nthreads: int = 1) -> np.ndarray:
    """host: numpy array of any strides (element strides taken from it)."""
    eb = host.dtype.itemsize
    image = np.empty(lay.numel_device(), dtype=host.dtype)
    strides = [s // eb for s in host.strides]
    rc = lib().oracle_to_sticks(
        host.ctypes.data, image.ctypes.data, eb, _i64(host.shape), _i64(strides), host.ndim,
        _i64(lay.device_size), _i64(lay.device_strides), _i32(lay.dim_map),
        len(lay.device_size), nthreads)
    assert rc == 0
    return image


def from_sticks(image: np.ndarray, lay: Layout, host_size: Sequence[int], nthreads: int = 1,
                out: np.ndarray | None = None) -> np.ndarray:
    eb = image.dtype.itemsize
    if out is None:
        out = np.zeros(tuple(host_size), dtype=image.dtype)
    strides = [s // eb for s in out.strides]
    rc = lib().oracle_from_sticks(
        image.ctypes.data, out.ctypes.data, eb, _i64(host_size), _i64(strides), len(host_size),
        _i64(lay.device_size), _i64(lay.device_strides), _i32(lay.dim_map),
        len(lay.device_size), nthreads)
    assert rc == 0
    return out
