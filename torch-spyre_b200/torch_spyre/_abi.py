"""ctypes binding of libspyre_b200.so, the C ABI declared in include/spyre_b200.h.

There is no fallback: if the library is missing or a call fails, an exception is
raised.  Pointers are passed as integers (``tensor.data_ptr()``), streams as the
integer ``cuda_stream`` handle.
"""
from __future__ import annotations

import ctypes
import os
from typing import Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libspyre_b200.so")

TS_OK = 0
TS_ERR_INVALID, TS_ERR_UNSUPPORTED, TS_ERR_CUDA, TS_ERR_ALIGNMENT, TS_ERR_TOO_LARGE = -1, -2, -3, -4, -5
TS_MAX_DIMS = 8

c_i64p = ctypes.POINTER(ctypes.c_int64)
c_i32p = ctypes.POINTER(ctypes.c_int32)
vp = ctypes.c_void_p


class PwInsn(ctypes.Structure):
    """struct ts_pw_insn."""

    _fields_ = [
        ("op", ctypes.c_int32),
        ("a_kind", ctypes.c_int32),
        ("a_idx", ctypes.c_int32),
        ("b_kind", ctypes.c_int32),
        ("b_idx", ctypes.c_int32),
        ("a_imm", ctypes.c_float),
        ("b_imm", ctypes.c_float),
    ]


_RELAYOUT_SIG = [vp, vp, ctypes.c_int, c_i64p, c_i64p, ctypes.c_int, c_i64p, c_i64p, c_i32p,
                 ctypes.c_int, vp]
_COPY_SIG = [vp, vp, vp, ctypes.c_int, c_i64p, c_i64p, ctypes.c_int, c_i64p, c_i64p, c_i32p,
             ctypes.c_int, vp]

# name -> (restype, argtypes); every symbol include/spyre_b200.h declares.
SIGNATURES = {
    "ts_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "ts_abi_version": (ctypes.c_int, []),
    "ts_last_cuda_error": (ctypes.c_char_p, []),
    "ts_relayout_to_sticks": (ctypes.c_int, _RELAYOUT_SIG),
    "ts_relayout_from_sticks": (ctypes.c_int, _RELAYOUT_SIG),
    "ts_host_span_bytes": (ctypes.c_int64, [ctypes.c_int, c_i64p, c_i64p, ctypes.c_int]),
    "ts_copy_host_to_sticks": (ctypes.c_int, _COPY_SIG),
    "ts_copy_sticks_to_host": (ctypes.c_int, _COPY_SIG),
    "ts_copy_staging_bytes": (ctypes.c_int64, [ctypes.c_int, c_i64p, c_i64p, ctypes.c_int]),
    "ts_copy_host_to_sticks_pipelined": (ctypes.c_int, [vp, vp, ctypes.c_int64, vp, ctypes.c_int, c_i64p, c_i64p,
                                                        ctypes.c_int, c_i64p, c_i64p, c_i32p, ctypes.c_int, vp]),
    "ts_copy_sticks_to_host_pipelined": (ctypes.c_int, [vp, vp, ctypes.c_int64, vp, ctypes.c_int, c_i64p, c_i64p,
                                                        ctypes.c_int, c_i64p, c_i64p, c_i32p, ctypes.c_int, vp]),
    "ts_transpose_tiles": (ctypes.c_int, [vp, c_i64p, ctypes.c_int, c_i64p, ctypes.c_int64, vp, c_i64p,
                                          ctypes.c_int, c_i64p, ctypes.c_int64, c_i64p, ctypes.c_int,
                                          ctypes.c_int, vp]),
    "ts_convert_sticks": (ctypes.c_int, [vp, ctypes.c_int, vp, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, vp]),
    "ts_embedding_rows": (ctypes.c_int, [vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, vp,
                                         ctypes.c_int64, ctypes.c_int64, vp]),
    "ts_gather_error_state": (ctypes.c_int, []),
    "ts_cumsum_rows": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int64, vp]),
    "ts_cumsum_mid": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, vp]),
    "ts_upsample_nearest2d": (ctypes.c_int, [vp, vp] + [ctypes.c_int64] * 5 + [vp]),
    "ts_layout_init": (ctypes.c_int, [c_i64p, ctypes.c_int, ctypes.c_int, c_i32p, c_i64p, c_i64p,
                                      c_i32p]),
    "ts_pointwise_chain": (ctypes.c_int, [ctypes.POINTER(PwInsn), ctypes.c_int,
                                          ctypes.POINTER(vp), c_i64p, ctypes.c_int,
                                          ctypes.POINTER(vp), ctypes.c_int, c_i64p, ctypes.c_int,
                                          ctypes.c_float, vp, ctypes.c_int, ctypes.c_int64, vp]),
    "ts_pointwise_static_count": (ctypes.c_int, []),
    "ts_softmax_rows": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, vp]),
    "ts_softmax_rows_causal": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                              ctypes.c_float, vp]),
    "ts_layernorm_rows": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_float, vp]),
    "ts_rmsnorm_rows": (ctypes.c_int, [vp, vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_float,
                                       ctypes.c_int, vp]),
    "ts_reduce_mid_scratch_bytes": (ctypes.c_int64, [ctypes.c_int64] * 3),
    "ts_reduce_mid": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                     ctypes.c_int, ctypes.c_float, vp, vp]),
    "ts_reduce_mid_static": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                            ctypes.c_int, ctypes.c_float, vp]),
    "ts_reduce_mid_static_max_bytes": (ctypes.c_int64, []),
    "ts_gemm_f16": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                   ctypes.c_int64, ctypes.c_int, ctypes.c_int, vp]),
    "ts_gemm_error_state": (ctypes.c_int, []),
    "ts_gemm_wait_selftest": (ctypes.c_int, [ctypes.c_int64, vp]),
    "ts_host_copy_selftest": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int]),
    "ts_peer_copy_2d": (ctypes.c_int, [vp, ctypes.c_int64, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, vp]),
    "ts_gemm_f16_scatter_add": (ctypes.c_int, [vp, vp, ctypes.POINTER(vp), ctypes.c_int, ctypes.c_int64,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_int, vp]),
    "ts_gemm_f16_scatter_store": (ctypes.c_int, [vp, vp, ctypes.POINTER(vp), ctypes.c_int, ctypes.c_int64,
                                                 ctypes.c_int64, ctypes.c_int64, ctypes.c_int, vp]),
    "ts_sum_slots_f16": (ctypes.c_int, [vp, ctypes.c_int, ctypes.c_int64, vp, vp, ctypes.c_int64, vp]),
    "ts_gemm_f16_swiglu": (ctypes.c_int, [vp, vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                          ctypes.c_int64, vp]),
    "ts_gemm_f16_residual": (ctypes.c_int, [vp, vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int64,
                                            ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                            vp]),
    "ts_gemm_f16_ex": (ctypes.c_int, [vp, ctypes.c_int64, ctypes.c_int64, vp, ctypes.c_int64,
                                      ctypes.c_int64, vp, vp, ctypes.c_int64, ctypes.c_int64,
                                      ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                      ctypes.c_int64, ctypes.c_int, ctypes.c_int, vp]),
    "ts_rotary_f16": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                     ctypes.c_int64, vp]),
    "ts_softmax_mid": (ctypes.c_int, [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                      ctypes.c_int, vp]),
    "ts_attention_causal_f16": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int64,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_float, vp]),
    "ts_attention_error_state": (ctypes.c_int, []),
}

_lib = None


class SpyreKernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SpyreKernelError(
                f"{LIB_PATH} is missing: build it with `python build.py` in the package's parent "
                "directory (nvcc, sm_100a).  There is no fallback path.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != TS_OK:
        text = lib().ts_status_string(status).decode()
        cuda = lib().ts_last_cuda_error().decode()
        raise SpyreKernelError(f"{what}: {text} ({status})" + (f"; CUDA: {cuda}" if cuda else ""))


def i64(values: Sequence[int]):
    return (ctypes.c_int64 * max(len(values), 1))(*values)


def i32(values: Sequence[int]):
    return (ctypes.c_int32 * max(len(values), 1))(*values)


def ptrs(values: Sequence[int]):
    return (vp * max(len(values), 1))(*values)
