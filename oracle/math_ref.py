"""Math oracle: torch CPU eager on seeded inputs.  TEST INFRASTRUCTURE ONLY.

The reference's own tests compare the device against torch CPU eager
(tests/test_ops.py:40-55, tests/test_modules.py:39-67,
tests/_inductor/utils_inductor.py:186-249), and that is the oracle the
benchmark configurations name.  Tolerance for fp16 math: rtol 1e-2, atol 1e-3
(tests/test_modules.py:39-40).
"""
from __future__ import annotations

import torch

RTOL, ATOL = 1e-2, 1e-3


def gen(seed: int = 0) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def softmax_inputs(rows=256, cols=4096, seed=0):
    """Config 1: fp16 softmax over dim -1, values N(0,1) from seed 0."""
    return torch.randn(rows, cols, generator=gen(seed)).half()


def fused_inputs(rows=8192, cols=8192, seed=0):
    """Config 2: x N(0,1) [rows, cols]; a, b U(-1,1) [cols]."""
    g = gen(seed)
    x = torch.randn(rows, cols, generator=g).half()
    a = (torch.rand(cols, generator=g) * 2 - 1).half()
    b = (torch.rand(cols, generator=g) * 2 - 1).half()
    return x, a, b


def fused_ref(x, a, b):
    return torch.exp(x * a + b).sum(-1)


def relayout_inputs(shape=(64, 2048, 4096), seed=0, permuted=False):
    """Config 3: uniform random 16-bit patterns viewed as fp16.  permuted=True
    stores the same logical tensor with strides of a (0,2,1)-permuted buffer."""
    g = gen(seed)
    bits = torch.randint(-32768, 32768, shape, dtype=torch.int16, generator=g)
    if permuted:
        bits = bits.permute(0, 2, 1).contiguous().permute(0, 2, 1)
    return bits.view(torch.float16)


def bmm_inputs(batch=32, m=2048, k=4096, n=4096, seed=0):
    """Config 4: activations N(0,1), weights N(0,0.02)."""
    g = gen(seed)
    a = torch.randn(batch, m, k, generator=g).half()
    b = (torch.randn(batch, k, n, generator=g) * 0.02).half()
    return a, b


def assert_close(actual: torch.Tensor, expected: torch.Tensor, rtol=RTOL, atol=ATOL):
    torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), rtol=rtol, atol=atol)


def errors_against_fp32(got: torch.Tensor, cpu_fp16: torch.Tensor, truth_fp32: torch.Tensor,
                        rtol=RTOL, atol=ATOL) -> dict:
    """How far a device result and the CPU fp16 eager result each are from an fp32 evaluation of
    the same inputs: maximum and RMS error of both, and the share of device elements that meet
    rtol / atol against the CPU fp16 result.  Used where a chain of fp16 ops is deep enough that
    two correct evaluations differ by more than atol element by element."""
    t = truth_fp32.float().cpu()
    eg = (got.float().cpu() - t).abs()
    ec = (cpu_fp16.float().cpu() - t).abs()
    d = (got.float().cpu() - cpu_fp16.float().cpu()).abs()
    inside = d <= atol + rtol * cpu_fp16.float().cpu().abs()
    return {"gpu_max": float(eg.max()), "cpu_max": float(ec.max()),
            "gpu_rms": float(eg.pow(2).mean().sqrt()), "cpu_rms": float(ec.pow(2).mean().sqrt()),
            "frac_within_tol": float(inside.float().mean())}


def assert_no_worse_than_cpu_fp16(got, cpu_fp16, truth_fp32, factor=1.5, what="result") -> dict:
    """The device result may be at most `factor` times as far from the fp32 evaluation as torch
    CPU fp16 eager is, in maximum and in RMS error."""
    e = errors_against_fp32(got, cpu_fp16, truth_fp32)
    if not torch.isfinite(got.float()).all():
        raise AssertionError(f"{what}: non-finite values in the device result")
    if e["gpu_max"] > factor * e["cpu_max"] + 1e-6 or e["gpu_rms"] > factor * e["cpu_rms"] + 1e-7:
        raise AssertionError(f"{what}: device error against fp32 (max {e['gpu_max']:.3e}, rms "
                             f"{e['gpu_rms']:.3e}) exceeds {factor} x CPU fp16 eager's (max "
                             f"{e['cpu_max']:.3e}, rms {e['cpu_rms']:.3e})")
    return e
