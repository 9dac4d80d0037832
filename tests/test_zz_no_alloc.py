"""The scratch-free reduction entry point, ts_reduce_mid_static.

It serves callers that cannot allocate device memory themselves (a plug-in handed only
input/output pointers by its host application, or a loop that must not call cudaMalloc
because an allocation may stall the device): its split-reduction partials live in a fixed
512 KiB array inside the library.  The test drives it through the C ABI, twice in a row on
different data (the array is shared and keeps the previous call's contents), and checks
each result against ts_reduce_mid, which uses caller-provided scratch.  The file name keeps
it last in collection order so that a run stopping at the first failure has already run
every other test.
"""
import pytest
import torch

from torch_spyre import _abi, stick_ops as K

pytestmark = pytest.mark.gpu


def _reduce_both(x_host: torch.Tensor, op: str, cuda):
    sx = K.to_sticks(x_host.to(cuda))
    outer, red, inner = K._mid_view(sx.shape, 0)
    lib = _abi.lib()
    need = lib.ts_reduce_mid_scratch_bytes(outer, red, inner)
    assert 0 < need <= lib.ts_reduce_mid_static_max_bytes(), "case must split and fit"
    want = K.reduce_mid(sx, 0, op)                       # existing entry point, own scratch
    got = K.empty(want.shape, torch.float16, cuda)
    rc = lib.ts_reduce_mid_static(sx.ptr(), got.ptr(), outer, red, inner, K.RED[op], 1.0,
                                  torch.cuda.current_stream().cuda_stream)
    _abi.check(rc, "ts_reduce_mid_static")
    torch.cuda.synchronize()
    return K.from_sticks(got).cpu(), K.from_sticks(want).cpu()


def test_static_scratch_matches_on_two_calls_in_a_row(cuda):
    g = torch.Generator().manual_seed(11)
    first = (torch.randn(20000, 64, generator=g) * 0.1).half()
    second = (torch.randn(30000, 128, generator=g) * 0.1 + 0.5).half()   # different size: stale partials must not leak
    for x, op in ((first, "sum"), (second, "sum"), (first, "max")):
        got, want = _reduce_both(x, op, cuda)
        # same kernels, same split, same order of additions: results are identical bit for bit,
        # well inside the rtol 1e-2 / atol 1e-3 the math tests use
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-3)
        assert torch.equal(got, want)
        ref = x.float().sum(0) if op == "sum" else x.float().amax(0)
        torch.testing.assert_close(got.float(), ref, rtol=1e-2, atol=2e-2)


def test_static_scratch_rejects_oversized_requests(cuda):
    lib = _abi.lib()
    outer, red, inner = 1, 1 << 16, 64 * 2048      # 2 splits x 131072 fp32 partials = 1 MiB
    assert lib.ts_reduce_mid_scratch_bytes(outer, red, inner) > lib.ts_reduce_mid_static_max_bytes()
    assert lib.ts_reduce_mid_static(16, 16, outer, red, inner, 1, 1.0, None) == -5
    assert b"exceeds" in lib.ts_status_string(-5)
