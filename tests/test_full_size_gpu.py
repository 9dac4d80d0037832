"""The benchmark configurations at their full sizes, on the device, checked through properties
that do not need a full CPU evaluation (config 3 at full size lives in test_relayout_gpu.py and
test_restickify_gpu.py, config 5 at full width in test_llama_fullwidth_gpu.py):

  config 1  softmax [256, 4096] against CPU eager in full; [65536, 4096]: every row sums to one,
            sampled rows against CPU eager;
  config 2  exp(x*a+b).sum(-1) on [8192, 8192] against CPU eager in full, through torch.compile;
  config 4  bmm [32, 2048, 4096] x [32, 4096, 4096]: sampled elements against float64 dot products,
            and every row of every product against the checksum  A_b[i, :] @ (B_b summed over n).
Tolerances: rtol 1e-2 / atol 1e-3 (tests/test_modules.py:39-40 of the reference) unless stated."""
import pytest
import torch

import torch_spyre  # noqa: F401
from oracle import math_ref
from oracle.math_ref import assert_close
from torch_spyre import _abi

pytestmark = pytest.mark.gpu
DEV = "spyre"


@pytest.fixture(autouse=True)
def _need_gpu(cuda):
    torch._dynamo.reset()
    yield


def test_config1_softmax_full_and_scaled():
    x = math_ref.softmax_inputs()
    assert_close(torch.softmax(x.to(DEV), -1).cpu(), torch.softmax(x, -1))
    big = x.repeat(256, 1)                                   # [65536, 4096], as the bench scales it
    big[1::256] = big[1::256].flip(-1)                       # not every block the same
    got = torch.softmax(big.to(DEV), -1).cpu()
    sums = got.float().sum(-1)
    assert (sums - 1).abs().max() < 2e-2                     # 4096 fp16 roundings of values around 2e-4 each
    rows = torch.randint(0, big.shape[0], (64,), generator=torch.Generator().manual_seed(2))
    assert_close(got[rows], torch.softmax(big[rows], -1))
    assert torch.equal(got.argmax(-1)[rows], torch.softmax(big[rows].float(), -1).argmax(-1))


def test_config2_fused_full_size_through_compile():
    x, a, b = math_ref.fused_inputs()
    f = torch.compile(lambda t, u, v: torch.exp(t * u + v).sum(-1))
    got = f(x.to(DEV), a.to(DEV), b.to(DEV)).cpu()
    want = torch.exp(x * a + b).sum(-1)
    assert got.shape == (8192,)
    assert_close(got, want)


def test_config4_bmm_full_size_properties():
    batch, m, k, n = 32, 2048, 4096, 4096
    g = torch.Generator().manual_seed(0)
    a0 = torch.randn(m, k, generator=g).half()
    b0 = (torch.randn(k, n, generator=g) * 0.02).half()
    # distinct batch entries without generating 1.5 G random numbers: entry e is entry 0 rolled by e
    a = torch.stack([a0.roll(e, 1) for e in range(batch)])
    b = torch.stack([b0.roll(e, 0) for e in range(batch)])
    c = torch.bmm(a.to(DEV), b.to(DEV)).cpu()
    assert _abi.lib().ts_gemm_error_state() == 0
    assert c.shape == (batch, m, n)
    # sampled elements against float64 dot products
    gs = torch.Generator().manual_seed(1)
    e = torch.randint(0, batch, (4000,), generator=gs)
    i = torch.randint(0, m, (4000,), generator=gs)
    j = torch.randint(0, n, (4000,), generator=gs)
    want = (a[e, i].double() * b[e, :, j].double()).sum(-1)
    assert_close(c[e, i, j], want.float())
    # every row of every product: the sum over its n outputs is A_b[i, :] @ (sum over n of B_b).  Each
    # output carries an fp16 rounding (values of std 1.3 => 3e-4 each, 0.02 over 4096 of them).
    colsum = b.double().sum(-1)                              # [batch, k]
    check = torch.einsum("bik,bk->bi", a.double(), colsum)   # [batch, m]
    got = c.double().sum(-1)
    assert (got - check).abs().max() < 0.5
    assert ((got - check).pow(2).mean().sqrt()) < 0.05
