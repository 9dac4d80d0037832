"""GPU parity: tcgen05 matmul / bmm against torch CPU eager (rtol 1e-2, atol 1e-3)."""
import pytest
import torch

from oracle import math_ref
from oracle.math_ref import assert_close
from torch_spyre import _abi, stick_ops as K

pytestmark = pytest.mark.gpu


def up(t, cuda):
    return K.to_sticks(t.to(cuda))


def down(st):
    return K.from_sticks(st).cpu()


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).half()


def no_kernel_timeout():
    assert _abi.lib().ts_gemm_error_state() == 0, "a GEMM kernel gave up on an internal wait"


MM_SHAPES = [(128, 64, 256), (128, 128, 256), (3, 5, 7), (67, 256, 128), (256, 128, 512),
             (130, 70, 300), (1, 64, 64), (512, 1024, 768), (1000, 4096, 520),
             # more 256x256 tiles than CTA pairs, and a last band of tile columns narrower than 8
             (2304, 192, 2304 + 64)]


@pytest.mark.parametrize("m,k,n", MM_SHAPES)
def test_mm(m, k, n, cuda):
    a, b = rnd(m, k, seed=1), rnd(k, n, seed=2, scale=0.05)
    c = K.matmul(up(a, cuda), up(b, cuda))
    torch.cuda.synchronize()
    no_kernel_timeout()
    assert_close(down(c), a @ b)
    if n % 64:
        img = c.image.cpu().view(-1, m, 64)
        assert (img[-1, :, n % 64:] == 0).all()


@pytest.mark.parametrize("m,k,n", MM_SHAPES)
def test_linear_weight_layout(m, k, n, cuda):
    """a @ w.T with w stored [N, K]; bias fused into the epilogue."""
    a, w, bias = rnd(m, k, seed=1), rnd(n, k, seed=2, scale=0.05), rnd(n, seed=3)
    c = K.matmul(up(a, cuda), up(w, cuda), bias=up(bias, cuda), b_kmajor=True)
    torch.cuda.synchronize()
    no_kernel_timeout()
    assert_close(down(c), torch.nn.functional.linear(a, w, bias))


@pytest.mark.parametrize("bsz,m,k,n", [(1, 128, 64, 256), (4, 200, 192, 320), (3, 67, 256, 128),
                                       (2, 3, 5, 7), (5, 256, 512, 256)])
def test_bmm(bsz, m, k, n, cuda):
    a, b = rnd(bsz, m, k, seed=1), rnd(bsz, k, n, seed=2, scale=0.05)
    c = K.matmul(up(a, cuda), up(b, cuda))
    torch.cuda.synchronize()
    no_kernel_timeout()
    assert_close(down(c), torch.bmm(a, b))
    # batched a, shared b; batched a, batched transposed b
    c2 = K.matmul(up(a, cuda), up(b[0], cuda))
    assert_close(down(c2), a @ b[0])
    bt = b.transpose(1, 2).contiguous()
    c3 = K.matmul(up(a, cuda), up(bt, cuda), b_kmajor=True)
    assert_close(down(c3), torch.bmm(a, b))
    no_kernel_timeout()


def test_attention_building_block(cuda):
    # tests/_inductor/test_building_blocks.py:67-89 of the reference
    q, k, v = rnd(256, 128, seed=1), rnd(256, 128, seed=2), rnd(256, 128, seed=3)
    scale = 128 ** -0.5
    sq, sk, sv = up(q, cuda), up(k, cuda), up(v, cuda)
    s = K.matmul(sq, sk, b_kmajor=True)           # q @ k^T
    c = K.Chain()
    c.emit("LOAD", c.tensor(s)).emit("MUL", c.imm(scale)).store(0)
    (s,), _ = K.run_chain(c, s.shape)
    p = K.softmax(s, -1)
    o = K.matmul(p, sv)
    want = torch.softmax((q @ k.t()) * scale, -1) @ v
    assert_close(down(o), want)
    no_kernel_timeout()


def test_config4_slice(cuda):
    """Two batch entries of the [32,2048,4096] x [32,4096,4096] benchmark bmm."""
    a, b = math_ref.bmm_inputs(batch=2)
    c = K.matmul(up(a, cuda), up(b, cuda))
    torch.cuda.synchronize()
    no_kernel_timeout()
    want = torch.bmm(a[:1, :512], b[:1])          # CPU time: check a slab of rows exactly
    assert_close(down(c)[:1, :512], want)
    # and the rest against an fp32 GPU matmul of the same fp16 inputs
    ref = torch.bmm(a.to(cuda).float(), b.to(cuda).float()).half().cpu()
    assert_close(down(c), ref)


def test_linearity_property_full_width(cuda):
    """(a1 + a2) @ b == a1 @ b + a2 @ b up to rounding, at K = 4096."""
    a1, a2 = rnd(256, 4096, seed=1), rnd(256, 4096, seed=2)
    b = rnd(4096, 512, seed=3, scale=0.02)
    sb = up(b, cuda)
    lhs = down(K.matmul(up((a1 + a2), cuda), sb)).float()
    rhs = down(K.matmul(up(a1, cuda), sb)).float() + down(K.matmul(up(a2, cuda), sb)).float()
    torch.testing.assert_close(lhs, rhs, rtol=2e-2, atol=2e-2)
    no_kernel_timeout()


@pytest.mark.parametrize("m,k,n", [(128, 64, 256), (130, 70, 300), (512, 1024, 768), (67, 256, 128)])
def test_residual_in_epilogue(m, k, n, cuda):
    """c = fp16(a @ w.T + bias) + residual, bit for bit what a separate fp16 add would give."""
    a, w, bias, res = rnd(m, k, seed=1), rnd(n, k, seed=2, scale=0.05), rnd(n, seed=3), rnd(m, n, seed=4)
    fused = K.matmul(up(a, cuda), up(w, cuda), bias=up(bias, cuda), b_kmajor=True, residual=up(res, cuda))
    plain = K.matmul(up(a, cuda), up(w, cuda), bias=up(bias, cuda), b_kmajor=True)
    torch.cuda.synchronize()
    no_kernel_timeout()
    assert torch.equal(down(fused), down(plain) + res)
    assert_close(down(fused), (a.float() @ w.float().t() + bias.float()).half() + res)


@pytest.mark.parametrize("m,k,n", [(128, 64, 128), (130, 70, 320), (512, 256, 704), (67, 128, 64)])
def test_swiglu_gemm(m, k, n, cuda):
    """silu(a @ wg.T) * (a @ wu.T) as one GEMM over the interleaved weight, against the unfused
    device sequence and the CPU formula."""
    import torch.nn.functional as F
    from torch_spyre._inductor.customops import interleave_gate_up

    a, wg, wu = rnd(m, k, seed=1), rnd(n, k, seed=2, scale=0.1), rnd(n, k, seed=3, scale=0.1)
    fused = down(K.swiglu_matmul(up(a, cuda), up(interleave_gate_up(wg, wu), cuda)))
    torch.cuda.synchronize()
    no_kernel_timeout()
    gate = down(K.matmul(up(a, cuda), up(wg, cuda), b_kmajor=True))
    upp = down(K.matmul(up(a, cuda), up(wu, cuda), b_kmajor=True))
    assert_close(fused, F.silu(gate) * upp)
    assert_close(fused, F.silu(F.linear(a, wg)) * F.linear(a, wu))


def test_a_wait_that_gives_up_reports_and_leaves_the_device_usable(cuda):
    """The bounded waits' give-up path, driven without a fault: a warp waits a few thousand cycles
    on a barrier nothing arrives on, the kernel returns, the sticky status reads 1 then 0, and the
    next GEMM is correct."""
    lib = _abi.lib()
    assert lib.ts_gemm_error_state() == 0
    assert lib.ts_gemm_wait_selftest(5000, None) == 0
    torch.cuda.synchronize()
    assert lib.ts_gemm_error_state() == 1
    assert lib.ts_gemm_error_state() == 0
    g = torch.Generator().manual_seed(21)
    a, b = torch.randn(300, 256, generator=g).half(), (torch.randn(256, 192, generator=g) * 0.1).half()
    got = K.from_sticks(K.matmul(K.to_sticks(a.to(cuda)), K.to_sticks(b.to(cuda)))).cpu()
    assert_close(got, a @ b)
    assert lib.ts_gemm_error_state() == 0


@pytest.mark.parametrize("owners,m,k,n", [(2, 512, 256, 320), (4, 1024, 512, 256), (8, 2048, 384, 1024), (1, 256, 128, 128)])
def test_scatter_add_epilogue_on_one_gpu(owners, m, k, n, cuda):
    """The reduce-scatter epilogue with every owner's buffer on this GPU: two "ranks", each holding
    half of K, add their partial products into the owners' buffers, which start out holding a
    residual.  Result: residual + a @ w^T, block of rows by block of rows."""
    g = torch.Generator().manual_seed(31)
    a = torch.randn(m, 2 * k, generator=g).half()
    w = (torch.randn(n, 2 * k, generator=g) * 0.05).half()
    res = torch.randn(m, n, generator=g).half()
    rows = m // owners
    outs = [up(res[r * rows:(r + 1) * rows].contiguous(), cuda) for r in range(owners)]
    ptrs = [o.ptr() for o in outs]
    for half in range(2):      # the two ranks' launches, one after the other on this stream
        sa = up(a[:, half * k:(half + 1) * k].contiguous(), cuda)
        sw = up(w[:, half * k:(half + 1) * k].contiguous(), cuda)
        K.matmul_scatter_add(sa, sw, ptrs, b_kmajor=True)
    torch.cuda.synchronize()
    no_kernel_timeout()
    got = torch.cat([down(o) for o in outs], 0)
    want = (res.float() + a.float() @ w.float().t()).half()
    assert_close(got, want, atol=4e-3)       # three fp16 roundings (residual + two partial sums) instead of one
    lib = _abi.lib()
    p = outs[0].ptr()
    assert lib.ts_gemm_f16_scatter_add(p, p, _abi.ptrs([p]), 1, 48, 64, 64, 1, None) == _abi.TS_ERR_UNSUPPORTED   # rows % 32
    assert lib.ts_gemm_f16_scatter_add(p, p, _abi.ptrs([p] * 9), 9, 288, 64, 64, 1, None) == _abi.TS_ERR_INVALID
    assert lib.ts_gemm_f16_scatter_add(p, p, _abi.ptrs([0]), 1, 64, 64, 64, 1, None) == _abi.TS_ERR_ALIGNMENT


@pytest.mark.parametrize("owners,m,k,n,ranks", [(2, 512, 256, 320, 2), (4, 1024, 512, 256, 2), (8, 2048, 384, 1024, 2),
                                                  (1, 256, 128, 128, 2), (8, 2048, 128, 512, 8), (4, 512, 64, 192, 4)])
def test_scatter_store_epilogue_and_slot_sum_on_one_gpu(owners, m, k, n, ranks, cuda):
    """The reduce-scatter with plain stores, every owner's slots on this GPU: `ranks` "ranks", each
    holding a slice of K, store their partial products into their own slot of each owner's buffer;
    the owners then add their slots and the residual in fp32.  One rounding after the sum: the
    result meets the default tolerance where the reduction form needs a looser one."""
    g = torch.Generator().manual_seed(32)
    a = torch.randn(m, ranks * k, generator=g).half()
    w = (torch.randn(n, ranks * k, generator=g) * 0.05).half()
    res = torch.randn(m, n, generator=g).half()
    rows = m // owners
    slot = -(-n // 64) * rows * 64                       # elements of one [rows, n] image
    bufs = [torch.full((ranks * slot,), float("nan"), dtype=torch.float16, device=cuda) for _ in range(owners)]
    for rank in range(ranks):     # the ranks' launches, one after the other on this stream
        sa = up(a[:, rank * k:(rank + 1) * k].contiguous(), cuda)
        sw = up(w[:, rank * k:(rank + 1) * k].contiguous(), cuda)
        K.matmul_scatter_store(sa, sw, [b.data_ptr() + rank * slot * 2 for b in bufs], b_kmajor=True)
    outs = [K.sum_slots(bufs[r], ranks, (rows, n), up(res[r * rows:(r + 1) * rows].contiguous(), cuda))
            for r in range(owners)]
    torch.cuda.synchronize()
    no_kernel_timeout()
    got = torch.cat([down(o) for o in outs], 0)
    partial = [(a[:, r * k:(r + 1) * k].float() @ w[:, r * k:(r + 1) * k].float().t()).half().float() for r in range(ranks)]
    total = sum(partial)
    want = (res.float() + total).half()
    assert_close(got, want)
    # without a residual
    plain = K.sum_slots(bufs[0], ranks, (rows, n))
    assert_close(down(plain), total[:rows].half())
    lib = _abi.lib()
    p = bufs[0].data_ptr()
    assert lib.ts_sum_slots_f16(p, 0, slot, None, p, slot, None) == _abi.TS_ERR_INVALID
    assert lib.ts_sum_slots_f16(p, 2, slot, None, p + 2, slot, None) == _abi.TS_ERR_ALIGNMENT
    assert lib.ts_sum_slots_f16(p, 2, slot, None, p, 12, None) == _abi.TS_ERR_UNSUPPORTED
    assert lib.ts_gemm_f16_scatter_store(p, p, _abi.ptrs([p]), 1, 48, 64, 64, 1, None) == _abi.TS_ERR_UNSUPPORTED
