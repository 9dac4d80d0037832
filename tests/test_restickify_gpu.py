"""GPU parity of the one-pass device restickify (ts_transpose_tiles): stick image -> stick image
for transposed, permuted, sliced, narrowed and expanded views, bit for bit against the CPU
oracle (numpy view of the logical base, then the oracle's image of the result), through the C
ABI and through the `spyre` device.  The transposes are the ones the reference's own tests name
(tests/_inductor/test_inductor_ops.py:198-218: (1088, 320) 2-D, (512, 256, 128) dims (0,2) and
(1,2))."""
import numpy as np
import pytest
import torch

from oracle import layout as L
from oracle import relayout_c as C
from torch_spyre import _abi

pytestmark = pytest.mark.gpu


def _bits(shape, seed=0, dtype=np.uint16):
    rng = np.random.default_rng(seed)
    info = np.iinfo(dtype)
    return rng.integers(0, int(info.max) + 1, size=shape, dtype=np.uint64).astype(dtype)


def _image(host: np.ndarray) -> np.ndarray:
    lay = L.generic_stick_layout(host.shape, host.dtype.itemsize)
    return C.to_sticks(np.ascontiguousarray(host), lay)


def _cuda(a: np.ndarray) -> torch.Tensor:
    view = {2: np.int16, 1: np.int8, 4: np.int32}[a.dtype.itemsize]
    return torch.from_numpy(a.view(view).copy()).cuda()


def _call(src_img, src_base, sstr, soff, dst_img, dst_base, dstr, doff, size, eb):
    i64 = _abi.i64
    rc = _abi.lib().ts_transpose_tiles(src_img.data_ptr(), i64(src_base), len(src_base), i64(sstr), soff,
                                       dst_img.data_ptr(), i64(dst_base), len(dst_base), i64(dstr), doff,
                                       i64(size), len(size), eb, None)
    torch.cuda.synchronize()
    return rc


def _elem_strides(a: np.ndarray):
    return [s // a.dtype.itemsize for s in a.strides]


def _offset(view: np.ndarray, base: np.ndarray) -> int:
    return (view.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // base.dtype.itemsize


def check_view_to_canonical(base: np.ndarray, view: np.ndarray, expect_rc=0):
    """src = image of `base`, viewed as `view` (a numpy view of base); dst = canonical image."""
    eb = base.dtype.itemsize
    src_img = _cuda(_image(base))
    want = _image(np.ascontiguousarray(view))
    dst_img = torch.full((want.size,), 0x55, dtype=src_img.dtype, device="cuda")   # garbage: pads must be zeroed
    size = list(view.shape)
    dstr = _elem_strides(np.empty(view.shape, dtype=base.dtype))
    rc = _call(src_img, list(base.shape), _elem_strides(view), _offset(view, base), dst_img, size, dstr, 0,
               size, eb)
    assert rc == expect_rc, rc
    if rc == 0:
        got = dst_img.cpu().numpy().view(base.dtype)
        assert np.array_equal(got, want), "restickified image differs from the oracle"


def test_reference_transposes_2d_and_3d():
    b = _bits((1088, 320))
    check_view_to_canonical(b, b.T)
    b = _bits((512, 256, 128), 1)
    check_view_to_canonical(b, b.transpose(2, 1, 0))    # dims (0, 2)
    check_view_to_canonical(b, b.transpose(0, 2, 1))    # dims (1, 2)
    check_view_to_canonical(b, b.transpose(1, 0, 2))    # outer dims only: no tile transpose needed


@pytest.mark.parametrize("shape,perm", [((67, 130), (1, 0)), ((3, 70, 65), (0, 2, 1)), ((5, 64, 64), (2, 1, 0)),
                                        ((2, 3, 100, 40), (0, 3, 2, 1)), ((130, 1), (1, 0)), ((1, 200), (1, 0)),
                                        ((16, 16), (1, 0)), ((2, 2048, 320), (0, 2, 1))])
def test_padded_and_odd_transposes(shape, perm):
    b = _bits(shape, 2)
    check_view_to_canonical(b, b.transpose(perm))


def test_slices_narrows_selects_and_expands():
    b = _bits((6, 40, 200), 3)
    check_view_to_canonical(b, b[1:5])                       # outer slice
    check_view_to_canonical(b, b[:, 3:30:2])                 # stepped middle slice
    check_view_to_canonical(b, b[:, :, 64:192])              # stick-aligned slice of the stick dim
    check_view_to_canonical(b, b[:, :, 128:])                # to the (padded) end
    check_view_to_canonical(b, b[:, :, 70:100])              # inside one stick
    check_view_to_canonical(b, b[2])                         # select
    check_view_to_canonical(b, b[:, :, 5])                   # select on the stick dim
    check_view_to_canonical(b, b[:, 7, 64:128].T)            # slice + transpose
    row = _bits((1, 40, 200), 4)
    check_view_to_canonical(row, np.broadcast_to(row, (6, 40, 200)))    # expand (stride 0 in the source)
    col = _bits((130, 1), 5)
    check_view_to_canonical(col, np.broadcast_to(col, (130, 70)))       # expand along the stick dim's place


@pytest.mark.parametrize("dtype", [np.uint8, np.uint32])
def test_other_element_sizes(dtype):
    b = _bits((5, 40, 300), 6, dtype)
    check_view_to_canonical(b, b.transpose(1, 0, 2))
    check_view_to_canonical(b, b[:, 2:9])
    check_view_to_canonical(b, b.transpose(0, 2, 1))         # element by element for these sizes


def test_views_the_kernel_cannot_walk_are_refused():
    b = _bits((8, 200), 7)
    check_view_to_canonical(b, b[:, 3:100], expect_rc=_abi.TS_ERR_UNSUPPORTED)     # crosses sticks, unaligned
    check_view_to_canonical(b, b[:, ::2], expect_rc=_abi.TS_ERR_UNSUPPORTED)       # stepped along the stick dim
    flat = _bits((64,), 8)
    diag = np.lib.stride_tricks.as_strided(flat, shape=(7,), strides=(18,))          # 9 elements apart
    check_view_to_canonical(flat, diag)                                              # one base dim, step 9: fine
    sq = _bits((8, 8), 9)
    d2 = np.lib.stride_tricks.as_strided(sq, shape=(8,), strides=(18,))              # the diagonal: two dims at once
    check_view_to_canonical(sq, d2, expect_rc=_abi.TS_ERR_UNSUPPORTED)
    # null pointers and bad ranks
    lib = _abi.lib()
    one = _abi.i64([4])
    assert lib.ts_transpose_tiles(None, one, 1, one, 0, None, one, 1, one, 0, one, 1, 2, None) == _abi.TS_ERR_INVALID
    buf = torch.zeros(256, dtype=torch.int16, device="cuda")
    assert lib.ts_transpose_tiles(buf.data_ptr(), one, 1, _abi.i64([1]), 0, buf.data_ptr(), one, 1, _abi.i64([1]), 0,
                                  one, 1, 3, None) == _abi.TS_ERR_INVALID
    assert lib.ts_transpose_tiles(buf.data_ptr(), one, 1, _abi.i64([0]), 0, buf.data_ptr(), one, 1, _abi.i64([0]), 0,
                                  one, 1, 2, None) == _abi.TS_ERR_UNSUPPORTED      # zero stride in the destination


def test_writing_into_a_slice_of_the_destination():
    """What a one-pass cat does: each input's image goes straight into its slice of the result."""
    out = _bits((4, 300, 200), 10)                 # existing contents of the destination
    a, b = _bits((4, 100, 200), 11), _bits((4, 200, 200), 12)
    dst = _cuda(_image(out))
    for piece, lo in ((a, 0), (b, 100)):
        view = out[:, lo:lo + piece.shape[1]]
        rc = _call(_cuda(_image(piece)), list(piece.shape), _elem_strides(piece), 0, dst, list(out.shape),
                   _elem_strides(view), _offset(view, out), list(piece.shape), 2)
        assert rc == 0
        view[...] = piece
    assert np.array_equal(dst.cpu().numpy().view(np.uint16), _image(out))
    # along the stick dim: the first piece ends on a stick boundary, the second reaches the padded end
    out2 = _bits((3, 50, 200), 13)
    p0, p1 = _bits((3, 50, 128), 14), _bits((3, 50, 72), 15)
    dst2 = torch.full((_image(out2).size,), 0x33, dtype=torch.int16, device="cuda")
    for piece, lo in ((p0, 0), (p1, 128)):
        view = out2[:, :, lo:lo + piece.shape[2]]
        rc = _call(_cuda(_image(piece)), list(piece.shape), _elem_strides(piece), 0, dst2, list(out2.shape),
                   _elem_strides(view), _offset(view, out2), list(piece.shape), 2)
        assert rc == 0
        view[...] = piece
    assert np.array_equal(dst2.cpu().numpy().view(np.uint16), _image(out2))


def test_device_views_take_the_one_pass_route_and_agree_with_the_two_pass_route():
    import torch_spyre  # noqa: F401
    from torch_spyre import _C

    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 130, 200, generator=g).half()
    xs = x.to("spyre")
    cases = [lambda t: t.transpose(1, 2), lambda t: t.permute(2, 0, 1), lambda t: t[1:4, :, 64:],
             lambda t: t[:, 5], lambda t: t[..., 3:100], lambda t: t.transpose(0, 2)[10:70],
             lambda t: t[:1].expand(6, 130, 200)]
    for f in cases:
        want = f(x).contiguous()
        got = f(xs).contiguous().cpu()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        _C.set_restickify_enabled(False)
        try:
            slow = f(xs).contiguous().cpu()
        finally:
            _C.set_restickify_enabled(True)
        assert torch.equal(slow.view(torch.int16), want.view(torch.int16))
    # a copy into a view of the destination, and cat along every dim
    ys = torch.zeros(6, 130, 200, dtype=torch.float16).to("spyre")
    ys[:, 10:40] = xs[:, 50:80]
    ref = torch.zeros(6, 130, 200, dtype=torch.float16)
    ref[:, 10:40] = x[:, 50:80]
    assert torch.equal(ys.cpu(), ref)
    for dim in (0, 1, 2):
        parts = [x, x * 2, x + 1]
        got = torch.cat([p.to("spyre") for p in parts], dim).cpu()
        assert torch.equal(got, torch.cat(parts, dim))
    w = torch.randn(6, 130, 128, generator=g).half()
    assert torch.equal(torch.cat([w.to("spyre"), xs], 2).cpu(), torch.cat([w, x], 2))   # stick-aligned: one pass


def test_full_size_transpose_round_trip():
    """(2048, 4096) per batch entry, the benchmark's permuted case on the device side: transposing
    twice is the identity and the image equals the closed form."""
    import torch_spyre  # noqa: F401

    bits = torch.randint(-32768, 32768, (8, 2048, 4096), dtype=torch.int16,
                         generator=torch.Generator().manual_seed(1))
    x = bits.view(torch.float16)
    xs = x.to("spyre")
    t = xs.transpose(1, 2).contiguous()
    assert torch.equal(t.cpu().view(torch.int16), bits.transpose(1, 2).contiguous())
    back = t.transpose(1, 2).contiguous()
    assert torch.equal(back.cpu().view(torch.int16), bits)
