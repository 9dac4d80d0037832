"""GPU parity: the relayout kernels against the CPU oracle, bit for bit, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from oracle import layout as L
from oracle import relayout_c as C
from torch_spyre import _abi, stick_ops as K
from torch_spyre.layout import SpyreTensorLayout

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _as_layout(lay: L.Layout) -> SpyreTensorLayout:
    return SpyreTensorLayout(lay.device_size, lay.device_strides, lay.dim_map, 1, 0)


def _np_to_torch_bits(a: np.ndarray) -> torch.Tensor:
    view = {2: np.int16, 1: np.int8, 4: np.int32}[a.dtype.itemsize]
    return torch.from_numpy(np.ascontiguousarray(a).view(view))


def _strided_cuda(host: np.ndarray, cuda) -> torch.Tensor:
    """CUDA tensor with the same element strides as the numpy array `host`."""
    eb = host.dtype.itemsize
    strides = [s // eb for s in host.strides]
    order = sorted(range(host.ndim), key=lambda d: -strides[d])
    base = np.ascontiguousarray(host.transpose(order))
    t = _np_to_torch_bits(base).to(cuda)
    inv = [order.index(d) for d in range(host.ndim)]
    t = t.permute(inv)
    assert list(t.shape) == list(host.shape)
    return t


def _check(host: np.ndarray, lay: L.Layout, cuda, raw=None):
    if raw is None:
        raw = _strided_cuda(host, cuda)
    st = K.to_sticks(raw, _as_layout(lay))
    torch.cuda.synchronize()
    got = st.image.cpu().numpy().view(host.dtype)
    want = C.to_sticks(host, lay) if host.size else L.to_sticks(host, lay)
    assert np.array_equal(got, want), "to_sticks image differs"
    # back, into a contiguous and into a same-strided destination
    back = K.from_sticks(st, layout=_as_layout(lay))
    assert np.array_equal(back.cpu().numpy().view(host.dtype), host)
    dst = torch.zeros_like(raw)  # preserves strides for dense permutations
    K.from_sticks(st, out=dst, layout=_as_layout(lay))
    assert np.array_equal(dst.cpu().numpy().view(host.dtype), host)


SHAPES = [(1,), (3,), (64,), (100,), (256,), (8, 64), (3, 3), (5, 70), (256, 128), (67, 256),
          (130, 200), (3, 3, 3), (4, 8, 256), (3, 5, 67), (256, 128, 512 // 4), (2, 6, 3, 128),
          (2, 3, 4, 65), (3, 3, 3, 3), (2, 3, 2, 2, 70)]


@pytest.mark.parametrize("shape", SHAPES)
def test_contiguous_and_permuted_hosts(shape, cuda):
    rng = np.random.default_rng(hash(shape) % 1000)
    rank = len(shape)
    base = rng.integers(0, 65536, size=shape, dtype=np.uint16)
    perms = {tuple(range(rank)), tuple(reversed(range(rank)))}
    if rank >= 3:
        perms.add((0, 2, 1) + tuple(range(3, rank)))
        perms.add(tuple(range(rank - 2)) + (rank - 1, rank - 2))
    for perm in perms:
        host = np.ascontiguousarray(base.transpose(perm)).transpose(np.argsort(perm))
        _check(host, L.generic_stick_layout(shape), cuda)
        if rank <= 4:
            _check(host, L.legacy_copy_layout(shape), cuda)
        if rank >= 2:
            _check(host, L.generic_stick_layout(shape, 2, list(reversed(range(rank)))), cuda)


def test_golden_images(cuda):
    z = np.load(os.path.join(GOLD, "relayout_images.npz"))
    for n in sorted(k[:-5] for k in z.files if k.endswith("_host")):
        host = z[n + "_host"]
        raw = _np_to_torch_bits(host).to(cuda)
        st = K.to_sticks(raw)
        assert np.array_equal(st.image.cpu().numpy().view(np.uint16), z[n + "_generic"])
        st2 = K.to_sticks(raw, _as_layout(L.legacy_copy_layout(host.shape)))
        assert np.array_equal(st2.image.cpu().numpy().view(np.uint16), z[n + "_legacy"])


def test_sliced_and_offset_hosts(cuda):
    rng = np.random.default_rng(7)
    big = rng.integers(0, 65536, size=(6, 300), dtype=np.uint16)
    dev = _np_to_torch_bits(big).to(cuda)
    views = [lambda a: a[:, 3:203], lambda a: a[1:5, ::2], lambda a: a[::2, 64:192],
             lambda a: a.T[:100], lambda a: a[:, 8:136]]
    for f in views:
        host, raw = f(big), f(dev)
        assert tuple(raw.stride()) == tuple(s // 2 for s in host.strides)
        _check(host, L.generic_stick_layout(host.shape), cuda, raw=raw)


@pytest.mark.parametrize("dt", [np.uint8, np.uint32])
def test_other_element_sizes(dt, cuda):
    rng = np.random.default_rng(3)
    for shape in [(5, 200), (3, 4, 130), (128, 256)]:
        host = rng.integers(0, 255, size=shape).astype(dt)
        _check(host, L.generic_stick_layout(shape, host.dtype.itemsize), cuda)
        _check(np.ascontiguousarray(host.T).T, L.generic_stick_layout(shape, host.dtype.itemsize), cuda)


def test_pad_lanes_zero_and_destination_untouched_outside(cuda):
    host = np.full((5, 70), 0xFFFF, dtype=np.uint16)
    st = K.to_sticks(_np_to_torch_bits(host).to(cuda))
    img = st.image.cpu().numpy().view(np.uint16).reshape(2, 5, 64)
    assert (img[1, :, 6:] == 0).all() and (img[1, :, :6] == 0xFFFF).all()
    # from_sticks must write only the tensor's elements of a wider destination
    wide = torch.full((5, 80), 0x1234, dtype=torch.int16, device=cuda)
    K.from_sticks(st, out=wide[:, :70])
    w = wide.cpu().numpy().view(np.uint16)
    assert (w[:, 70:] == 0x1234).all() and (w[:, :70] == 0xFFFF).all()


def test_host_buffer_entry_points(cuda):
    g = torch.Generator().manual_seed(5)
    for shape, perm in [((7, 130), None), ((4, 96, 128), (0, 2, 1)), ((3,), None)]:
        bits = torch.randint(-32768, 32768, shape, dtype=torch.int16, generator=g)
        if perm:
            bits = bits.permute(perm).contiguous().permute(perm)
        host = bits.view(torch.float16).pin_memory()
        st = K.copy_host_to_sticks(host)
        want = C.to_sticks(bits.numpy().view(np.uint16), L.generic_stick_layout(shape))
        torch.cuda.synchronize()
        assert np.array_equal(st.image.cpu().numpy().view(np.uint16), want)
        back = torch.empty_like(host).pin_memory() if not perm else torch.empty_strided(
            host.shape, host.stride(), dtype=host.dtype).pin_memory()
        K.copy_sticks_to_host(st, back)
        torch.cuda.synchronize()
        assert torch.equal(back.view(torch.int16), bits)


@pytest.mark.parametrize("shape,perm", [((40, 512, 1024), None), ((37, 300, 1000), None), ((24, 1024, 512), (0, 2, 1)),
                                        ((5, 2048, 4096), None), ((3000, 4100), None)])
def test_pipelined_host_copies_in_chunks(shape, perm, cuda):
    """Tensors large enough to be cut into several chunks (8 MiB, or one leading slice if that
    is larger): image against the oracle, round trip bit for bit, with the small staging block the
    library asks for, from pinned and from pageable host memory, and through the spyre device."""
    g = torch.Generator().manual_seed(6)
    bits = torch.randint(-32768, 32768, shape, dtype=torch.int16, generator=g)
    if perm:
        bits = bits.permute(perm).contiguous().permute(perm)
    host = bits.view(torch.float16)
    strides = host.stride()
    want = C.to_sticks(np.lib.stride_tricks.as_strided(
        bits.numpy().view(np.uint16), shape=host.shape, strides=[s * 2 for s in strides]),
        L.generic_stick_layout(tuple(host.shape)), nthreads=8)
    need = int(_abi.lib().ts_copy_staging_bytes(2, _abi.i64(tuple(host.shape)), _abi.i64(strides), host.dim()))
    assert 0 < need <= max(2 * 8 << 20, 2 * (host[0].numel() * 2 + 255)) and need < host.numel() * 2
    for src in (host.pin_memory() if not perm else torch.empty_strided(host.shape, strides, dtype=host.dtype)
                .pin_memory().copy_(host), host):
        st = K.copy_host_to_sticks(src)
        torch.cuda.synchronize()
        assert np.array_equal(st.image.cpu().numpy().view(np.uint16), want)
        back = torch.empty_strided(host.shape, strides, dtype=host.dtype)
        back = back.pin_memory() if src.is_pinned() else back
        K.copy_sticks_to_host(st, back)
        torch.cuda.synchronize()
        assert torch.equal(back.view(torch.int16), bits)
    import torch_spyre  # noqa: F401
    xs = host.to("spyre")
    assert torch.equal(xs.cpu().view(torch.int16), bits)
    assert _abi.lib().ts_copy_host_to_sticks_pipelined(None, None, 0, None, 2, _abi.i64([4, 4]), _abi.i64([4, 1]), 2,
                                                       _abi.i64([1, 4, 64]), _abi.i64([256, 64, 1]),
                                                       _abi.i32([1, 0, 1]), 3, None) == _abi.TS_ERR_INVALID


def test_scalar_becomes_one_element(cuda):
    t = torch.tensor(3.5, dtype=torch.float16, device=cuda)
    st = K.to_sticks(t)
    assert st.shape == (1,) and st.image.numel() == 64
    assert K.from_sticks(st).item() == 3.5


@pytest.mark.parametrize("permuted", [False, True])
def test_config3_slice_full_inner_dims(permuted, cuda):
    """A [4, 2048, 4096] slice of the benchmark tensor against the C oracle."""
    from oracle import math_ref
    host = math_ref.relayout_inputs((4, 2048, 4096), seed=0, permuted=permuted)
    raw = host.to(cuda)
    assert raw.stride() == host.stride()
    st = K.to_sticks(raw)
    lay = L.generic_stick_layout(host.shape)
    want = C.to_sticks(host.view(torch.int16).numpy().view(np.uint16), lay, nthreads=8)
    got = st.image.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, want)
    back = torch.empty_strided(host.shape, host.stride(), dtype=host.dtype, device=cuda)
    K.from_sticks(st, out=back)
    assert torch.equal(back.view(torch.int16).cpu(), host.view(torch.int16))


@pytest.mark.parametrize("permuted", [False, True])
def test_config3_full_size_properties(permuted, cuda):
    """Full [64, 2048, 4096]: round trip is the identity, the image is a permutation of the
    input (same multiset checksum), and it equals the reshape/movedim form of the layout."""
    g = torch.Generator(device=cuda).manual_seed(0)
    shape = (64, 2048, 4096)
    if permuted:
        raw = torch.randint(-32768, 32768, (64, 4096, 2048), dtype=torch.int16, device=cuda,
                            generator=g).permute(0, 2, 1)
    else:
        raw = torch.randint(-32768, 32768, shape, dtype=torch.int16, device=cuda, generator=g)
    st = K.to_sticks(raw)
    img = st.image.view(torch.int16)
    assert img.numel() == 64 * 64 * 2048 * 64
    # closed form of the generic layout with no padding
    expect = raw.reshape(64, 2048, 64, 64).permute(2, 0, 1, 3)
    for s in (0, 17, 63):
        assert torch.equal(img.view(64, 64, 2048, 64)[s], expect[s])
    assert int(img.to(torch.int64).sum()) == int(raw.to(torch.int64).sum())
    back = torch.empty_strided(raw.shape, raw.stride(), dtype=torch.int16, device=cuda)
    K.from_sticks(st, out=back)
    assert torch.equal(back, raw)
