"""CPU tests: the oracles against the reference's golden vectors and each other."""
import json
import os

import numpy as np
import pytest

from oracle import layout as L
from oracle import relayout_c as C

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _ref_vectors():
    with open(os.path.join(GOLD, "layout_reference_vectors.json")) as f:
        return json.load(f)


def test_layout_matches_reference_vectors():
    for v in _ref_vectors()["layouts"]:
        lay = L.generic_stick_layout(v["host_size"], 2, v["dim_order"])
        assert lay.device_size == v["device_size"]
        assert lay.device_strides == v["device_strides"]
        assert lay.dim_map == v["dim_map"]
        assert lay.num_stick_dims == 1 and lay.format == L.DENSE


def test_layout_str_matches_reference():
    v = _ref_vectors()["str"]
    assert str(L.generic_stick_layout(v["host_size"])) == v["text"]


def test_storage_nbytes_matches_reference():
    for v in _ref_vectors()["storage_nbytes"]:
        assert L.storage_nbytes(v["host_size"], 2) == v["nbytes"]
    assert L.storage_nbytes([], 2) == 128  # 0-dim is laid out as [1]


def test_dense_strides_agree_with_reference_python_twin():
    with open(os.path.join(GOLD, "dci_strides.json")) as f:
        gold = json.load(f)
    assert gold["elems_per_stick_fp16"] == L.BYTES_IN_STICK // 2
    for c in gold["cases"]:
        if c["format"] != "DENSE":
            continue
        # The reference's logical strides for a dim order are the strides of the
        # host-contiguous tensor in that order; the device layout must visit the
        # non-stick dims in the same order, stick dim last.
        lay = L.generic_stick_layout(c["size"], 2, c["dim_order"])
        assert lay.dim_map[-1] == c["stick_dims"][0] == lay.dim_map[0]
        assert lay.dim_map[1:-1] == c["dim_order"][:-1]
        order = sorted(range(len(c["size"])), key=lambda d: -c["strides"][d])
        sized = [d for d in order if c["size"][d] > 1]
        assert sized == [d for d in c["dim_order"] if c["size"][d] > 1]


SHAPES = [(128,), (3,), (1,), (512, 256), (5, 70), (4, 8, 256), (3, 5, 67), (2, 6, 3, 128),
          (2, 3, 4, 65), (0, 64), (3, 0)]


@pytest.mark.parametrize("shape", SHAPES)
def test_numpy_and_c_oracles_agree(shape):
    rng = np.random.default_rng(1)
    base = rng.integers(0, 65536, size=shape, dtype=np.uint16)
    rank = len(shape)
    perms = [tuple(range(rank)), tuple(reversed(range(rank)))]
    for perm in perms:
        host = np.ascontiguousarray(base.transpose(perm)).transpose(np.argsort(perm))
        assert host.shape == tuple(shape)
        layouts = [L.generic_stick_layout(shape)]
        if rank <= 4:
            layouts.append(L.legacy_copy_layout(shape))
        if rank >= 2:
            layouts.append(L.generic_stick_layout(shape, 2, list(reversed(range(rank)))))
        for lay in layouts:
            a = L.to_sticks(host, lay)
            if host.size:
                b = C.to_sticks(host, lay, nthreads=3)
                assert np.array_equal(a, b)
                assert np.array_equal(C.from_sticks(b, lay, shape, nthreads=2), host)
            assert np.array_equal(L.from_sticks(a, lay, shape), host)
        if host.size:
            fast = L.to_sticks_generic_fast(host)
            assert np.array_equal(fast, L.to_sticks(host, layouts[0]))
            assert np.array_equal(L.from_sticks_generic_fast(fast, shape), host)


def test_pad_lanes_are_zero():
    host = np.full((3, 70), 0xFFFF, dtype=np.uint16)
    lay = L.generic_stick_layout(host.shape)
    img = C.to_sticks(host, lay).reshape(lay.device_size)
    assert (img[1, :, 6:] == 0).all() and (img[1, :, :6] == 0xFFFF).all() and (img[0] == 0xFFFF).all()


def test_golden_images_reproduce():
    z = np.load(os.path.join(GOLD, "relayout_images.npz"))
    names = sorted(k[:-5] for k in z.files if k.endswith("_host"))
    assert names
    for n in names:
        host = z[n + "_host"]
        assert np.array_equal(C.to_sticks(host, L.generic_stick_layout(host.shape)), z[n + "_generic"])
        assert np.array_equal(C.to_sticks(host, L.legacy_copy_layout(host.shape)), z[n + "_legacy"])


def test_other_element_sizes():
    rng = np.random.default_rng(2)
    for dt, eb in ((np.uint8, 1), (np.uint32, 4)):
        host = rng.integers(0, 255, size=(3, 200)).astype(dt)
        lay = L.generic_stick_layout(host.shape, eb)
        assert lay.device_size[-1] == 128 // eb
        img = C.to_sticks(host, lay)
        assert np.array_equal(img, L.to_sticks(host, lay))
        assert np.array_equal(C.from_sticks(img, lay, host.shape), host)
