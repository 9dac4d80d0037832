"""CPU tests of the `spyre` device plumbing that need no GPU: backend name, device module,
the pybind SpyreTensorLayout against the reference's golden vectors."""
import json
import os

import torch

import torch_spyre  # noqa: F401  (registers the backend)
from torch_spyre._C import SpyreTensorLayout

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_backend_is_renamed():
    # tests/test_spyre.py:26-27 and tests/tensor/test_tensor_layout.py:24-25 of the reference
    assert torch._C._get_privateuse1_backend_name() == "spyre"
    assert hasattr(torch, "spyre")
    for fn in ("is_available", "device_count", "current_device", "set_device", "manual_seed",
               "manual_seed_all", "_is_in_bad_fork", "_is_compiled"):
        assert hasattr(torch.spyre, fn), fn
    assert torch.spyre._is_compiled() is True
    assert torch.spyre._is_in_bad_fork() is False


def test_pybind_layout_reference_vectors():
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


def test_pybind_layout_explicit_and_sparse():
    x = SpyreTensorLayout([512, 256], torch.float16)
    y = SpyreTensorLayout([4, 512, 64], [32768, 64, 1], [1, 0, 1], 1, SpyreTensorLayout.StickFormat.Dense)
    assert (x.format, x.num_stick_dims, x.dim_map, x.device_strides, x.device_size) == \
        (y.format, y.num_stick_dims, y.dim_map, y.device_strides, y.device_size)
    s = SpyreTensorLayout([4, 512, 64], [32768, 64, 1], [1, 0, 1], 1, SpyreTensorLayout.StickFormat.Sparse)
    assert s.format == SpyreTensorLayout.StickFormat.Sparse
    x.device_size = [1, 2, 64]          # fields are read/write, as in the reference binding
    assert x.device_size == [1, 2, 64]


def test_python_and_pybind_layouts_agree():
    from torch_spyre.layout import SpyreTensorLayout as PyLayout
    for shape, order in [([128], None), ([5, 70], None), ([3, 4, 130], [2, 0, 1]), ([2, 3, 4, 65], None)]:
        a = PyLayout(shape, torch.float16, *([order] if order else []))
        b = SpyreTensorLayout(shape, torch.float16, *([order] if order else []))
        assert str(a) == str(b)


def test_eager_ops_are_registered():
    from torch_spyre import ops
    names = set(ops.registered_ops())
    for must in ("add.Tensor", "mul.Tensor", "exp", "_softmax", "native_layer_norm", "mm", "bmm",
                 "addmm", "sum.dim_IntList", "mean.dim", "fill_.Scalar", "clone", "where.self"):
        assert must in names, must


def test_plain_shape_broadcast_matches_torch():
    """The eager ops broadcast operand shapes without torch's symbolic-shape machinery."""
    import pytest

    from torch_spyre.ops import _broadcast_shapes

    cases = [((3, 1), (1, 4)), ((5,), (2, 1, 5)), ((), (3,)), ((0, 3), (1, 3)), ((2, 3), (2, 3)), ((7, 1, 1), (1, 6, 5)),
             ((), ())]
    for shapes in cases:
        assert _broadcast_shapes(*shapes) == tuple(torch.broadcast_shapes(*shapes)), shapes
    with pytest.raises(RuntimeError):
        _broadcast_shapes((2, 3), (4, 3))
