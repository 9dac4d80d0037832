"""CPU test of the eager ops' cached marshalling (torch_spyre/ops.py:_launch_cached): for a set of
programs and shapes the cached plan hands ts_pointwise_chain exactly the instruction structs,
shape arrays, counts and flags that the general route (stick_ops.prepare_chain) builds.  No
kernel runs: the library entry is replaced by a recorder."""
import types

import pytest
import torch

import torch_spyre  # noqa: F401
from torch_spyre import _abi, ops, stick_ops as K


class _Image:
    device = torch.device("cpu")

    def data_ptr(self):
        return 0


class _Sticks:
    def __init__(self, shape):
        self.shape, self.image = tuple(shape), _Image()

    def ptr(self):
        return 0


@pytest.fixture
def recorder(monkeypatch):
    calls = []

    def entry(*args):
        calls.append(args)
        return 0

    monkeypatch.setattr(_abi, "lib", lambda: types.SimpleNamespace(ts_pointwise_chain=entry))
    monkeypatch.setattr(K, "_stream", lambda: 0)
    monkeypatch.setattr(ops, "_C", types.SimpleNamespace(storage_ptr=lambda t: 0, is_canonical=lambda t: True))
    ops._tls.plans = {}
    yield calls
    ops._tls.plans = {}


def _general(program, out_shape, in_shapes, calls):
    c = K.Chain()
    program(c, [c.tensor(_Sticks(s)) for s in in_shapes])
    launch, _, _ = K.prepare_chain(c, out_shape, outputs=[_Sticks(out_shape)])
    launch()
    return calls.pop()


CASES = [
    ("s-mul", lambda c, t: c.emit("LOAD", t[0]).emit("MUL", c.imm(0.125)).store(0),
     lambda c, t: c.emit("LOAD", t[0]).emit("MUL", c.imm(0.0)).store(0), (256, 256), [(256, 256)], 0.125),
    ("b-add-rowvec", lambda c, t: c.emit("LOAD", t[0]).emit("ADD", t[1]).store(0), None, (8, 64), [(8, 64), (64,)], None),
    ("b-sub-both-broadcast", lambda c, t: c.emit("LOAD", t[0]).emit("SUB", t[1]).store(0), None, (5, 3, 8, 64),
     [(1, 64), (5, 3, 8, 1)], None),
    ("u-exp-5d", lambda c, t: c.emit("LOAD", t[0]).emit("EXP").store(0), None, (2, 3, 4, 5, 70), [(2, 3, 4, 5, 70)], None),
    ("u-abs-0d", lambda c, t: c.emit("LOAD", t[0]).emit("ABS").store(0), None, (), [()], None),
    ("s-rsub", lambda c, t: c.emit("LOAD", t[0]).emit("RSUB", c.imm(-3.5)).store(0),
     lambda c, t: c.emit("LOAD", t[0]).emit("RSUB", c.imm(0.0)).store(0), (3, 130), [(3, 130)], -3.5),
]


@pytest.mark.parametrize("name,general,cached,out_shape,in_shapes,imm", CASES, ids=[c[0] for c in CASES])
def test_cached_plan_marshals_what_the_general_route_does(name, general, cached, out_shape, in_shapes, imm, recorder):
    want = _general(general, out_shape, in_shapes, recorder)
    for _ in range(2):      # built, then reused
        assert ops._launch_cached((name,), cached or general, out_shape, in_shapes,
                                  tuple(object() for _ in in_shapes), object(), imm=imm)
        got = recorder.pop()
        assert got[1] == want[1]
        for i in range(want[1]):
            for field, _ in _abi.PwInsn._fields_:
                assert getattr(got[0][i], field) == getattr(want[0][i], field), (i, field)
        n_in = want[4]
        assert got[4] == n_in and list(got[3])[:4 * n_in] == list(want[3])[:4 * n_in]
        assert got[6] == want[6] == 1 and list(got[7])[:4] == list(want[7])[:4]
        assert tuple(got[8:13]) == tuple(want[8:13])
    assert len(ops._tls.plans) == 1


def test_views_that_are_not_their_own_image_take_the_general_route(recorder, monkeypatch):
    monkeypatch.setattr(ops, "_C", types.SimpleNamespace(storage_ptr=lambda t: 0, is_canonical=lambda t: False))
    assert not ops._launch_cached(("x",), CASES[3][1], (4, 64), [(4, 64)], (object(),), object())
    assert not recorder and not ops._tls.plans
