"""A whole forward pass on the device: token ids -> embedding -> three decoder layers -> final RMS
norm -> logits (examples/llama_model.py), eagerly and through torch.compile, against the CPU oracle.
The reference's module ladder stops at one decoder layer (tests/test_modules.py:133-211).

Three layers deep, the device and torch CPU fp16 eager round in different places, so both are
measured against an fp32 evaluation of the same fp16 weights (the criterion of the full-width
layer tests): the device may be at most 1.5 times as far from it as CPU eager is."""
import pytest
import torch

import torch_spyre  # noqa: F401
from examples.llama_model import LlamaStyleModel
from oracle import llama_ref as L
from oracle import math_ref
from torch_spyre import _abi

pytestmark = pytest.mark.gpu
DEV = "spyre"
VOCAB, LAYERS, BATCH, SEQ = 1000, 3, 2, 256


@pytest.fixture(autouse=True)
def _need_gpu(cuda):
    torch._dynamo.reset()
    yield


@pytest.fixture(scope="module")
def small():
    cfg = L.LayerConfig(d_model=256, heads=2, ffn=704)
    mw = L.make_model_weights(cfg, VOCAB, LAYERS)
    ids = torch.randint(0, VOCAB, (BATCH, SEQ), generator=torch.Generator().manual_seed(3))
    cpu16 = L.model_forward(ids, mw, cfg)
    truth = L.model_forward(ids, mw, cfg, dtype=torch.float32)
    return cfg, mw, ids, cpu16, truth


def _model(cfg, mw):
    cos, sin = L.rope_tables(SEQ, cfg.head_dim)
    to = lambda t: t.to(DEV)      # noqa: E731
    return LlamaStyleModel(to(mw["embed"]), [{k: to(v) for k, v in w.items()} for w in mw["layers"]],
                           to(mw["final_norm"]), to(mw["lm_head"]), cfg.heads, cfg.eps, to(cos), to(sin))


@pytest.mark.parametrize("compiled", [False, True])
def test_model_forward(small, compiled):
    cfg, mw, ids, cpu16, truth = small
    model = _model(cfg, mw)
    fn = torch.compile(model) if compiled else model
    got = fn(ids.to(DEV)).cpu()
    assert got.shape == (BATCH, SEQ, VOCAB) and got.dtype == torch.float16
    math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, what="model logits")
    assert _abi.lib().ts_gemm_error_state() == 0 and _abi.lib().ts_attention_error_state() == 0
    assert _abi.lib().ts_gather_error_state() == 0

