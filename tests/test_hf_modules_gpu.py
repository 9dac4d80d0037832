"""Module tests of the reference that it carries as skipped (tests/test_modules.py:43-131), moved
to the spyre device eagerly, unmodified: nn.Linear, transformers' RobertaSelfAttention and
RobertaLayer with the reference's sizes (hidden 144, 12 heads of 12: nothing is a multiple of a
stick).  Oracle: the same module on CPU; the layer, a dozen fp16 ops deep, against an fp32
evaluation as well (the device may be at most 1.5 times as far from it as CPU fp16 eager is)."""
import copy

import pytest
import torch
import torch.nn as nn

import torch_spyre  # noqa: F401
from oracle import math_ref
from oracle.math_ref import assert_close

transformers = pytest.importorskip("transformers")
pytestmark = pytest.mark.gpu
DEV = "spyre"
H = torch.float16


@pytest.fixture(autouse=True)
def _need_gpu(cuda):
    yield


def test_linear_module():
    torch.manual_seed(0)
    m = nn.Linear(3, 5, dtype=H)
    ms = copy.deepcopy(m).to(DEV)
    x = torch.arange(6, dtype=H).view(2, 3)
    with torch.no_grad():
        assert_close(ms(x.to(DEV)).cpu(), m(x))


def _first(y):
    return y if torch.is_tensor(y) else y[0]


def _roberta(cls, shape):
    from transformers import RobertaConfig

    torch.manual_seed(0)
    cfg = RobertaConfig()
    cfg.hidden_size = 144
    m = cls(cfg).eval().to(H)
    ms = copy.deepcopy(m).to(DEV)
    x = torch.rand(*shape, cfg.hidden_size, dtype=H)
    with torch.no_grad():
        cpu16 = _first(m(x))
        got = _first(ms(x.to(DEV))).cpu()
        truth = _first(copy.deepcopy(m).float()(x.float()))
    return got, cpu16, truth


def test_roberta_self_attention():
    from transformers.models.roberta.modeling_roberta import RobertaSelfAttention

    got, cpu16, _ = _roberta(RobertaSelfAttention, (2, 10))
    assert_close(got, cpu16)


def test_roberta_layer():
    from transformers.models.roberta.modeling_roberta import RobertaLayer

    got, cpu16, truth = _roberta(RobertaLayer, (2, 10))
    assert got.shape == cpu16.shape
    math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, what="RobertaLayer")


def test_roberta_encoder():
    """tests/test_modules.py:112-131 (skipped there): twelve layers, [10, 384, 144]."""
    from transformers.models.roberta.modeling_roberta import RobertaEncoder

    got, cpu16, truth = _roberta(RobertaEncoder, (10, 384))
    assert got.shape == (10, 384, 144)
    math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, what="RobertaEncoder")


@pytest.mark.parametrize("which", ["attention", "layer"])
def test_llama_modules_with_the_reference_config(which):
    """tests/test_modules.py:133-211 (skipped there), with its sizes: hidden 1024, 32 heads of 32,
    1000 positions.  Through torch.compile (eagerly the module's RMS norm and softmax ask for fp32
    arithmetic, which the device refuses; compiled, those idioms are rewritten onto fp16 kernels that
    compute in fp32 inside).  A head size of 32 keeps torch's own attention decomposition."""
    from transformers.models.llama.modeling_llama import (LlamaAttention, LlamaConfig, LlamaDecoderLayer,
                                                          LlamaRotaryEmbedding)

    torch._dynamo.reset()
    torch.manual_seed(0)
    cfg = LlamaConfig()
    cfg.hidden_size = 1024
    cfg.head_dim = cfg.hidden_size // 32
    t = 1000
    m = (LlamaAttention if which == "attention" else LlamaDecoderLayer)(cfg, 0).eval().to(H)
    ms = copy.deepcopy(m).to(DEV).requires_grad_(False)
    x = torch.rand(1, t, cfg.hidden_size, dtype=H)
    cos, sin = LlamaRotaryEmbedding(cfg)(x, torch.arange(t).unsqueeze(0))
    cos, sin = cos.to(H), sin.to(H)
    fn = torch.compile(lambda a, c, s: ms(hidden_states=a, position_embeddings=(c, s), attention_mask=None))
    with torch.no_grad():
        cpu16 = _first(m(hidden_states=x, position_embeddings=(cos, sin), attention_mask=None))
        got = _first(fn(x.to(DEV), cos.to(DEV), sin.to(DEV))).cpu()
        truth = _first(copy.deepcopy(m).float()(hidden_states=x.float(), position_embeddings=(cos.float(), sin.float()),
                                                attention_mask=None))
    e = math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, what=f"Llama {which}")
    assert e["frac_within_tol"] > 0.999
