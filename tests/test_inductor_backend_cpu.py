"""The spyre classes inside Inductor, exercised without a device: fake spyre tensors are enough
for lowering, scheduling, kernel analysis and wrapper generation (running the wrapper needs the
GPU and is covered by the gpu tests).  Reference: torch_spyre/_inductor/dsc.py:28-63 (define_kernel /
call_kernel lines), spyre_kernel.py:85-369 (KernelSpec derivation), wrapper.py:51-62 (header)."""
import math

import pytest
import torch
import torch.nn.functional as F
from torch._subclasses.fake_tensor import FakeTensorMode
from torch.fx.experimental.proxy_tensor import make_fx

import torch_spyre  # noqa: F401
import torch._inductor.graph as G
import torch._inductor.lowering as L
from torch_spyre._inductor import compiler, patterns


def _compile(fn, *shapes):
    """Traces fn on fake spyre fp16 tensors and compiles it through Inductor; returns
    (generated wrapper source, record of the compilation)."""
    sources = []
    orig = G.GraphLowering.codegen

    def codegen(self):
        out = orig(self)
        sources.append(out[0].value)
        return out

    mode = FakeTensorMode()
    with mode:
        args = [torch.empty(*s, dtype=torch.float16, device="spyre") for s in shapes]
        gm = make_fx(fn, tracing_mode="fake", decomposition_table=compiler.spyre_decompositions())(*args)
    patterns.rewrite_aten_graph(gm)
    G.GraphLowering.codegen = codegen
    try:
        with mode:
            compiler.compile_with_inductor(gm, args)
    finally:
        G.GraphLowering.codegen = orig
    return sources[-1], compiler.last_compiled[-1]


def test_benchmark_graph_is_one_kernel_in_the_generated_wrapper():
    before = dict(L.lowerings)
    src, rec = _compile(lambda x, a, b: (torch.exp(x * a + b).sum(-1),), (8192, 8192), (8192,), (8192,))
    assert src.count("async_compile.sdsc(") == 1
    assert "from torch_spyre._inductor.runtime import ConstantArg, TensorArg, KernelSpec, UnimplementedOp" in src
    assert "async_compile = SpyreAsyncCompile()" in src
    assert ".run(x_1, a_1, b_1, buf0)" in src                   # inputs first, the output last
    assert "buf0 = empty_strided((8192, ), (1, ), device='spyre', dtype=torch.float16)" in src
    (spec,) = rec.kernel_specs
    assert spec.op == "fused_pointwise_rowreduce" and spec.is_reduction and spec.dimensions == [8192, 8192]
    assert [i[0] for i in spec.op_info["insns"]] == ["LOAD", "MUL", "ADD", "EXP"]
    assert spec.scales == [[1, 1], [-1, 1], [-1, 1], [1, -1]]   # x walks both dims, a and b only the inner one
    assert [a.is_input for a in spec.args] == [True, True, True, False]
    assert dict(L.lowerings) == before                          # nothing registered outlives the compilation


def test_pointwise_group_with_two_results_and_a_mean():
    def fn(t, u):
        s = torch.relu(t + u)
        return s, torch.tanh(s) * 2.0, (s * 0.5).mean(-1)

    src, rec = _compile(fn, (16, 128), (16, 128))
    specs = rec.kernel_specs
    assert all(s.op.startswith("fused_pointwise") for s in specs) and len(specs) <= 2
    red = [s for s in specs if s.is_reduction]
    assert len(red) == 1 and abs(red[0].op_info["reduce_scale"] - 1 / 128) < 1e-12
    assert src.count(".run(") == len(specs)


def test_decoder_layer_goes_through_extern_kernels_and_custom_ops():
    def layer(x, wq, wk, wv, wo, wg, wu, wd, n1, n2, cos, sin):
        heads = 4
        scale = 1.0 / math.sqrt(x.shape[-1] // heads)
        h = torch.ops.spyre.rms_norm(x, n1, 1e-5)
        q = torch.ops.spyre.rotary(F.linear(h, wq), cos, sin, heads)
        k = torch.ops.spyre.rotary(F.linear(h, wk), cos, sin, heads)
        v = F.linear(h, wv)
        attn = torch.ops.spyre.causal_attention(q, k, v, heads, scale)
        x = x + F.linear(attn, wo)
        h = torch.ops.spyre.rms_norm(x, n2, 1e-5)
        return (x + F.linear(F.silu(F.linear(h, wg)) * F.linear(h, wu), wd),)

    d, f = 512, 1024
    src, rec = _compile(layer, (2, 256, d), (d, d), (d, d), (d, d), (d, d), (f, d), (f, d), (d, f), (d,), (d,),
                        (256, 128), (256, 128))
    assert src.count("extern_kernels.mm(") == 3 and src.count("extern_kernels.addmm(") == 2   # residuals ride in the GEMMs
    assert src.count("torch.ops.spyre.rms_norm.default(") == 2 and src.count("torch.ops.spyre.rotary.default(") == 2
    assert "torch.ops.spyre.causal_attention.default(" in src and "torch.ops.spyre.swiglu_linear.default(" in src
    assert rec.kernel_specs == []          # nothing left for a pointwise kernel: 11 launches in all


def test_softmax_and_layer_norm_stay_whole():
    src, rec = _compile(lambda x, w, b: (torch.softmax(x, -1), F.layer_norm(x, (256,), w, b) + 1.0),
                        (64, 256), (256,), (256,))
    assert "torch.ops.aten._softmax.default(" in src and "torch.ops.aten.native_layer_norm.default(" in src
    assert len(rec.kernel_specs) == 1      # the "+ 1.0"


def test_what_the_scheduling_cannot_express_is_refused():
    from torch_spyre._inductor import Unsupported
    from torch._inductor.exc import InductorError

    with pytest.raises((Unsupported, InductorError), match="row-major walk|not an iteration variable|offset"):
        _compile(lambda x, y: (torch.relu(x.t() + y),), (64, 128), (128, 64))


def test_reference_names_import():
    from torch_spyre._inductor.choices import SpyreHeuristics
    from torch_spyre._inductor.dsc import SuperDSCScheduling
    from torch_spyre._inductor.spyre_kernel import SpyreKernel  # noqa: F401
    from torch_spyre._inductor.stickify import SpyreDCI, SpyreFixedLayout, StickFormat
    from torch_spyre._inductor.wrapper import SpyrePythonWrapperCodegen
    from torch_spyre.utils.device_op_overrides import SpyreDeviceOpOverrides
    from torch._inductor.codegen.common import get_scheduling_for_device, get_wrapper_codegen_for_device

    assert get_scheduling_for_device("spyre") is SuperDSCScheduling
    assert get_wrapper_codegen_for_device("spyre") is SpyrePythonWrapperCodegen
    assert SpyreHeuristics.reduction_split_factor(torch.device("spyre"), 8192, 8192, True) == 1
    dci = SpyreDCI([0, 1, 2])
    assert dci.spyre_strides([4, 8, 128], torch.float16) == [1024, 128, 1] and dci.is_stick_dim(2)
    assert SpyreDCI([2, 0, 1]).spyre_strides([3, 4, 130], torch.float16) == [4, 1, 12]
    assert SpyreDCI([0, 1], format=StickFormat.SPARSE).spyre_strides([5, 7], torch.float16) == [448, 64]
    lay = dci.spyre_layout(torch.device("spyre"), [4, 8, 128], torch.float16)
    assert isinstance(lay, SpyreFixedLayout) and "dci=" in str(lay)
    assert "set_device" in SpyreDeviceOpOverrides().set_device(0)
