#!/usr/bin/env python
"""Benchmark of the hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload ("fused"): y = exp(x*a + b).sum(-1), x fp16 [8192, 8192] N(0,1),
a and b fp16 [8192] U(-1,1), one fused kernel per step over inputs resident in
HBM as stick images.  A step reads a different x buffer of a ring larger than L2.
Other workloads: softmax, softmax_scaled, pointwise, relayout, relayout_permuted, bmm, attention,
llama_layer.
Under torchrun every rank runs the same per-GPU workload on its own shard of
rows (weak scaling, no collective on the data path).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "torch-spyre_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return (p.get("hbm_gbs", 6650.0), p.get("bf16_tflops", 1590.0),
                p.get("bf16_tflops_sustained", 1400.0), "measured")
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- workloads

def make_workload(name: str, dev, scale_rows=None):
    """Returns dict(step_dev, step_e2e, alg_bytes, h2d, d2h, launches, desc, cpu_step, sample)."""
    from oracle import math_ref
    from torch_spyre import stick_ops as K

    if name == "fused":
        rows = cols = 8192
        x, a, b = math_ref.fused_inputs(rows, cols)
        xp, ap, bp = x.pin_memory(), a.pin_memory(), b.pin_memory()
        ring = max(2, -(-2 * L2_BYTES // (rows * cols * 2)) + 1)  # ring of x buffers > 2x L2
        sa, sb = K.copy_host_to_sticks(ap), K.copy_host_to_sticks(bp)
        xs = [K.copy_host_to_sticks(xp)]
        for _ in range(ring - 1):
            xs.append(K.StickTensor(xs[0].image.clone(), xs[0].shape))
        out = K.empty((rows,))

        def chain_on(sx, sa_, sb_):
            c = K.Chain()
            c.emit("LOAD", c.tensor(sx)).emit("MUL", c.tensor(sa_)).emit("ADD", c.tensor(sb_)).emit("EXP")
            return c

        launches = [K.prepare_chain(chain_on(sx, sa, sb), (rows, cols), n_outputs=0, reduce="sum")[0]
                    for sx in xs]
        state = {"i": 0}

        def step_dev():
            launches[state["i"] % ring]()
            state["i"] += 1

        # end to end through the public API: host tensors -> .to("spyre") -> torch.compile'd
        # graph (one fused kernel) -> .cpu()
        import torch_spyre  # noqa: F401
        spyre_dev = torch.device("spyre", dev.index)
        compiled = torch.compile(lambda t, u, v: torch.exp(t * u + v).sum(-1))

        def step_e2e():
            y = compiled(xp.to(spyre_dev), ap.to(spyre_dev), bp.to(spyre_dev))
            return y.cpu()

        alg = rows * cols * 2 + cols * 2 * 2 + rows * 2

        def cpu_step():
            return math_ref.fused_ref(x, a, b)

        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=alg,
                    h2d=rows * cols * 2 + 2 * cols * 2, d2h=rows * 2, launches=1,
                    # ncu, one launch at this size: 134,263,296 B read + 3,333,632 B written
                    traffic=137596928 if (rows, cols) == (8192, 8192) else None,
                    graph_period=ring,
                    desc=f"exp(x*a+b).sum(-1), x fp16 [{rows},{cols}] (BASELINE configs[1])",
                    l2=f"ring of {ring} x buffers ({ring * rows * cols * 2 >> 20} MiB) > L2",
                    cpu_step=cpu_step, sample="full [8192,8192] graph per CPU step",
                    check=lambda: math_ref.assert_close(step_e2e().clone(), cpu_step()))

    if name == "pointwise":
        rows = cols = 8192
        x, a, b = math_ref.fused_inputs(rows, cols)
        xp = x.pin_memory()
        sb = K.copy_host_to_sticks(b.pin_memory())
        ring = 3
        xs = [K.copy_host_to_sticks(xp)]
        for _ in range(ring - 1):
            xs.append(K.StickTensor(xs[0].image.clone(), xs[0].shape))
        outs = [K.empty((rows, cols)) for _ in range(ring)]

        def chain_on(sx):
            c = K.Chain()
            c.emit("LOAD", c.tensor(sx)).emit("ADD", c.tensor(sb)).store(0)
            return c

        launches = [K.prepare_chain(chain_on(sx), (rows, cols), outputs=[o])[0] for sx, o in zip(xs, outs)]
        state = {"i": 0}

        def step_dev():
            launches[state["i"] % ring]()
            state["i"] += 1

        staging = torch.empty(rows * cols * 2, dtype=torch.uint8, device=dev)
        sx_e = K.empty((rows, cols))
        y_host = torch.empty(rows, cols, dtype=torch.float16).pin_memory()

        def step_e2e():
            K.copy_host_to_sticks(xp, sx_e, staging)
            (o,), _ = K.run_chain(chain_on(sx_e), (rows, cols), outputs=[outs[0]])
            K.copy_sticks_to_host(o, y_host, staging)
            torch.cuda.current_stream().synchronize()
            return y_host

        def cpu_step():
            return x + b

        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=2 * rows * cols * 2 + cols * 2,
                    h2d=rows * cols * 2, d2h=rows * cols * 2, launches=1,
                    # ncu, one launch at this size: 134,248,704 B read + 77,152,000 B written
                    # (the rest of the output was still in L2 when the kernel ended)
                    traffic=211400704 if (rows, cols) == (8192, 8192) else None,
                    graph_period=ring,
                    desc=f"pointwise x + b (b broadcast along rows), fp16 [{rows},{cols}]",
                    l2=f"ring of {ring} input and output buffers ({2 * ring * rows * cols * 2 >> 20} MiB) > L2",
                    cpu_step=cpu_step, sample="full [8192,8192] add per CPU step",
                    check=lambda: math_ref.assert_close(step_e2e().clone(), cpu_step()))

    if name in ("softmax", "softmax_scaled"):
        rows, cols = (256, 4096) if name == "softmax" else (scale_rows or 65536, 4096)
        x = math_ref.softmax_inputs(256, cols)
        if rows != 256:
            x = x.repeat(rows // 256, 1)
        xp = x.pin_memory()
        ring = max(2, -(-2 * L2_BYTES // (rows * cols * 2)) + 1)
        ring = min(ring, 160)
        xs = [K.copy_host_to_sticks(xp)]
        for _ in range(ring - 1):
            xs.append(K.StickTensor(xs[0].image.clone(), xs[0].shape))
        outs = [K.empty((rows, cols)) for _ in range(min(ring, 4) if rows > 256 else ring)]
        state = {"i": 0}

        def step_dev():
            i = state["i"]
            state["i"] += 1
            K.softmax_rows(xs[i % ring], out=outs[i % len(outs)])

        staging = torch.empty(rows * cols * 2, dtype=torch.uint8, device=dev)
        sx_e, sy_e = K.empty((rows, cols)), K.empty((rows, cols))
        y_host = torch.empty(rows, cols, dtype=torch.float16).pin_memory()

        def step_e2e():
            K.copy_host_to_sticks(xp, sx_e, staging)
            K.softmax_rows(sx_e, out=sy_e)
            K.copy_sticks_to_host(sy_e, y_host, staging)
            torch.cuda.current_stream().synchronize()
            return y_host

        def cpu_step():
            return torch.softmax(x, -1)

        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=2 * rows * cols * 2,
                    h2d=rows * cols * 2, d2h=rows * cols * 2, launches=1,
                    # ncu at [16384, 4096]: 134,235,648 B read + 79,373,312 B written (part of
                    # the output still in L2), scaled by rows
                    traffic=int(213608960 * rows / 16384) if cols == 4096 else None,
                    graph_period=ring if rows == 256 else 0,
                    desc=f"softmax(dim=-1) fp16 [{rows},{cols}]" +
                         (" (BASELINE configs[0])" if rows == 256 else " (configs[0] scaled along rows)"),
                    l2=f"ring of {ring} input buffers ({ring * rows * cols * 2 >> 20} MiB) > L2",
                    cpu_step=cpu_step, sample=f"full [{rows},{cols}] softmax per CPU step",
                    check=lambda: math_ref.assert_close(step_e2e().clone(), cpu_step()))

    if name in ("relayout", "relayout_permuted"):
        permuted = name.endswith("permuted")
        shape = (scale_rows or 64, 2048, 4096)
        # a [4,...] seeded block repeated along dim 0 keeps host generation quick
        blk = math_ref.relayout_inputs((4,) + shape[1:], 0, permuted=False)
        host = blk.repeat(shape[0] // 4, 1, 1)
        if permuted:
            host = host.permute(0, 2, 1).contiguous().permute(0, 2, 1)
        hp = host.pin_memory()
        raw = hp.to(dev, non_blocking=True)
        assert raw.stride() == host.stride()
        st = K.to_sticks(raw)
        back = torch.empty_strided(shape, host.stride(), dtype=host.dtype, device=dev)
        state = {"i": 0}

        def step_dev():
            # one step = host image -> sticks -> host image, both directions of copy_
            K.to_sticks(raw, out=st)
            K.from_sticks(st, out=back)

        staging = torch.empty(host.numel() * 2, dtype=torch.uint8, device=dev)
        out_host = torch.empty_strided(shape, host.stride(), dtype=host.dtype).pin_memory()

        def step_e2e():
            K.copy_host_to_sticks(hp, st, staging)
            K.copy_sticks_to_host(st, out_host, staging)
            torch.cuda.current_stream().synchronize()
            return out_host

        nbytes = host.numel() * 2

        def check():
            if not torch.equal(step_e2e().view(torch.int16), host.view(torch.int16)):
                raise AssertionError("relayout round trip is not the identity")
            if not torch.equal(back.view(torch.int16).cpu()[:2], host.view(torch.int16)[:2]):
                step_dev()
                torch.cuda.synchronize()
                assert torch.equal(back.view(torch.int16).cpu(), host.view(torch.int16))

        def cpu_step():
            import numpy as np
            from oracle import layout as OL, relayout_c as OC
            h = host[:8].view(torch.int16).numpy().view(np.uint16)
            img = OC.to_sticks(h, OL.generic_stick_layout(h.shape), nthreads=os.cpu_count() or 1)
            return OC.from_sticks(img, OL.generic_stick_layout(h.shape), h.shape,
                                  nthreads=os.cpu_count() or 1)

        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=4 * nbytes,
                    h2d=nbytes, d2h=nbytes, launches=2,
                    # ncu at [16, 2048, 4096], one direction: 268.45 MB read + 213.6 MB written
                    # (contiguous) / 213.3 MB (permuted), scaled by the outer extent
                    traffic=int((482078208 if not permuted else 481772544) * shape[0] / 16),
                    desc=f"stick relayout fp16 {list(shape)} host strides {list(host.stride())}, "
                         "to sticks and back (BASELINE configs[2])",
                    l2="1 GiB tensors, far larger than L2", cpu_step=cpu_step, cpu_scale=8.0,
                    sample="C oracle on a [8,2048,4096] slice (1/8 of the tensor), all host threads",
                    cpu_kind="port", check=check)
    if name == "bmm":
        batch, m, k, n = scale_rows or 32, 2048, 4096, 4096
        a1, b1 = math_ref.bmm_inputs(batch=1)
        sa1, sb1 = K.copy_host_to_sticks(a1.pin_memory()), K.copy_host_to_sticks(b1.pin_memory())
        # the seeded [1, ...] block repeated along the batch keeps host generation quick
        sa = K.StickTensor(sa1.image.view(k // 64, 1, m * 64).repeat(1, batch, 1).reshape(-1), (batch, m, k))
        sb = K.StickTensor(sb1.image.view(n // 64, 1, k * 64).repeat(1, batch, 1).reshape(-1), (batch, k, n))
        sc = K.empty((batch, m, n))

        def step_dev():
            K.matmul(sa, sb, out=sc)

        ah = a1.repeat(batch, 1, 1).pin_memory()
        bh = b1.repeat(batch, 1, 1).pin_memory()
        ch = torch.empty(batch, m, n, dtype=torch.float16).pin_memory()
        staging = torch.empty(bh.numel() * 2, dtype=torch.uint8, device=dev)
        sa_e, sb_e = K.empty((batch, m, k)), K.empty((batch, k, n))

        def step_e2e():
            K.copy_host_to_sticks(ah, sa_e, staging)
            K.copy_host_to_sticks(bh, sb_e, staging)
            K.matmul(sa_e, sb_e, out=sc)
            K.copy_sticks_to_host(sc, ch, staging)
            torch.cuda.current_stream().synchronize()
            return ch

        def cpu_step():
            return torch.bmm(a1, b1)

        def check():
            got = step_e2e()[batch - 1, :256].clone()
            math_ref.assert_close(got, torch.bmm(a1[:, :256], b1)[0])
            if K._abi.lib().ts_gemm_error_state() != 0:
                raise AssertionError("GEMM kernel gave up on an internal wait")

        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=0,
                    flops=2.0 * batch * m * k * n, cpu_scale=float(batch),
                    h2d=(ah.numel() + bh.numel()) * 2, d2h=ch.numel() * 2, launches=1,
                    # ncu at batch 4: 248,113,408 B read + 52,386,048 B written, scaled by batch
                    traffic=int(300499456 * batch / 4) if (m, k, n) == (2048, 4096, 4096) else None,
                    desc=f"bmm fp16 [{batch},{m},{k}] x [{batch},{k},{n}], fp32 accumulate "
                         "(BASELINE configs[3])",
                    l2="operands 1.5 GiB, far larger than L2", cpu_step=cpu_step,
                    sample="one batch entry [1,2048,4096]x[1,4096,4096] per CPU step (1/32 of the job)",
                    check=check)
    if name in ("llama_layer", "hf_llama_layer"):
        import torch_spyre  # noqa: F401
        from oracle import llama_ref as LR
        world = int(os.environ.get("WORLD_SIZE", "1"))
        cfg = LR.LayerConfig()
        batch, seq = max(1, (scale_rows or 8) // world), 2048   # the batch of 8 is sharded over the ranks
        w = LR.make_weights(cfg)
        cos, sin = LR.rope_tables(seq, cfg.head_dim)
        sdev = torch.device("spyre", dev.index)
        if name == "llama_layer":
            from examples.llama_layer import LlamaStyleLayer
            layer = LlamaStyleLayer({k: v.to(sdev) for k, v in w.items()}, cfg.heads, cfg.eps,
                                    cos.to(sdev), sin.to(sdev))
            compiled = torch.compile(layer)
        else:
            # the module the reference's own (skipped) test builds, unmodified, same weights
            import transformers as tf
            from transformers.models.llama.modeling_llama import LlamaDecoderLayer
            hc = tf.LlamaConfig(hidden_size=cfg.d_model, num_attention_heads=cfg.heads,
                                num_key_value_heads=cfg.heads, intermediate_size=cfg.ffn,
                                rms_norm_eps=cfg.eps, num_hidden_layers=1,
                                max_position_embeddings=seq, attn_implementation="sdpa")
            with torch.device("meta"):
                hf = LlamaDecoderLayer(hc, 0).half().eval()
            hf = hf.to_empty(device="cpu")
            hf.load_state_dict({
                "self_attn.q_proj.weight": w["q"], "self_attn.k_proj.weight": w["k"],
                "self_attn.v_proj.weight": w["v"], "self_attn.o_proj.weight": w["o"],
                "mlp.gate_proj.weight": w["gate"], "mlp.up_proj.weight": w["up"],
                "mlp.down_proj.weight": w["down"], "input_layernorm.weight": w["norm1"],
                "post_attention_layernorm.weight": w["norm2"]}, strict=False)
            hf = hf.to(sdev).requires_grad_(False)     # forward only: the fused ops define no backward
            cos_b = cos.unsqueeze(0).expand(batch, -1, -1).contiguous().to(sdev)
            sin_b = sin.unsqueeze(0).expand(batch, -1, -1).contiguous().to(sdev)
            pos = torch.arange(seq)[None].expand(batch, -1)

            def hf_forward(x):
                out = hf(x, position_embeddings=(cos_b, sin_b), attention_mask=None, position_ids=pos)
                return out[0] if isinstance(out, tuple) else out

            compiled = torch.compile(hf_forward)
        x1 = (torch.randn(1, seq, cfg.d_model, generator=torch.Generator().manual_seed(0))).half()
        xh = x1.repeat(batch, 1, 1).pin_memory()
        xd = xh.to(sdev)
        compiled(xd)  # compile once, outside every timed region

        def step_dev():
            compiled(xd)

        def step_e2e():
            return compiled(xh.to(sdev)).cpu()

        def cpu_step():
            return LR.layer_forward(x1[:, :512], w, cfg)

        def check():
            got = step_e2e()[batch - 1, :64]
            want = LR.layer_forward(x1[:, :64], w, cfg)[0]      # causal: a prefix depends on itself only
            # A whole layer at full width (K up to 11008, ~10 fp16 roundings deep): two fp16
            # evaluations that round in different places agree to a few fp16 ulps of the
            # output scale, not element by element at atol 1e-3.  Require that all but 1 % of
            # the elements meet rtol 1e-2 / atol 5e-3 and that none is off by more than 3e-2.
            diff = (got.float() - want.float()).abs()
            bad = diff > (5e-3 + 1e-2 * want.float().abs())
            if bad.float().mean() > 0.01 or diff.max() > 3e-2:
                raise AssertionError(f"layer parity: {bad.float().mean():.4f} of elements out of "
                                     f"tolerance, max abs diff {diff.max():.4f}")
            if K._abi.lib().ts_gemm_error_state() != 0:
                raise AssertionError("GEMM kernel gave up on an internal wait")

        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=0,
                    flops=LR.layer_flops(batch, seq, cfg, causal=True),
                    cpu_flops=LR.layer_flops(1, 512, cfg, causal=True), scaling="strong",
                    h2d=xh.numel() * 2, d2h=xh.numel() * 2, launches=11,
                    desc=("transformers LlamaDecoderLayer (unmodified)" if name == "hf_llama_layer"
                          else "Llama-style decoder layer") +
                         " through torch.compile on spyre: d_model 4096, 32 heads x 128, "
                         f"SwiGLU 11008, RMSNorm, rotary, causal attention, batch {batch} x seq {seq} per GPU, "
                         "causal-useful flops (BASELINE configs[4])",
                    l2="activations and weights (> 1 GiB) far larger than L2", cpu_step=cpu_step,
                    sample="oracle layer on [1, 512, 4096] per CPU step", check=check)
    if name == "attention":
        # config 5's attention block on its own: packed [B*S, H*128] q / k / v images in, packed out
        import math
        batch, seq, heads, hd = scale_rows or 8, 2048, 32, 128
        g = torch.Generator().manual_seed(0)
        qh, kh, vh = (torch.randn(batch, seq, heads * hd, generator=g).half().pin_memory() for _ in range(3))
        scale = 1.0 / math.sqrt(hd)
        qs, ks, vs = (K.copy_host_to_sticks(t) for t in (qh, kh, vh))
        out = K.empty((batch, seq, heads * hd), torch.float16, dev)
        out_host = torch.empty_like(qh).pin_memory()

        def step_dev():
            K.causal_attention(qs, ks, vs, batch, seq, heads, scale, out=out)

        def step_e2e():
            q2, k2, v2 = (K.copy_host_to_sticks(t) for t in (qh, kh, vh))
            o = K.causal_attention(q2, k2, v2, batch, seq, heads, scale)
            K.copy_sticks_to_host(o, out_host)
            torch.cuda.synchronize()
            return out_host

        def ref(nb, nh):
            q4, k4, v4 = (t[:nb, :, :nh * hd].reshape(nb, seq, nh, hd).transpose(1, 2).float()
                          for t in (qh, kh, vh))
            o = torch.nn.functional.scaled_dot_product_attention(q4, k4, v4, is_causal=True, scale=scale)
            return o.transpose(1, 2).reshape(nb, seq, nh * hd).half()

        def cpu_step():
            return ref(1, 4)

        def check():
            got = step_e2e()[:1, :, :4 * hd]
            math_ref.assert_close(got, ref(1, 4), atol=2e-3)
            if K._abi.lib().ts_attention_error_state() != 0:
                raise AssertionError("attention kernel gave up on an internal wait")

        flops = 4.0 * batch * heads * hd * (seq * (seq + 1) / 2)   # causal-useful: keys <= query
        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=0, flops=flops,
                    cpu_flops=flops / (batch * heads / 4), h2d=3 * qh.numel() * 2, d2h=qh.numel() * 2,
                    launches=1,
                    desc=f"causal attention fp16, batch {batch} x seq {seq} x {heads} heads x {hd}, "
                         "causal-useful flops (the attention block of BASELINE configs[4])",
                    l2="q, k, v, out 512 MiB, larger than L2", cpu_step=cpu_step,
                    sample="torch CPU scaled_dot_product_attention (fp32) on 1 batch entry x 4 heads",
                    check=check)
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------- timing

def time_device(step, steps, warmup, graph_period=0):
    """Times exactly `steps` calls of `step` with CUDA events.  When the workload says its
    steps repeat with period `graph_period` (a ring of buffers), one period is captured in a
    CUDA graph and replayed, so that host launch overhead stays out of a microsecond-scale
    kernel's timing; the remainder is launched directly."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    graph = None
    if graph_period and steps >= 2 * graph_period:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(graph_period):
                step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(graph_period):
                    step()
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    if graph is not None:
        for _ in range(steps // graph_period):
            graph.replay()
        for _ in range(steps % graph_period):
            step()
    else:
        for _ in range(steps):
            step()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / 1e3


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs are meant to use every host
    core this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def time_cpu(fn, budget_s=12.0, min_runs=3):
    fn()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_runs or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
        if len(times) >= 200:
            break
    times.sort()
    return times[len(times) // 2], len(times)


def run_reference(args, rank, world):
    """Reference arm: the path's CPU implementation (torch CPU eager, which is what
    the reference's tests hold the device to) on the host cores."""
    if rank != 0:
        return
    from oracle import math_ref  # noqa: F401
    use_all_host_threads()
    wl = make_workload_cpu(args.workload)
    wl["cpu_step"]()
    for _ in range(max(args.warmup - 1, 0)):
        wl["cpu_step"]()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl["cpu_step"]()
    dt = (time.perf_counter() - t0) / args.steps
    scale = wl.get("cpu_scale", 1.0)
    is_flops = "flops" in wl
    gbs = (wl["flops"] / 1e3 if is_flops else wl["alg_bytes"]) / scale / dt / 1e9
    cores = torch.get_num_threads()
    unit = "TFLOP/s" if is_flops else "GB/s"
    line = {"impl": "reference",
            "metric": "fp16 GEMM TFLOP/s" if is_flops else "achieved GB/s (algorithmic bytes / time)",
            "value": gbs, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3 * scale, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": wl["desc"]},
            "cpu_baseline": {"value": gbs, "unit": unit, "cores": cores, "kind": "port",
                             "sample": wl["sample"] + "; torch CPU eager / C oracle on host cores"},
            "e2e": {"value": gbs, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def make_workload_cpu(name):
    """CPU-only description of a workload (no CUDA needed): used by the reference arm."""
    from oracle import math_ref
    if name == "fused":
        x, a, b = math_ref.fused_inputs()
        return dict(cpu_step=lambda: math_ref.fused_ref(x, a, b), alg_bytes=134266880,
                    desc="exp(x*a+b).sum(-1), x fp16 [8192,8192] (BASELINE configs[1])",
                    sample="full [8192,8192] graph per CPU step")
    if name == "pointwise":
        rows = cols = 8192
        x, a, b = math_ref.fused_inputs(rows, cols)
        xp = x.pin_memory()
        sb = K.copy_host_to_sticks(b.pin_memory())
        ring = 3
        xs = [K.copy_host_to_sticks(xp)]
        for _ in range(ring - 1):
            xs.append(K.StickTensor(xs[0].image.clone(), xs[0].shape))
        outs = [K.empty((rows, cols)) for _ in range(ring)]

        def chain_on(sx):
            c = K.Chain()
            c.emit("LOAD", c.tensor(sx)).emit("ADD", c.tensor(sb)).store(0)
            return c

        launches = [K.prepare_chain(chain_on(sx), (rows, cols), outputs=[o])[0] for sx, o in zip(xs, outs)]
        state = {"i": 0}

        def step_dev():
            launches[state["i"] % ring]()
            state["i"] += 1

        staging = torch.empty(rows * cols * 2, dtype=torch.uint8, device=dev)
        sx_e = K.empty((rows, cols))
        y_host = torch.empty(rows, cols, dtype=torch.float16).pin_memory()

        def step_e2e():
            K.copy_host_to_sticks(xp, sx_e, staging)
            (o,), _ = K.run_chain(chain_on(sx_e), (rows, cols), outputs=[outs[0]])
            K.copy_sticks_to_host(o, y_host, staging)
            torch.cuda.current_stream().synchronize()
            return y_host

        def cpu_step():
            return x + b

        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=2 * rows * cols * 2 + cols * 2,
                    h2d=rows * cols * 2, d2h=rows * cols * 2, launches=1,
                    # ncu, one launch at this size: 134,248,704 B read + 77,152,000 B written
                    # (the rest of the output was still in L2 when the kernel ended)
                    traffic=211400704 if (rows, cols) == (8192, 8192) else None,
                    graph_period=ring,
                    desc=f"pointwise x + b (b broadcast along rows), fp16 [{rows},{cols}]",
                    l2=f"ring of {ring} input and output buffers ({2 * ring * rows * cols * 2 >> 20} MiB) > L2",
                    cpu_step=cpu_step, sample="full [8192,8192] add per CPU step",
                    check=lambda: math_ref.assert_close(step_e2e().clone(), cpu_step()))

    if name in ("softmax", "softmax_scaled"):
        rows = 256 if name == "softmax" else 65536
        x = math_ref.softmax_inputs(256, 4096).repeat(rows // 256, 1)
        return dict(cpu_step=lambda: torch.softmax(x, -1), alg_bytes=2 * rows * 4096 * 2,
                    desc=f"softmax(dim=-1) fp16 [{rows},4096]", sample="full softmax per CPU step")
    if name in ("relayout", "relayout_permuted"):
        import numpy as np
        from oracle import layout as OL, relayout_c as OC
        host = math_ref.relayout_inputs((8, 2048, 4096), 0, permuted=name.endswith("permuted"))
        h = host.view(torch.int16).numpy().view(np.uint16)
        lay = OL.generic_stick_layout(h.shape)
        nt = os.cpu_count() or 1

        def cpu_step():
            return OC.from_sticks(OC.to_sticks(h, lay, nthreads=nt), lay, h.shape, nthreads=nt)

        return dict(cpu_step=cpu_step, alg_bytes=4 * 64 * 2048 * 4096 * 2, cpu_scale=8.0,
                    desc="stick relayout fp16 [64,2048,4096], to sticks and back (BASELINE configs[2])",
                    sample="C oracle on a [8,2048,4096] slice (1/8 of the tensor)")
    if name == "bmm":
        a1, b1 = math_ref.bmm_inputs(batch=1)
        return dict(cpu_step=lambda: torch.bmm(a1, b1), flops=2.0 * 32 * 2048 * 4096 * 4096,
                    cpu_scale=32.0, alg_bytes=0,
                    desc="bmm fp16 [32,2048,4096] x [32,4096,4096] (BASELINE configs[3])",
                    sample="one batch entry per CPU step (1/32 of the job)")
    if name == "attention":
        # config 5's attention block on its own: packed [B*S, H*128] q / k / v images in, packed out
        import math
        batch, seq, heads, hd = scale_rows or 8, 2048, 32, 128
        g = torch.Generator().manual_seed(0)
        qh, kh, vh = (torch.randn(batch, seq, heads * hd, generator=g).half().pin_memory() for _ in range(3))
        scale = 1.0 / math.sqrt(hd)
        qs, ks, vs = (K.copy_host_to_sticks(t) for t in (qh, kh, vh))
        out = K.empty((batch, seq, heads * hd), torch.float16, dev)
        out_host = torch.empty_like(qh).pin_memory()

        def step_dev():
            K.causal_attention(qs, ks, vs, batch, seq, heads, scale, out=out)

        def step_e2e():
            q2, k2, v2 = (K.copy_host_to_sticks(t) for t in (qh, kh, vh))
            o = K.causal_attention(q2, k2, v2, batch, seq, heads, scale)
            K.copy_sticks_to_host(o, out_host)
            torch.cuda.synchronize()
            return out_host

        def ref(nb, nh):
            q4, k4, v4 = (t[:nb, :, :nh * hd].reshape(nb, seq, nh, hd).transpose(1, 2).float()
                          for t in (qh, kh, vh))
            o = torch.nn.functional.scaled_dot_product_attention(q4, k4, v4, is_causal=True, scale=scale)
            return o.transpose(1, 2).reshape(nb, seq, nh * hd).half()

        def cpu_step():
            return ref(1, 4)

        def check():
            got = step_e2e()[:1, :, :4 * hd]
            math_ref.assert_close(got, ref(1, 4), atol=2e-3)
            if K._abi.lib().ts_attention_error_state() != 0:
                raise AssertionError("attention kernel gave up on an internal wait")

        flops = 4.0 * batch * heads * hd * (seq * (seq + 1) / 2)   # causal-useful: keys <= query
        return dict(step_dev=step_dev, step_e2e=step_e2e, alg_bytes=0, flops=flops,
                    cpu_flops=flops / (batch * heads / 4), h2d=3 * qh.numel() * 2, d2h=qh.numel() * 2,
                    launches=1,
                    desc=f"causal attention fp16, batch {batch} x seq {seq} x {heads} heads x {hd}, "
                         "causal-useful flops (the attention block of BASELINE configs[4])",
                    l2="q, k, v, out 512 MiB, larger than L2", cpu_step=cpu_step,
                    sample="torch CPU scaled_dot_product_attention (fp32) on 1 batch entry x 4 heads",
                    check=check)
    raise SystemExit(f"unknown workload {name}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="fused")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host")
    ap.add_argument("--rows", type=int, default=None,
                    help="profiling aid: rows of softmax_scaled / outer extent of relayout")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    wl = make_workload(args.workload, dev, args.rows)
    wl["check"]()  # parity of one step against the CPU oracle before timing anything

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    barrier()
    if rank == 0:
        # keep the device busy long enough for the clock sampler to see it under load
        t_end = time.perf_counter() + 0.5
        while time.perf_counter() < t_end:
            for _ in range(8):
                wl["step_dev"]()
            torch.cuda.synchronize()
    barrier()
    dt = time_device(wl["step_dev"], args.steps, args.warmup,
                     0 if args.no_graph else wl.get("graph_period", 0))
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    e2e_dt = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            wl["step_e2e"]()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            wl["step_e2e"]()
        torch.cuda.synchronize()
        e2e_dt = (time.perf_counter() - t0) / e2e_steps

    if dist is not None:
        t = torch.tensor([dt, e2e_dt or 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt, e2e_dt = float(t[0]), (float(t[1]) if e2e_dt is not None else None)

    if rank == 0:
        hbm, tflops_burst, tflops_sustained, which = measured_peaks()
        is_flops = "flops" in wl
        # a timed region of a fraction of a second is a burst; a longer one runs under the power
        # cap like the seconds-long loop the sustained figure was taken from
        long_run = dt > 0.25
        tflops_peak = tflops_sustained if long_run else tflops_burst
        work = wl["flops"] / 1e3 if is_flops else wl["alg_bytes"]   # per step, in units of 1e-9 * unit
        per_gpu = work * args.steps / dt / 1e9
        unit = "TFLOP/s" if is_flops else "GB/s"
        line = {
            "metric": ("fp16 GEMM TFLOP/s" if is_flops else "achieved GB/s (algorithmic bytes / time)"),
            "value": per_gpu * world,
            "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": wl.get("scaling", "weak"),
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": wl["desc"], "l2": wl["l2"],
                       "launch": ("CUDA graph of one ring period" if (wl.get("graph_period") and not args.no_graph)
                                  else "one host launch per step"),
                       "sharding": f"{world} x the per-GPU workload, rows sharded, no collective"},
            "roofline": {"bound": "tensor" if is_flops else "hbm", "achieved": per_gpu,
                         "peak": tflops_peak if is_flops else hbm, "unit": unit,
                         "frac": per_gpu / (tflops_peak if is_flops else hbm),
                         "traffic": wl.get("traffic"),
                         "peak_source": which + ((" (bf16 cuBLAS, sustained: timed region > 0.25 s)"
                                                  if long_run else " (bf16 cuBLAS, burst)")
                                                 if is_flops else " (copy)")},
            "gpu_launches": wl["launches"] * args.steps,
            "clocks": clocks,
        }
        if is_flops:
            line["roofline"]["frac_of_burst"] = per_gpu / tflops_burst
            line["roofline"]["frac_of_sustained"] = per_gpu / tflops_sustained
        if e2e_dt is not None:
            line["e2e"] = {"value": work / e2e_dt / 1e9 * world, "unit": unit,
                           "h2d_bytes_per_step": wl["h2d"], "d2h_bytes_per_step": wl["d2h"],
                           "ms_per_step": e2e_dt * 1e3}
        if not args.no_cpu_baseline and world == 1:
            use_all_host_threads()
            med, n = time_cpu(wl["cpu_step"])
            scale = wl.get("cpu_scale", 1.0)
            cpu_work = wl["cpu_flops"] / 1e3 if "cpu_flops" in wl else work / scale
            line["cpu_baseline"] = {"value": cpu_work / med / 1e9, "unit": unit,
                                    "cores": torch.get_num_threads(),
                                    "kind": wl.get("cpu_kind", "port"),
                                    "sample": f"{wl['sample']}; median of {n} runs; "
                                              "torch CPU eager / C oracle on the host cores"}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
