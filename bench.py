#!/usr/bin/env python
"""Benchmark of the hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME|all] [--impl reference]

One JSON line.  Its top-level fields describe the headline workload ("fused"):
y = exp(x*a + b).sum(-1), x fp16 [8192, 8192] N(0,1), a and b fp16 [8192] U(-1,1), one fused
kernel per step over inputs resident in HBM as stick images.  With the default `--workload all`
the line also carries a "configs" object with the same measurements for every other benchmark
configuration: softmax [256, 4096] and scaled along the rows, the stick relayout of
[64, 2048, 4096] with contiguous and permuted host strides, bmm [32, 2048, 4096] x
[32, 4096, 4096], and the Llama-style decoder layer (hand-written module and the unmodified
transformers module) through torch.compile on spyre.

Timing: a timed region is exactly K steps between two CUDA events on the launching stream; the
region is repeated until at least 50 ms of device time have been measured and the median region
gives ms_per_step.  Every workload is checked against the CPU oracle before it is timed.

Under torchrun every rank takes its shard (torch_spyre.sharding.shard_rows) of each workload:
the headline workload is weak-scaled (the global problem is N x 8192 rows, one 8192-row shard
per rank; the stated 8192 x 8192 problem split N ways is reported beside it as "strong"), the
others split their stated leading dim over the ranks.  No collective touches the data.
"""
from __future__ import annotations

import argparse
import gc
import json
import math
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
MIN_TIMED_S = 0.050
HEADLINE = "fused"
OTHER_CONFIGS = ("softmax", "softmax_scaled", "relayout", "relayout_permuted", "bmm", "llama_layer",
                 "hf_llama_layer")
SEQ_OVERRIDE = None      # --seq: sequence length of the attention workload (profiling aid: an odd number of
                         # 128-row tiles runs the one-tile kernel)
EXTRA_WORKLOADS = ("pointwise", "attention", "restickify")      # not part of the default line


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return (p.get("hbm_gbs", 6650.0), p.get("bf16_tflops", 1590.0),
                p.get("bf16_tflops_sustained", 1400.0), "measured")
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""

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
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def mark(self) -> float:
        return time.perf_counter()

    def summary(self, t0: float, t1: float):
        """Median SM clock and the throttle reasons seen between two marks."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, s in self.samples:
            if t < t0 or t > t1 + 0.06:
                continue
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

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


# --------------------------------------------------------------------------- CPU side

def shard(total: int, rank: int, world: int) -> int:
    """Extent of this rank's contiguous block of `total` leading indices."""
    from torch_spyre.sharding import shard_rows
    lo, hi = shard_rows(total, rank, world)
    return hi - lo


def cpu_side(name: str, rank: int = 0, world: int = 1, rows=None, strong: bool = False):
    """Everything about a workload that needs no GPU: seeded host inputs (this rank's shard),
    the CPU implementation the reference's tests hold the device to (torch CPU eager; the C
    oracle for the relayout) on a bounded sample, and the algorithmic work of one step.
    Used by the reference arm, by the cpu_baseline leg and by the GPU side for its inputs."""
    from oracle import math_ref

    if name == "fused":
        cols = 8192
        nrows = rows or (shard(8192, rank, world) if strong else 8192)
        # weak: rank r holds rows [r*8192, (r+1)*8192) of the global [world*8192, 8192] problem
        x, a, b = math_ref.fused_inputs(nrows, cols, seed=0)       # a, b: the same columns on every rank
        if not strong and rank:
            x = torch.randn(nrows, cols, generator=math_ref.gen(1000 + rank)).half()
        work = nrows * cols * 2 + cols * 2 * 2 + nrows * 2
        return dict(host=(x, a, b), cpu_step=lambda: math_ref.fused_ref(x, a, b), work=work,
                    cpu_work=work, unit="GB/s", scaling="strong" if strong else "weak",
                    desc=f"exp(x*a+b).sum(-1), x fp16 [{nrows},{cols}] (BASELINE configs[1])",
                    sample=f"full [{nrows},{cols}] graph per CPU step",
                    sharding=("rows of the stated [8192,8192] problem split over the ranks" if strong else
                              "global problem [N*8192, 8192], one 8192-row shard per rank") + ", no collective")
    if name == "pointwise":
        nrows = cols = 8192
        x, a, b = math_ref.fused_inputs(nrows, cols)
        work = 2 * nrows * cols * 2 + cols * 2
        return dict(host=(x, b), cpu_step=lambda: x + b, work=work, cpu_work=work, unit="GB/s",
                    scaling="weak", desc=f"pointwise x + b (b broadcast along rows), fp16 [{nrows},{cols}]",
                    sample="full [8192,8192] add per CPU step",
                    sharding="every rank runs its own [8192,8192] block, no collective")
    if name in ("softmax", "softmax_scaled"):
        cols = 4096
        if name == "softmax":
            nrows, scaling = 256, "weak"
        else:
            nrows, scaling = rows or shard(65536, rank, world), "strong"
        x = math_ref.softmax_inputs(256, cols, seed=rank)
        if nrows != 256:
            x = x.repeat(-(-nrows // 256), 1)[:nrows].contiguous()
        work = 2 * nrows * cols * 2
        return dict(host=(x,), cpu_step=lambda: torch.softmax(x, -1), work=work, cpu_work=work,
                    unit="GB/s", scaling=scaling,
                    desc=f"softmax(dim=-1) fp16 [{nrows},{cols}]" +
                         (" (BASELINE configs[0])" if name == "softmax" else " (configs[0] scaled along rows)"),
                    sample=f"full [{nrows},{cols}] softmax per CPU step",
                    sharding=("every rank runs its own [256,4096] block" if name == "softmax" else
                              "the 65536 rows split over the ranks") + ", no collective")
    if name in ("relayout", "relayout_permuted"):
        import numpy as np
        from oracle import layout as OL, relayout_c as OC
        permuted = name.endswith("permuted")
        outer = rows or shard(64, rank, world)
        shape = (outer, 2048, 4096)
        # a seeded [4, ...] block repeated along dim 0 keeps host generation quick
        blk = math_ref.relayout_inputs((4,) + shape[1:], rank, permuted=False)
        host = blk.repeat(-(-outer // 4), 1, 1)[:outer].contiguous()
        if permuted:
            host = host.permute(0, 2, 1).contiguous().permute(0, 2, 1)
        nbytes = host.numel() * 2
        sample_outer = min(outer, 8)
        h = host[:sample_outer].view(torch.int16).numpy().view(np.uint16)
        lay = OL.generic_stick_layout(h.shape)
        nt = usable_threads()

        def cpu_step():
            return OC.from_sticks(OC.to_sticks(h, lay, nthreads=nt), lay, h.shape, nthreads=nt)

        return dict(host=(host,), cpu_step=cpu_step, work=4 * nbytes, cpu_work=4 * nbytes * sample_outer / outer,
                    unit="GB/s", scaling="strong", cpu_kind="port",
                    desc=f"stick relayout fp16 {list(shape)} host strides {list(host.stride())}, "
                         "to sticks and back (BASELINE configs[2])",
                    sample=f"C oracle on a [{sample_outer},2048,4096] slice, all host threads",
                    sharding="the outer 64 split over the ranks, no collective")
    if name == "bmm":
        batch, m, k, n = rows or shard(32, rank, world), 2048, 4096, 4096
        a1, b1 = math_ref.bmm_inputs(batch=1, seed=rank)
        flops = 2.0 * batch * m * k * n
        return dict(host=(a1, b1), batch=batch, cpu_step=lambda: torch.bmm(a1, b1), work=flops,
                    cpu_work=flops / batch, unit="TFLOP/s", scaling="strong",
                    desc=f"bmm fp16 [{batch},{m},{k}] x [{batch},{k},{n}], fp32 accumulate "
                         "(BASELINE configs[3])",
                    sample="one batch entry [1,2048,4096]x[1,4096,4096] per CPU step",
                    sharding="the batch of 32 split over the ranks, no collective")
    if name in ("llama_layer", "hf_llama_layer"):
        from oracle import llama_ref as LR
        cfg = LR.LayerConfig()
        batch, seq = rows or shard(8, rank, world), 2048
        w = LR.make_weights(cfg)
        x1 = torch.randn(1, seq, cfg.d_model, generator=torch.Generator().manual_seed(rank)).half()
        cpu_seq = 256
        return dict(host=(x1,), weights=w, cfg=cfg, batch=batch, seq=seq,
                    cpu_step=lambda: LR.layer_forward(x1[:, :cpu_seq], w, cfg),
                    work=LR.layer_flops(batch, seq, cfg, causal=True),
                    cpu_work=LR.layer_flops(1, cpu_seq, cfg, causal=True), unit="TFLOP/s",
                    scaling="strong",
                    desc=("transformers LlamaDecoderLayer (unmodified)" if name == "hf_llama_layer"
                          else "Llama-style decoder layer") +
                         " through torch.compile on spyre: d_model 4096, 32 heads x 128, "
                         f"SwiGLU 11008, RMSNorm, rotary, causal attention, batch {batch} x seq {seq} per GPU, "
                         "causal-useful flops (BASELINE configs[4])",
                    sample=f"oracle layer (torch CPU eager fp16) on [1, {cpu_seq}, 4096] per CPU step",
                    sharding="the batch of 8 split over the ranks, weights replicated, no collective")
    if name == "attention":
        from oracle import llama_ref as LR
        batch, seq, heads, hd = rows or shard(8, rank, world), SEQ_OVERRIDE or 2048, 32, 128
        g = torch.Generator().manual_seed(rank)
        q, k, v = (torch.randn(batch, seq, heads * hd, generator=g).half() for _ in range(3))
        scale = 1.0 / math.sqrt(hd)
        flops = 4.0 * batch * heads * hd * (seq * (seq + 1) / 2)   # causal-useful: keys <= query
        nh = 4

        def cpu_step():
            return LR.attention_forward(q[:1, :, :nh * hd], k[:1, :, :nh * hd], v[:1, :, :nh * hd], nh, scale)

        return dict(host=(q, k, v), batch=batch, seq=seq, heads=heads, scale=scale, cpu_step=cpu_step,
                    cpu_heads=nh, work=flops, cpu_work=flops / (batch * heads / nh), unit="TFLOP/s",
                    scaling="strong",
                    desc=f"causal attention fp16, batch {batch} x seq {seq} x {heads} heads x {hd}, "
                         "causal-useful flops (the attention block of BASELINE configs[4])",
                    sample="torch CPU eager attention (fp16 matmuls, fp32 softmax) on 1 batch entry x 4 heads",
                    sharding="the batch of 8 split over the ranks, no collective")
    if name == "restickify":
        outer = rows or shard(64, rank, world)
        bits = torch.randint(-32768, 32768, (1, 2048, 4096), dtype=torch.int16,
                             generator=torch.Generator().manual_seed(7 + rank))
        host = bits.view(torch.float16).repeat(outer, 1, 1)
        nbytes = host.numel() * 2

        def cpu_step():
            return host[:4].transpose(1, 2).contiguous()

        return dict(host=(host,), cpu_step=cpu_step, work=2 * nbytes, cpu_work=2 * nbytes * 4 / outer, unit="GB/s",
                    scaling="strong",
                    desc=f"device-side restickify: fp16 [{outer}, 2048, 4096] spyre tensor, .transpose(1, 2).contiguous() "
                         "(stick image to stick image in one pass)",
                    sample="torch CPU x.transpose(1, 2).contiguous() on 4 outer entries",
                    sharding="the outer 64 split over the ranks, no collective")
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------- GPU side

def gpu_side(name: str, dev, cpu: dict):
    """Adds the device legs to a workload: step_dev (inputs resident in HBM), step_e2e (host
    buffers in, host result out, through the public API), check (parity before timing)."""
    from oracle import math_ref
    from torch_spyre import stick_ops as K

    wl = dict(cpu)
    if name == "fused":
        x, a, b = cpu["host"]
        rows, cols = x.shape
        xp, ap, bp = x.pin_memory(), a.pin_memory(), b.pin_memory()
        ring = max(2, -(-2 * L2_BYTES // (rows * cols * 2)) + 1)  # ring of x buffers > 2x L2
        sa, sb = K.copy_host_to_sticks(ap), K.copy_host_to_sticks(bp)
        xs = [K.copy_host_to_sticks(xp)]
        for _ in range(ring - 1):
            xs.append(K.StickTensor(xs[0].image.clone(), xs[0].shape))

        def chain_on(sx):
            c = K.Chain()
            c.emit("LOAD", c.tensor(sx)).emit("MUL", c.tensor(sa)).emit("ADD", c.tensor(sb)).emit("EXP")
            return c

        launches = [K.prepare_chain(chain_on(sx), (rows, cols), n_outputs=0, reduce="sum")[0] for sx in xs]
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
            # pinned host tensors, so the copies may be queued without waiting for each one
            return compiled(xp.to(spyre_dev, non_blocking=True), ap.to(spyre_dev, non_blocking=True),
                            bp.to(spyre_dev, non_blocking=True)).cpu()

        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=1,
                  h2d=rows * cols * 2 + 2 * cols * 2, d2h=rows * 2, graph_period=ring,
                  # ncu, one launch at [8192,8192]: 134,263,296 B read + 3,333,632 B written
                  traffic=int(137596928 * rows / 8192) if cols == 8192 else None,
                  l2=f"ring of {ring} x buffers ({ring * rows * cols * 2 >> 20} MiB) > L2",
                  check=lambda: math_ref.assert_close(step_e2e().clone(), cpu["cpu_step"]()))
        return wl

    if name == "pointwise":
        x, b = cpu["host"]
        rows, cols = x.shape
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

        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=1, h2d=rows * cols * 2,
                  d2h=rows * cols * 2, graph_period=ring,
                  # ncu, one launch at this size: 134,248,704 B read + 77,152,000 B written
                  # (the rest of the output was still in L2 when the kernel ended)
                  traffic=211400704,
                  l2=f"ring of {ring} input and output buffers ({2 * ring * rows * cols * 2 >> 20} MiB) > L2",
                  check=lambda: math_ref.assert_close(step_e2e().clone(), cpu["cpu_step"]()))
        return wl

    if name in ("softmax", "softmax_scaled"):
        (x,) = cpu["host"]
        rows, cols = x.shape
        xp = x.pin_memory()
        ring = min(max(2, -(-2 * L2_BYTES // (rows * cols * 2)) + 1), 160)
        xs = [K.copy_host_to_sticks(xp)]
        for _ in range(ring - 1):
            xs.append(K.StickTensor(xs[0].image.clone(), xs[0].shape))
        outs = [K.empty((rows, cols)) for _ in range(min(ring, 4) if rows > 256 else ring)]
        state = {"i": 0}

        def step_dev():
            i = state["i"]
            state["i"] += 1
            K.softmax_rows(xs[i % ring], out=outs[i % len(outs)])

        import torch_spyre  # noqa: F401
        spyre_dev = torch.device("spyre", dev.index)

        y_host = torch.empty(rows, cols, dtype=torch.float16).pin_memory()

        def step_e2e():
            # the calls a user makes: pinned host tensor -> spyre -> eager softmax -> pinned host tensor
            return y_host.copy_(torch.softmax(xp.to(spyre_dev, non_blocking=True), -1))

        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=1, h2d=rows * cols * 2,
                  d2h=rows * cols * 2, graph_period=ring if rows == 256 else 0,
                  # ncu at [16384, 4096]: 134,235,648 B read + 79,373,312 B written (part of the
                  # output still in L2), scaled by rows
                  traffic=int(213608960 * rows / 16384),
                  l2=f"ring of {ring} input buffers ({ring * rows * cols * 2 >> 20} MiB) > L2",
                  check=lambda: math_ref.assert_close(step_e2e().clone(), cpu["cpu_step"]()))
        return wl

    if name in ("relayout", "relayout_permuted"):
        (host,) = cpu["host"]
        permuted = name.endswith("permuted")
        shape = tuple(host.shape)
        hp = host.pin_memory()
        raw = hp.to(dev, non_blocking=True)
        assert raw.stride() == host.stride()
        st = K.to_sticks(raw)
        back = torch.empty_strided(shape, host.stride(), dtype=host.dtype, device=dev)

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
            import numpy as np
            from oracle import layout as OL, relayout_c as OC
            if not torch.equal(step_e2e().view(torch.int16), host.view(torch.int16)):
                raise AssertionError("relayout round trip is not the identity")
            step_dev()
            torch.cuda.synchronize()
            if not torch.equal(back.view(torch.int16).cpu(), host.view(torch.int16)):
                raise AssertionError("device-side relayout round trip is not the identity")
            # the image of the first slice against the C oracle, bit for bit
            h = host[:1].view(torch.int16).numpy().view(np.uint16)
            one = K.to_sticks(raw[:1])
            want = OC.to_sticks(h, OL.generic_stick_layout(h.shape), nthreads=usable_threads())
            got = one.image.view(torch.int16).cpu().numpy().view(np.uint16)
            if not np.array_equal(got, want):
                raise AssertionError("stick image differs from the oracle")

        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=2, h2d=nbytes, d2h=nbytes,
                  # ncu at [16, 2048, 4096], one direction: 268.45 MB read + 213.6 MB written
                  # (contiguous) / 213.3 MB (permuted), scaled by the outer extent
                  traffic=int((482078208 if not permuted else 481772544) * shape[0] / 16),
                  l2=f"{nbytes >> 20} MiB tensors, far larger than L2", check=check)
        return wl

    if name == "restickify":
        import torch_spyre  # noqa: F401
        (host,) = cpu["host"]
        sdev = torch.device("spyre", dev.index)
        hp = host.pin_memory()
        xs = hp.to(sdev)

        def step_dev():
            return xs.transpose(1, 2).contiguous()

        out_host = torch.empty(host.shape[0], host.shape[2], host.shape[1], dtype=torch.float16).pin_memory()

        def step_e2e():
            return out_host.copy_(hp.to(sdev).transpose(1, 2).contiguous())

        def check():
            got = step_dev()
            if not torch.equal(got[-1].cpu().view(torch.int16), host[-1].transpose(0, 1).contiguous().view(torch.int16)):
                raise AssertionError("restickified transpose differs from the host transpose")

        nbytes = host.numel() * 2
        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=1, h2d=nbytes, d2h=nbytes, traffic=None,
                  l2=f"{nbytes >> 20} MiB tensor, far larger than L2", check=check)
        return wl

    if name == "bmm":
        a1, b1 = cpu["host"]
        batch, (m, k), n = cpu["batch"], a1.shape[1:], b1.shape[2]
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

        def check():
            got = step_e2e()[batch - 1, :256].clone()
            math_ref.assert_close(got, torch.bmm(a1[:, :256], b1)[0])
            if K._abi.lib().ts_gemm_error_state() != 0:
                raise AssertionError("GEMM kernel gave up on an internal wait")

        def library_gemm(steps, warmup, sampler):
            """cuBLAS (torch.bmm) on the same shape in the same process, timed the same way: a
            yardstick beside the kernel's own figure, not part of any product path."""
            la = torch.randn(batch, m, k, device=dev, dtype=torch.float16)
            lb = torch.randn(batch, k, n, device=dev, dtype=torch.float16)
            lc = torch.empty(batch, m, n, device=dev, dtype=torch.float16)
            t_end = time.perf_counter() + 0.3
            while time.perf_counter() < t_end:
                torch.bmm(la, lb, out=lc)
                torch.cuda.synchronize()
            t0 = sampler.mark() if sampler else 0.0
            regions = time_device(lambda: torch.bmm(la, lb, out=lc), steps, warmup, 0)
            t1 = sampler.mark() if sampler else 0.0
            dt = median(regions) / steps
            out = {"what": "torch.bmm fp16 (cuBLAS), same shape, same process", "ms_per_step": dt * 1e3,
                   "value": cpu["work"] / dt / 1e12, "unit": "TFLOP/s"}
            if sampler:
                clk = sampler.summary(t0, t1)
                out["sm_mhz"] = clk.get("sm_mhz")
                if clk.get("sm_mhz"):
                    out["tflops_per_ghz"] = out["value"] / (clk["sm_mhz"] / 1e3)
            return out

        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=1, library_gemm=library_gemm,
                  h2d=(ah.numel() + bh.numel()) * 2, d2h=ch.numel() * 2,
                  # ncu at batch 8: 577,565,440 B read + 119,217,664 B written, scaled by batch
                  traffic=int(696783104 * batch / 8),
                  l2=f"operands {(ah.numel() + bh.numel()) * 2 >> 20} MiB, far larger than L2", check=check)
        return wl

    if name in ("llama_layer", "hf_llama_layer"):
        import torch_spyre  # noqa: F401
        from oracle import llama_ref as LR
        cfg, w, batch, seq = cpu["cfg"], cpu["weights"], cpu["batch"], cpu["seq"]
        (x1,) = cpu["host"]
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
        xh = x1.repeat(batch, 1, 1).pin_memory()
        xd = xh.to(sdev)
        compiled(xd)  # compile once, outside every timed region

        def step_dev():
            compiled(xd)

        yh = torch.empty_like(xh).pin_memory()

        def step_e2e():
            return yh.copy_(compiled(xh.to(sdev)))

        def check():
            # causal: a prefix depends on itself only.  A 4096-wide layer is ~10 fp16 roundings
            # deep with sums over up to 11008 terms, so two correct fp16 evaluations differ by a
            # few fp16 ulps of the residual stream; both are therefore measured against an fp32
            # evaluation of the same inputs, and the device may not be further from it than 1.5 x
            # what torch CPU fp16 eager is.
            n = 64
            got = step_e2e()[batch - 1, :n]
            cpu16 = LR.layer_forward(x1[:, :n], w, cfg)[0]
            truth = LR.layer_forward_fp32(x1[:, :n], w, cfg)[0]
            wl["parity_detail"] = math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, what=name)
            if K._abi.lib().ts_gemm_error_state() != 0 or K._abi.lib().ts_attention_error_state() != 0:
                raise AssertionError("a tensor-core kernel gave up on an internal wait")

        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=11, h2d=xh.numel() * 2,
                  d2h=xh.numel() * 2, traffic=None,
                  l2="activations and weights (> 1 GiB) far larger than L2", check=check)
        return wl

    if name == "attention":
        from oracle import llama_ref as LR
        q, k, v = (t.pin_memory() for t in cpu["host"])
        batch, seq, heads, scale, hd = cpu["batch"], cpu["seq"], cpu["heads"], cpu["scale"], 128
        qs, ks, vs = (K.copy_host_to_sticks(t) for t in (q, k, v))
        out = K.empty((batch, seq, heads * hd), torch.float16, dev)
        out_host = torch.empty_like(q).pin_memory()

        def step_dev():
            K.causal_attention(qs, ks, vs, batch, seq, heads, scale, out=out)

        def step_e2e():
            q2, k2, v2 = (K.copy_host_to_sticks(t) for t in (q, k, v))
            o = K.causal_attention(q2, k2, v2, batch, seq, heads, scale)
            K.copy_sticks_to_host(o, out_host)
            torch.cuda.synchronize()
            return out_host

        def check():
            nh = cpu["cpu_heads"]
            sl = [t[:1, :, :nh * hd] for t in (q, k, v)]
            got = step_e2e()[:1, :, :nh * hd]
            cpu16 = LR.attention_forward(*sl, nh, scale)
            truth = LR.attention_forward(*[t.float() for t in sl], nh, scale)
            math_ref.assert_close(got, truth.half(), atol=2e-3)
            wl["parity_detail"] = math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, what=name)
            if K._abi.lib().ts_attention_error_state() != 0:
                raise AssertionError("attention kernel gave up on an internal wait")

        wl.update(step_dev=step_dev, step_e2e=step_e2e, launches=1, h2d=3 * q.numel() * 2,
                  d2h=q.numel() * 2, traffic=None, l2="q, k, v, out 512 MiB, larger than L2", check=check)
        return wl
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------- timing

def time_device(step, steps, warmup, graph_period=0, min_total_s=MIN_TIMED_S, max_regions=400):
    """Times regions of exactly `steps` calls of `step` with CUDA events on the launching stream,
    repeating the region until `min_total_s` of device time has been measured.  Returns the list
    of region times in seconds.  When the workload's steps repeat with period `graph_period` (a
    ring of buffers larger than L2), regions are replayed from CUDA graphs so that host launch
    overhead stays out of a microsecond-scale kernel's timing: each graph holds `steps`
    consecutive steps, and there are enough graphs to walk the whole ring before a buffer is
    touched again, so every launch still reads its input from HBM."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    graphs = []
    if graph_period:
        n_graphs = max(1, min(-(-graph_period // steps), 64)) if steps < graph_period else 1
        if steps >= graph_period and steps % graph_period:
            n_graphs = graph_period     # every ring offset gets its own graph
        n_graphs = min(n_graphs, 64)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            for _ in range(n_graphs):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for _ in range(steps):
                        step()
                graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        for g in graphs:
            g.replay()
        torch.cuda.synchronize()
    regions, total = [], 0.0
    while total < min_total_s and len(regions) < max_regions:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        if graphs:
            graphs[len(regions) % len(graphs)].replay()
        else:
            for _ in range(steps):
                step()
        end.record()
        torch.cuda.synchronize()
        regions.append(start.elapsed_time(end) / 1e3)
        total += regions[-1]
    return regions


def median(values):
    v = sorted(values)
    return v[len(v) // 2]


def usable_threads() -> int:
    try:
        return max(len(os.sched_getaffinity(0)), 1)
    except AttributeError:
        return os.cpu_count() or 1


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs are meant to use every host
    core this process may run on."""
    torch.set_num_threads(usable_threads())
    return torch.get_num_threads()


def time_cpu(fn, budget_s, min_runs=2):
    fn()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_runs or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
        if len(times) >= 200:
            break
    return median(times), len(times)


def unit_scale(unit: str) -> float:
    return 1e12 if unit == "TFLOP/s" else 1e9


def metric_name(unit: str) -> str:
    return "fp16 GEMM TFLOP/s" if unit == "TFLOP/s" else "achieved GB/s (algorithmic bytes / time)"


def launch_mode(wl, no_graph=False) -> str:
    return ("CUDA graphs of K steps each, together walking the ring of buffers" if (wl.get("graph_period") and not no_graph)
            else "one host launch per step")


# --------------------------------------------------------------------------- reference arm

def reference_entry(name, steps, warmup, budget_s=None):
    """Times the CPU implementation of one workload: `steps` steps after `warmup`, or as many as
    fit `budget_s`."""
    cpu = cpu_side(name)
    cpu["cpu_step"]()
    for _ in range(max(warmup - 1, 0)):
        cpu["cpu_step"]()
    if budget_s is None:
        t0 = time.perf_counter()
        for _ in range(steps):
            cpu["cpu_step"]()
        dt, n = (time.perf_counter() - t0) / steps, steps
    else:
        dt, n = time_cpu(cpu["cpu_step"], budget_s)
    value = cpu["cpu_work"] / dt / unit_scale(cpu["unit"])
    return cpu, {"value": value, "unit": cpu["unit"], "ms_per_step": dt * 1e3 * cpu["work"] / cpu["cpu_work"],
                 "sample": cpu["sample"], "cpu_steps": n,
                 "cpu_baseline": {"value": value, "unit": cpu["unit"], "cores": torch.get_num_threads(),
                                  "kind": cpu.get("cpu_kind", "port"), "sample": cpu["sample"]}}


def run_reference(args, rank, world):
    """Reference arm: the path's CPU implementation (torch CPU eager, which is what the
    reference's tests hold the device to; the C oracle for the relayout) on the host cores.  The
    reference itself cannot be installed: its arithmetic lives in closed libraries."""
    if rank != 0:
        return
    use_all_host_threads()
    head = HEADLINE if args.workload == "all" else args.workload
    cpu, r = reference_entry(head, args.steps, args.warmup)
    line = {"impl": "reference", "metric": metric_name(cpu["unit"]), "value": r["value"],
            "unit": cpu["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": cpu["scaling"],
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_block(cpu, None, args),
            "cpu_baseline": dict(r["cpu_baseline"], sample=cpu["sample"] + "; torch CPU eager / C oracle on host cores"),
            "e2e": {"value": r["value"], "unit": cpu["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if args.workload == "all":
        line["configs"] = {}
        for name in OTHER_CONFIGS:
            _, rr = reference_entry(name, 2, 1, budget_s=args.cpu_budget)
            line["configs"][name] = rr
            gc.collect()
    print(json.dumps(line))


def config_block(wl, gpu_wl, args):
    """The `config` object: identical keys and values on both arms."""
    head = HEADLINE if args.workload == "all" else args.workload
    graph = head in ("fused", "pointwise", "softmax") and not args.no_graph
    return {"workload": wl["desc"],
            "l2": "inputs larger than L2 (ring of buffers where one input is smaller)",
            "launch": "CUDA graphs of K steps each, together walking the ring of buffers" if graph else "one host launch per step",
            "sharding": wl["sharding"]}


# --------------------------------------------------------------------------- the b200 arm

class Runner:
    def __init__(self, args, rank, world, local, dev, dist):
        self.args, self.rank, self.world, self.local, self.dev, self.dist = args, rank, world, local, dev, dist
        self.sampler = ClockSampler(local).start() if rank == 0 else None
        self.peaks = measured_peaks()

    def barrier(self):
        if self.dist is not None:
            # an all-reduce of a CUDA tensor: dist.barrier() resolves its device through the process's
            # accelerator type, which is spyre once the backend is loaded, and NCCL serves cuda tensors
            self._token = getattr(self, "_token", None)
            if self._token is None:
                self._token = torch.zeros(1, device=self.dev)
            self.dist.all_reduce(self._token)
        torch.cuda.synchronize()

    def max_over_ranks(self, *values):
        if self.dist is None:
            return values
        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return tuple(float(v) for v in t)

    def sum_over_ranks(self, value):
        if self.dist is None:
            return value
        t = torch.tensor([value], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t[0])

    def measure(self, name, strong=False, cpu_budget=None, e2e=True):
        """Builds, checks and times one workload; returns its result object (on every rank)."""
        args = self.args
        cpu = cpu_side(name, self.rank, self.world, args.rows, strong=strong)
        wl = gpu_side(name, self.dev, cpu)
        wl["check"]()  # parity of one step against the CPU oracle before timing anything
        self.barrier()
        # keep the device busy long enough for the clock sampler to see it under load
        t_end = time.perf_counter() + 0.3
        while time.perf_counter() < t_end:
            for _ in range(4):
                wl["step_dev"]()
            torch.cuda.synchronize()
        self.barrier()
        t0 = self.sampler.mark() if self.sampler else 0.0
        regions = time_device(wl["step_dev"], args.steps, args.warmup,
                              0 if args.no_graph else wl.get("graph_period", 0))
        t1 = self.sampler.mark() if self.sampler else 0.0
        self.barrier()
        dt = median(regions) / args.steps

        e2e_dt = None
        if e2e:
            for _ in range(3):
                wl["step_e2e"]()
            self.barrier()
            times = []
            while len(times) < 3 or (sum(times) < MIN_TIMED_S and len(times) < 50):
                t_start = time.perf_counter()
                wl["step_e2e"]()
                torch.cuda.synchronize()
                times.append(time.perf_counter() - t_start)
            e2e_dt = median(times)
        dt, e2e_dt_max = self.max_over_ranks(dt, e2e_dt or 0.0)
        total_work = self.sum_over_ranks(wl["work"])

        hbm, burst, sustained, which = self.peaks
        unit = wl["unit"]
        is_flops = unit == "TFLOP/s"
        per_gpu = wl["work"] / dt / unit_scale(unit)
        # a region of a fraction of a second is a burst; a longer one runs under the power cap
        # like the seconds-long loop the sustained figure was taken from
        long_run = sum(regions) > 0.25
        peak = (sustained if long_run else burst) if is_flops else hbm
        res = {"value": total_work / dt / unit_scale(unit), "unit": unit, "ms_per_step": dt * 1e3,
               "timed": {"regions": len(regions), "steps_per_region": args.steps,
                         "device_ms_total": sum(regions) * 1e3, "statistic": "median region / steps"},
               "scaling": wl["scaling"], "workload": wl["desc"], "l2": wl["l2"],
               "launch": launch_mode(wl, args.no_graph), "sharding": wl["sharding"],
               "roofline": {"bound": "tensor" if is_flops else "hbm", "achieved": per_gpu, "peak": peak,
                            "unit": unit, "frac": per_gpu / peak, "traffic": wl.get("traffic"),
                            "peak_source": which + ((" (bf16 cuBLAS, sustained: timed > 0.25 s)" if long_run
                                                     else " (bf16 cuBLAS, burst)") if is_flops else " (copy)")},
               "gpu_launches": wl["launches"] * args.steps * len(regions),
               "parity": "ok"}
        if "parity_detail" in wl:
            res["parity_detail"] = wl["parity_detail"]
        if "library_gemm" in wl and self.world == 1:
            lib = wl["library_gemm"](args.steps, args.warmup, self.sampler)
            lib["ratio_ours_to_library"] = per_gpu / lib["value"]
            res["library_gemm"] = lib
        if is_flops:
            res["roofline"]["frac_of_burst"] = per_gpu / burst
            res["roofline"]["frac_of_sustained"] = per_gpu / sustained
        if self.sampler:
            res["clocks"] = self.sampler.summary(t0, t1)
            if is_flops and res["clocks"].get("sm_mhz"):
                res["roofline"]["tflops_per_ghz"] = per_gpu / (res["clocks"]["sm_mhz"] / 1e3)
        if e2e_dt is not None:
            res["e2e"] = {"value": total_work / e2e_dt_max / unit_scale(unit), "unit": unit,
                          "h2d_bytes_per_step": wl["h2d"], "d2h_bytes_per_step": wl["d2h"],
                          "ms_per_step": e2e_dt_max * 1e3,
                          "h2d_gbs_per_rank": (wl["h2d"] + wl["d2h"]) / e2e_dt_max / 1e9}
        if cpu_budget and self.world == 1 and self.rank == 0:
            use_all_host_threads()
            med, n = time_cpu(wl["cpu_step"], cpu_budget)
            res["cpu_baseline"] = {"value": wl["cpu_work"] / med / unit_scale(unit), "unit": unit,
                                   "cores": torch.get_num_threads(), "kind": wl.get("cpu_kind", "port"),
                                   "sample": f"{wl['sample']}; median of {n} runs; "
                                             "torch CPU eager / C oracle on the host cores"}
        res["_wl"] = wl
        return res


def host_overheads(dev):
    """Host time per launch, in microseconds, of each way into the library: a prepared C-ABI launch
    (ctypes), one eager op on spyre tensors, and a compiled one-kernel graph by either compile
    route.  Tiny tensors, many calls, one synchronize at the end: the device is never the limit."""
    import torch_spyre  # noqa: F401
    from torch_spyre import stick_ops as K
    from torch_spyre._inductor import compiler

    sdev = torch.device("spyre", dev.index)
    g = torch.Generator().manual_seed(5)
    x, a, b = (torch.randn(64, 128, generator=g).half(), torch.rand(128, generator=g).half(),
               torch.rand(128, generator=g).half())
    xs, as_, bs = x.to(sdev), a.to(sdev), b.to(sdev)

    def per_call(fn, n=300):
        for _ in range(20):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        host = time.perf_counter() - t0
        torch.cuda.synchronize()
        return host / n * 1e6

    sx, sa, sb = K.copy_host_to_sticks(x), K.copy_host_to_sticks(a), K.copy_host_to_sticks(b)
    c = K.Chain()
    c.emit("LOAD", c.tensor(sx)).emit("MUL", c.tensor(sa)).emit("ADD", c.tensor(sb)).emit("EXP")
    prepared = K.prepare_chain(c, (64, 128), n_outputs=0, reduce="sum")[0]
    out = {"c_abi_prepared_launch": per_call(prepared), "eager_op": per_call(lambda: torch.add(xs, xs))}
    fn = lambda t, u, v: torch.exp(t * u + v).sum(-1)      # noqa: E731
    before = compiler.backend_mode
    try:
        for mode in ("inductor", "plan"):
            compiler.backend_mode = mode
            torch._dynamo.reset()
            del compiler.last_routes[:]
            compiled = torch.compile(fn)
            compiled(xs, as_, bs)
            out[f"compiled_graph_{mode}"] = per_call(lambda: compiled(xs, as_, bs))
            if mode == "inductor":      # says so if the graph fell back to the plan
                out["compiled_graph_inductor_route"] = compiler.last_routes[-1] if compiler.last_routes else "plan"
    finally:
        compiler.backend_mode = before
        torch._dynamo.reset()
    out["unit"] = "us of host time per call (1 kernel launch each)"
    return out


def host_copy_rates(dev):
    """GB/s of the device's host copies for a [4096, 8192] fp16 tensor (64 MiB) through the public
    API: pinned and pageable sources, an existing pageable destination and the fresh one `.cpu()`
    returns.  Wall clock around blocking calls."""
    import torch_spyre  # noqa: F401

    sdev = torch.device("spyre", dev.index)
    x = torch.randn(4096, 8192, generator=torch.Generator().manual_seed(6)).half()
    xp, y = x.pin_memory(), torch.empty_like(x)
    yp = torch.empty_like(x).pin_memory()
    d = xp.to(sdev)
    gb = x.numel() * 2 / 1e9

    def rate(fn, n=3):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        torch.cuda.synchronize()
        return gb * n / (time.perf_counter() - t0)

    return {"pinned_to_device": rate(lambda: xp.to(sdev)), "pageable_to_device": rate(lambda: x.to(sdev)),
            "device_to_pinned": rate(lambda: yp.copy_(d)), "device_to_pageable": rate(lambda: y.copy_(d)),
            "device_to_fresh_cpu_tensor": rate(lambda: d.cpu()), "unit": "GB/s, [4096, 8192] fp16"}


def measure_tp(run):
    """config 5's layer as ONE layer split over the ranks (tensor parallel, sequence-parallel
    activations): each rank holds 1/N of every weight and of the rows, the two reduce-scatters run in
    the GEMM epilogues over NVLink peer memory, the two all-gathers are peer copies.  Every rank makes
    the same number of calls (the layer's barriers are collective), so the region count is agreed
    on before timing."""
    from oracle import llama_ref as LR, math_ref
    from torch_spyre import stick_ops as K
    from torch_spyre.tensor_parallel import TPDecoderLayer, TPGroup

    args, rank, world = run.args, run.rank, run.world
    cfg = LR.LayerConfig()
    batch, seq = 8, 2048
    w = LR.make_weights(cfg)
    x1 = torch.randn(1, seq, cfg.d_model, generator=torch.Generator().manual_seed(0)).half()
    cos, sin = LR.rope_tables(seq, cfg.head_dim)
    tp = TPGroup()
    layer = TPDecoderLayer(tp, w, cfg.heads, cfg.eps, cos, sin, batch, seq)
    rows = batch * seq // world
    x_all = x1.repeat(batch, 1, 1).reshape(batch * seq, cfg.d_model)
    mine = x_all[rank * rows:(rank + 1) * rows].contiguous().pin_memory()
    xs = K.copy_host_to_sticks(mine)
    y = layer(xs)
    y = layer(xs)
    torch.cuda.synchronize()
    detail = None
    if rank == 0:      # rank 0's first rows are a causal prefix of batch entry 0
        n = 64
        got = K.from_sticks(y).cpu()[:n]
        cpu16 = LR.layer_forward(x1[:, :n], w, cfg)[0]
        truth = LR.layer_forward_fp32(x1[:, :n], w, cfg)[0]
        detail = math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, factor=2.0, what="TP layer")
    if K._abi.lib().ts_gemm_error_state() != 0 or K._abi.lib().ts_attention_error_state() != 0:
        raise AssertionError("a tensor-core kernel gave up on an internal wait")
    run.barrier()

    def region():
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            layer(xs)
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / 1e3

    for _ in range(args.warmup):
        layer(xs)
    (first,) = run.max_over_ranks(region())
    n_regions = int(min(max(MIN_TIMED_S / first, 1.0), 50.0) + 0.999)
    t0 = run.sampler.mark() if run.sampler else 0.0
    regions = [region() for _ in range(n_regions)]
    t1 = run.sampler.mark() if run.sampler else 0.0
    run.barrier()
    (dt,) = run.max_over_ranks(median(regions) / args.steps)
    flops = LR.layer_flops(batch, seq, cfg, causal=True)
    hbm, burst, sustained, which = run.peaks
    per_gpu = flops / world / dt / 1e12
    # NVLink roofline: the slower of the layer's flops at the measured GEMM peak and the bytes a
    # rank must send at the measured 770 GB/s per direction
    link_s = layer.nvlink_bytes_per_call / 770e9
    res = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "ms_per_step": dt * 1e3, "scaling": "strong",
           "timed": {"regions": n_regions, "steps_per_region": args.steps, "device_ms_total": sum(regions) * 1e3,
                     "statistic": "median region / steps, max over ranks"},
           "workload": "Llama-style decoder layer, batch 8 x seq 2048, d_model 4096, 32 heads x 128, SwiGLU 11008, as one "
                       f"tensor-parallel layer over {world} GPUs (column-parallel q/k/v/gate/up, row-parallel o/down with the "
                       "reduce-scatter in the GEMM epilogue over NVLink peer memory, all-gathers by peer copies)",
           "sharding": "weights, heads and rows split over the ranks; 2 all-gathers + 2 reduce-scatters per layer",
           "nvlink_bytes_per_step_per_rank": layer.nvlink_bytes_per_call,
           "nvlink_gbs_per_rank": layer.nvlink_bytes_per_call / dt / 1e9,
           "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": burst, "unit": "TFLOP/s",
                        "frac": per_gpu / burst, "frac_of_sustained": per_gpu / sustained, "traffic": None,
                        "peak_source": which + " (bf16 cuBLAS, burst)",
                        "link_time_ms": link_s * 1e3, "link_frac_of_step": link_s / dt},
           "gpu_launches": 15 * args.steps * n_regions, "parity": "ok"}
    if detail:
        res["parity_detail"] = detail
    if run.sampler:
        res["clocks"] = run.sampler.summary(t0, t1)
    return res


def release():
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    try:
        torch._dynamo.reset()
    except Exception:
        pass


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="all",
                    help="all (headline + every other configuration), or one of: fused " +
                         " ".join(OTHER_CONFIGS + EXTRA_WORKLOADS) + "; tp_llama_layer under torchrun")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host")
    ap.add_argument("--cpu-budget", type=float, default=4.0,
                    help="seconds of CPU work per secondary configuration's baseline")
    ap.add_argument("--rows", type=int, default=None,
                    help="profiling aid: leading extent of the workload (rows / outer / batch)")
    ap.add_argument("--seq", type=int, default=None,
                    help="profiling aid: sequence length of the attention workload (default 2048)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global SEQ_OVERRIDE
    SEQ_OVERRIDE = args.seq

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
        dist.init_process_group("nccl")     # no device_id: with spyre registered it is the process's accelerator type, not cuda

    run = Runner(args, rank, world, local, dev, dist)
    if args.workload == "tp_llama_layer":      # the tensor-parallel layer alone (needs more than one rank)
        if world < 2 or 32 % world:
            raise SystemExit("tp_llama_layer runs under torchrun on 2, 4 or 8 ranks")
        r = measure_tp(run)
        if run.sampler:
            run.sampler.stop()
        if rank == 0:
            line = {"metric": metric_name(r["unit"]), "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                    "higher_is_better": True, "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                    "config": {"workload": r["workload"], "sharding": r["sharding"],
                               "l2": "activations and weights far larger than L2", "launch": "one host launch per step"}}
            line.update({k: v for k, v in r.items() if k not in ("workload", "sharding")})
            print(json.dumps(line))
        dist.destroy_process_group()
        return
    head_name = HEADLINE if args.workload == "all" else args.workload
    head = run.measure(head_name, cpu_budget=None if args.no_cpu_baseline else 12.0, e2e=not args.no_e2e)
    wl = head.pop("_wl")
    line = {"metric": metric_name(head["unit"]), "value": head["value"], "unit": head["unit"],
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": head["scaling"],
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_block(wl, wl, args), "timed": head["timed"],
            "roofline": head["roofline"], "gpu_launches": head["gpu_launches"],
            "clocks": head.get("clocks"), "parity": head["parity"]}
    for key in ("e2e", "cpu_baseline", "parity_detail", "library_gemm"):
        if key in head:
            line[key] = head[key]
    del wl, head
    release()
    if world == 1 and not args.no_e2e:
        line["host_us_per_launch"] = host_overheads(dev)
        line["host_copy_gbs"] = host_copy_rates(dev)
        release()

    if args.workload == "all":
        if world > 1:
            # the stated [8192, 8192] problem split over the ranks, beside the weak-scaled headline
            r = run.measure(HEADLINE, strong=True, e2e=not args.no_e2e)
            r.pop("_wl")
            line["strong"] = r
            release()
        line["configs"] = {}
        for name in OTHER_CONFIGS:
            try:
                r = run.measure(name, cpu_budget=None if args.no_cpu_baseline else args.cpu_budget,
                                e2e=not args.no_e2e)
                r.pop("_wl")
                line["gpu_launches"] += r["gpu_launches"]
            except AssertionError as e:
                if world > 1:
                    raise       # the other ranks are waiting at a barrier: end the job
                r = {"parity": f"FAILED: {e}"}
            line["configs"][name] = r
            release()
        if world > 1 and 32 % world == 0:
            try:
                line["configs"]["tp_llama_layer"] = measure_tp(run)
                line["gpu_launches"] += line["configs"]["tp_llama_layer"]["gpu_launches"]
            except AssertionError:
                raise
            except Exception as e:      # e.g. no peer access between the GPUs of this box: say so, keep the line
                line["configs"]["tp_llama_layer"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
            release()
    if run.sampler:
        run.sampler.stop()
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
