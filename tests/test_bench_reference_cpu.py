"""The benchmark's reference arm needs no GPU: it times the CPU path and prints one JSON line with
the keys the measurement contract names."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_contract_line():
    env = dict(os.environ, OMP_NUM_THREADS="1")     # what torchrun exports to its workers
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True,
                         cwd=ROOT, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["higher_is_better"] is True and line["steps"] == 2 and line["warmup"] == 3
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] == line["value"]
    assert line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert "configs[1]" in line["config"]["workload"]


def test_reference_arm_other_ranks_exit_quietly():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--gpus", "2", "--steps", "1", "--warmup", "3"], capture_output=True,
                         text=True, cwd=ROOT, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip() == ""


def test_default_reference_line_carries_every_configuration():
    env = dict(os.environ, OMP_NUM_THREADS="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "3", "--cpu-budget", "0.2"], capture_output=True,
                         text=True, cwd=ROOT, env=env, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("workload", "l2", "launch", "sharding"):      # the keys the device arm's config has
        assert key in line["config"], key
    want = {"softmax": "GB/s", "softmax_scaled": "GB/s", "relayout": "GB/s", "relayout_permuted": "GB/s",
            "bmm": "TFLOP/s", "llama_layer": "TFLOP/s", "hf_llama_layer": "TFLOP/s"}
    assert set(line["configs"]) == set(want)
    for name, unit in want.items():
        c = line["configs"][name]
        assert c["unit"] == unit and c["value"] > 0 and c["ms_per_step"] > 0, name
        assert c["cpu_baseline"]["cores"] >= 1


def test_every_workload_has_a_cpu_side():
    """Each name the device arm accepts must also build and run on a machine without a GPU."""
    sys.path.insert(0, ROOT)
    import bench

    for name in (bench.HEADLINE,) + bench.OTHER_CONFIGS + bench.EXTRA_WORKLOADS:
        # small leading extents keep this quick; the shapes below the leading dim are the real ones
        rows = {"fused": 64, "pointwise": None, "softmax": None, "softmax_scaled": 512, "relayout": 1,
                "relayout_permuted": 1, "bmm": 1, "llama_layer": 1, "hf_llama_layer": 1,
                "attention": 1, "restickify": 4}[name]
        if name in ("llama_layer", "hf_llama_layer", "bmm", "pointwise"):
            cpu = bench.cpu_side(name, rows=rows)       # built, not run: seconds of CPU time each
            assert callable(cpu["cpu_step"])
        else:
            cpu = bench.cpu_side(name, rows=rows)
            assert cpu["cpu_step"]() is not None
        assert cpu["work"] > 0 and cpu["cpu_work"] > 0 and cpu["unit"] in ("GB/s", "TFLOP/s")
        assert cpu["desc"] and cpu["sample"] and cpu["sharding"] and cpu["scaling"] in ("weak", "strong")


def test_shards_cover_the_stated_problem():
    sys.path.insert(0, ROOT)
    import bench

    for world in (1, 2, 4, 8):
        assert sum(bench.shard(8192, r, world) for r in range(world)) == 8192
        assert sum(bench.shard(32, r, world) for r in range(world)) == 32
        assert sum(bench.shard(8, r, world) for r in range(world)) == 8
    strong = bench.cpu_side("fused", rank=1, world=4, strong=True)
    assert strong["host"][0].shape == (2048, 8192) and strong["scaling"] == "strong"
