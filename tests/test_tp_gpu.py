"""Tensor-parallel decoder layer on 2 (and 4) GPUs of one box against the unsharded CPU oracle:
the row-parallel linears reduce-scatter inside the GEMM epilogue over NVLink peer memory
(ts_gemm_f16_scatter_add), the gathers are peer copies (ts_peer_copy_2d).  Skipped on a box with
one GPU.  Reference goal: the sharded decoder layer of tests/test_modules.py:133-211."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, *dims, port=29611):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py"),
           *[str(d) for d in dims]]
    out = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert out.returncode == 0, (out.stdout[-3000:], out.stderr[-3000:])
    assert f"TP_OK world={world}" in out.stdout, out.stdout[-2000:]
    return out.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_layer_matches_the_unsharded_oracle(world, cuda):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, 512, 4, 1024, 2, 256, port=29611 + world)


def test_sharded_layer_full_width_two_ranks(cuda):
    """d_model 4096, 32 heads, FFN 11008 on a 256-token prefix, two ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, 4096, 32, 11008, 1, 256, port=29617)


def test_sharded_model_two_ranks(cuda):
    """Token ids -> embedding -> three sharded decoder layers sharing their peer buffers -> final
    norm -> logits (tensor_parallel.TPLlamaModel) on two ranks, against the unsharded CPU oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = _run(2, 512, 4, 1024, 2, 256, 1000, 3, port=29619)
    assert "model layers=3" in out
