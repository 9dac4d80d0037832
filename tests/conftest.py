import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "torch-spyre_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def _ensure_built():
    """Build the kernel library, the device extension and the C oracle if they are missing
    (nvcc cross-compiles, so this also works on a machine without a GPU)."""
    pkg = os.path.join(ROOT, "torch-spyre_b200", "torch_spyre")
    need = [os.path.join(pkg, "lib", "libspyre_b200.so"), os.path.join(pkg, "_C.so"),
            os.path.join(ROOT, "oracle", "librelayout_oracle.so")]
    if all(os.path.exists(p) for p in need):
        return
    import importlib.util
    spec = importlib.util.spec_from_file_location("graft_entry", os.path.join(ROOT, "__graft_entry__.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


_ensure_built()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("test marked gpu but no CUDA device is visible")
    return torch.device("cuda:0")
