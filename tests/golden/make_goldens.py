"""Regenerates the fixtures in this directory.  Run from the repo root in a
container where the reference checkout is mounted:

    python tests/golden/make_goldens.py /path/to/reference

* dci_strides.json - outputs of the reference's own Python layout twin
  (SpyreDCI.spyre_strides, torch_spyre/_inductor/stickify.py:93-101), obtained by
  importing that file (only that file: its parent package needs the closed
  stack) and calling it.
* relayout_images.npz - small stick images produced by the numpy oracle
  (oracle/layout.py); they pin the oracle against accidental change and give the
  GPU tests fixed expected bytes.
"""
import importlib.util
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import layout as L  # noqa: E402


def load_reference_stickify(ref_root):
    pkg = types.ModuleType("refpkg")
    pkg.__path__ = []

    class Unsupported(RuntimeError):
        pass

    pkg.Unsupported = Unsupported
    sys.modules["refpkg"] = pkg
    path = os.path.join(ref_root, "torch_spyre", "_inductor", "stickify.py")
    spec = importlib.util.spec_from_file_location("refpkg.stickify", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["refpkg.stickify"] = mod
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    ref = load_reference_stickify(ref_root)
    cases = []
    for size, order in [([128], [0]), ([512, 256], [0, 1]), ([512, 256], [1, 0]),
                        ([512, 8, 256], [0, 1, 2]), ([512, 8, 256], [2, 1, 0]),
                        ([3, 5, 7], [1, 0, 2]), ([2, 6, 3, 128], [0, 1, 2, 3]),
                        ([2, 6, 3, 128], [3, 0, 2, 1])]:
        for fmt in ("DENSE", "SPARSE"):
            dci = ref.SpyreDCI(list(order), format=getattr(ref.StickFormat, fmt))
            strides = dci.spyre_strides(torch.Size(size), torch.float16)
            cases.append({"size": size, "dim_order": order, "format": fmt,
                          "strides": [int(s) for s in strides],
                          "stick_dims": dci.get_stick_dims()})
    with open(os.path.join(HERE, "dci_strides.json"), "w") as f:
        json.dump({"_source": "SpyreDCI.spyre_strides, torch_spyre/_inductor/stickify.py:93-101",
                   "elems_per_stick_fp16": ref.elems_per_stick(torch.float16),
                   "cases": cases}, f, indent=1)

    images = {}
    rng = np.random.default_rng(20250101)
    for name, shape in [("r1_100", (100,)), ("r2_5x70", (5, 70)), ("r3_3x4x130", (3, 4, 130)),
                        ("r4_2x3x2x64", (2, 3, 2, 64))]:
        host = rng.integers(0, 65536, size=shape, dtype=np.uint16)
        images[name + "_host"] = host
        images[name + "_generic"] = L.to_sticks(host, L.generic_stick_layout(shape))
        images[name + "_legacy"] = L.to_sticks(host, L.legacy_copy_layout(shape))
    np.savez_compressed(os.path.join(HERE, "relayout_images.npz"), **images)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_goldens.py <path to a torch-spyre checkout>")
    main(sys.argv[1])
