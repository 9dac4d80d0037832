"""Builds libspyre_b200.so (the C-ABI kernel library) for sm_100a with nvcc.

Usage: python build.py [--force] [--verbose-ptxas]
Objects go to build/, the library next to the Python package in torch_spyre/lib/.
nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_DIR = os.path.join(HERE, "torch_spyre", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libspyre_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-I", INCLUDE,
]


def _newer(src: str, dst: str, deps) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(d) > t for d in [src, *deps])


def build_library(force: bool = False, verbose_ptxas: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else [])
    jobs = []
    for f in sources:
        src = os.path.join(CSRC, f)
        obj = os.path.join(OBJ_DIR, f[:-3] + ".o")
        if force or verbose_ptxas or _newer(src, obj, headers):
            jobs.append(["nvcc", *flags, "-c", src, "-o", obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for cmd, r in pool.map(run, jobs):
            out = (r.stdout + r.stderr).strip()
            if r.returncode != 0 or (verbose_ptxas and out):
                print(" ".join(cmd[-3:]), file=sys.stderr)
                print(out, file=sys.stderr)
            failed = failed or r.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    objs = [os.path.join(OBJ_DIR, f[:-3] + ".o") for f in sources]
    if jobs or not os.path.exists(LIB_PATH):
        subprocess.check_call(["nvcc", "-shared", "-o", LIB_PATH, *objs])
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose_ptxas="--verbose-ptxas" in sys.argv))
