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
    if not force and not verbose_ptxas and os.path.exists(LIB_PATH):
        # an up-to-date library needs no objects (a copy of the tree made without build/ has none)
        newest = max(os.path.getmtime(p) for p in [os.path.join(CSRC, f) for f in sources] + headers)
        if os.path.getmtime(LIB_PATH) >= newest:
            return LIB_PATH
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


EXT_SRC = os.path.join(CSRC, "ext")
EXT_BUILD = os.path.join(HERE, "build", "ext")
EXT_PATH = os.path.join(HERE, "torch_spyre", "_C.so")


def build_extension(force: bool = False) -> str:
    """Builds torch_spyre/_C.so: the `spyre` (PrivateUse1) device glue and pybind module.
    It links against libspyre_b200.so (rpath $ORIGIN/lib) and PyTorch's CUDA libraries."""
    import shutil

    from torch.utils import cpp_extension

    build_library()
    sources = sorted(os.path.join(EXT_SRC, f) for f in os.listdir(EXT_SRC) if f.endswith(".cpp"))
    deps = sources + [os.path.join(EXT_SRC, f) for f in os.listdir(EXT_SRC) if f.endswith(".h")]
    deps.append(os.path.join(INCLUDE, "spyre_b200.h"))
    if not force and os.path.exists(EXT_PATH) and not _newer(sources[0], EXT_PATH, deps):
        return EXT_PATH
    os.makedirs(EXT_BUILD, exist_ok=True)
    cpp_extension.load(
        name="_C", sources=sources, build_directory=EXT_BUILD, is_python_module=False,
        with_cuda=True, verbose=False,
        extra_cflags=["-O2", "-std=c++17", "-DTORCH_EXTENSION_NAME=_C"],
        extra_ldflags=[f"-L{LIB_DIR}", "-lspyre_b200", "-Wl,-rpath,\\$$ORIGIN/lib", "-Wl,-rpath,\\$$ORIGIN/../../torch_spyre/lib"],
        extra_include_paths=[INCLUDE])
    shutil.copyfile(os.path.join(EXT_BUILD, "_C.so"), EXT_PATH)
    return EXT_PATH


if __name__ == "__main__":
    if "--ext" in sys.argv:
        print(build_extension(force="--force" in sys.argv))
        sys.exit(0)
    print(build_library(force="--force" in sys.argv, verbose_ptxas="--verbose-ptxas" in sys.argv))
