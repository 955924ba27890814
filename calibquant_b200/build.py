"""Build the C-ABI CUDA library in-tree with plain nvcc for sm_100a.

    python -m calibquant_b200.build [--force] [--ptxas-v]

replaces the reference's ``qjl/setup.py`` (four torch CUDAExtensions with no arch
flags): one shared object, no torch headers, one architecture.  Every ``csrc/*.cu`` is
compiled to an object file of its own (in parallel, rebuilt only when it or a header
changed) and the objects are linked into ``libcalibquant_b200.so``.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libcalibquant_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
]


def find_nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build calibquant_b200")
    return cand


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(os.path.dirname(PKG_DIR), "include", "*.h"))


def _obj(src: str) -> str:
    return os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(p) > t for p in deps)


def needs_build() -> bool:
    return _stale(LIB_PATH, sources() + _headers())


def build_library(force: bool = False, verbose: bool = False, extra=()) -> str:
    if not force and not needs_build():
        return LIB_PATH
    nvcc = find_nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = _headers()
    todo = [s for s in sources() if force or extra or _stale(_obj(s), [s] + hdrs)]

    def compile_one(src):
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", _obj(src)]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1) or 1) as pool:
        for src, res in pool.map(compile_one, todo):
            if verbose or res.returncode:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB_PATH, *[_obj(s) for s in sources()]]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    extra = ["-Xptxas", "-v"] if "--ptxas-v" in sys.argv else []
    print(build_library(force="--force" in sys.argv or bool(extra), verbose=True, extra=extra))
