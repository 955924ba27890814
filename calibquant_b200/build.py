"""Build the C-ABI CUDA library in-tree with plain nvcc for sm_100a.

    python -m calibquant_b200.build

replaces the reference's ``qjl/setup.py`` (four torch CUDAExtensions with no arch
flags): one shared object, no torch headers, one architecture.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libcalibquant_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def find_nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build calibquant_b200")
    return cand


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(os.path.dirname(PKG_DIR), "include", "*.h"))
    return any(os.path.getmtime(p) > os.path.getmtime(LIB_PATH) for p in deps)


def build_library(force: bool = False, verbose: bool = False, extra=()) -> str:
    if not force and not needs_build():
        return LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS, *extra, "-o", LIB_PATH, *sources()]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    extra = ["-Xptxas", "-v"] if "--ptxas-v" in sys.argv else []
    print(build_library(force=True, verbose=True, extra=extra))
