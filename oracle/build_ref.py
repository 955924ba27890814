"""Build the reference's own CUDA extension for the quantized product into ``oracle/_ref/`` (test infrastructure).

    python oracle/build_ref.py [path/to/reference]

Compiles ``qjl/csrc/quantization.cu``, ``qjl_quant_kernel.cu`` and ``qjl_gqa_score_kernel.cu`` of
ActiveSky/calibquant, unchanged and where they lie in the reference checkout (default: the directory
``reference`` beside this repository), with
the flags of the reference's ``qjl/setup.py:5-15`` plus the sm_100a code generation flag, into
``oracle/_ref/<module>.so``.  Nothing of the reference is copied into
this repository: ``oracle/_ref/`` is ignored by git and holds build outputs only.

The extension is the only executable definition of ``cuda_quantized_bmm_dynamic``'s arithmetic
(``qjl/csrc/quantization.cu:67-169``).  ``tests/test_gpu_ref_pin.py`` runs it on a GPU for 2 and 4 bits (its
``psum[16]`` array cannot hold the 32 codes of a 1-bit word) and compares it with the CPU oracle and with
``cq_qbmm``; ``tests/test_gpu_ref_pin_qjl.py`` does the same for the two QJL kernels
(``qjl_quant_kernel.cu:53-168``, ``qjl_gqa_score_kernel.cu:40-180``).  The product never loads any of them.
"""

from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REFERENCE = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


# extension name -> source file under qjl/csrc (the module names the reference's qjl/setup.py:18-57 gives them)
EXTENSIONS = {
    "quantization": "quantization.cu",
    "cuda_qjl_quant": "qjl_quant_kernel.cu",
    "cuda_qjl_gqa_score": "qjl_gqa_score_kernel.cu",
}


def build_one(name: str, reference_root: str = DEFAULT_REFERENCE, verbose: bool = False) -> str | None:
    src = os.path.join(reference_root, "qjl", "csrc", EXTENSIONS[name])
    target = os.path.join(OUT, name + ".so")
    if not os.path.exists(src):
        return target if os.path.exists(target) else None
    if os.path.exists(target) and os.path.getmtime(target) >= os.path.getmtime(src):
        return target
    out_dir = os.path.join(OUT, "_build_" + name)
    os.makedirs(out_dir, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")      # no GPU is needed to compile
    from torch.utils.cpp_extension import load
    load(name=name, sources=[src], build_directory=out_dir, verbose=verbose,
         extra_cflags=["-O3"],
         extra_cuda_cflags=["-O3", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                            "--use_fast_math", "-gencode", "arch=compute_100a,code=sm_100a"])
    built = os.path.join(out_dir, name + ".so")
    if os.path.exists(built):
        os.replace(built, target)
    return target if os.path.exists(target) else None


def build(reference_root: str = DEFAULT_REFERENCE, verbose: bool = False) -> str | None:
    """Build every extension; returns the path of ``quantization.so`` (None if it could not be built)."""
    paths = {name: build_one(name, reference_root, verbose) for name in EXTENSIONS}
    return paths["quantization"]


if __name__ == "__main__":
    path = build(*(sys.argv[1:2]), verbose=True)
    print(path or "reference sources not found; nothing built")
