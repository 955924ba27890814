"""calibquant_b200 -- B200 (sm_100a) implementation of CalibQuant's quantized-KV attention path.

Layout
    csrc/            CUDA kernels and the C ABI (built into libcalibquant_b200.so)
    _lib.py          ctypes binding of that ABI
    ops.py           tensor-level entry points (device pointers + current stream)
    qjl/             drop-in modules with the reference's names and signatures
    build.py         nvcc build of the shared library

The CUDA library is the only implementation: importing the package works without it (so
that it can be built), but any compute call raises if the library is missing.
"""

from . import ops  # noqa: F401
from ._lib import CalibQuantError, lib  # noqa: F401

__version__ = "0.1.0"
