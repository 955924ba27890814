"""CPU oracle for the quantized-KV attention path (TEST INFRASTRUCTURE ONLY).

This package restates, in plain PyTorch on CPU, the arithmetic of the reference
(ActiveSky/calibquant) for the one hot path this library accelerates.  It exists
to *check* the CUDA kernels; it is never the product path.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
may import it.  The shipped package (``calibquant_b200``) never imports it and
fails loudly when its CUDA library is missing.

Parity pinning: the reference has no tests and no golden vectors of its own, so
the restatements here are pinned against *outputs of the reference's own
functions executed on CPU* (``qjl/new_pack.py`` and ``calibquant.py`` under the
Triton interpreter, ``calibquant.quant`` / ``encode`` natively).  The script
``tests/golden/make_golden.py`` runs the reference and writes the fixtures that
``tests/test_oracle_golden.py`` replays.  The reference's CUDA extensions
(``quantization``, ``cuda_qjl_quant``, ``cuda_qjl_gqa_score``) are built unchanged by
``oracle/build_ref.py`` and run on a GPU by ``tests/test_gpu_ref_pin*.py``, which pins
``group_format.qbmm`` at 2 and 4 bits, the decode composition and ``qjl.py``.  Two pieces
have no runnable reference at all and are "parity unpinned" by the reference itself:

* ``group_format.qbmm`` at 1 bit (the reference CUDA kernel cannot run 1-bit:
  ``qjl/matmul.py:24`` asserts bits in [2, 4]); it follows the dequantize-and-
  accumulate arithmetic of ``qjl/csrc/quantization.cu:108-123``.
* ``prefill.causal_attention`` (the reference calls the third-party flash_attn
  library, ``patch_internvl.py:464-468``); it is plain fp32 softmax attention, compared
  with that library on a GPU where it is installed (``tests/test_gpu_prefill.py``).
"""

from . import generator, group_format, calibquant_format, prefill, forward  # noqa: F401
