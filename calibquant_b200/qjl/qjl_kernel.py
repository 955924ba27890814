"""Drop-in for the reference module ``qjl/qjl_kernel.py``: the dtype-dispatching entry points of the
QJL sign-sketch kernels, served by ``libcalibquant_b200.so`` instead of the three pybind11 extensions
``cuda_qjl_quant``, ``cuda_qjl_score`` and ``cuda_qjl_gqa_score``.

Supported dtype pairs (keys or queries, projection): (half, half), (half, float), (bfloat16, bfloat16),
(bfloat16, float); anything else raises ``TypeError`` as the reference does.
"""

from __future__ import annotations

import torch

from .. import ops

_PAIRS = {(torch.float16, torch.float16), (torch.float16, torch.float32),
          (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)}


def qjl_quant(key_states, outlier_indices, rand_prj, outlier_sketch_dim):
    """``qjl/qjl_kernel.py:8-28``: (key_quant, key_outlier_quant, outlier_norms) of grouped keys."""
    if (key_states.dtype, rand_prj.dtype) not in _PAIRS:
        raise TypeError("Unsupported data types for QJL quantization")
    return ops.qjl_quant(key_states, outlier_indices, rand_prj, outlier_sketch_dim)


def qjl_gqa_score(key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices, query_sketch,
                  query_states, rand_prj):
    """``qjl/qjl_kernel.py:52-72``: fp32 scores [B,Hq,n*G,1]; keys at KV-head count."""
    if (query_states.dtype, rand_prj.dtype) not in _PAIRS:
        raise TypeError("Unsupported data types for QJL GQA score calculation")
    return ops.qjl_gqa_score(key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices,
                             query_sketch, query_states, rand_prj)


def qjl_score(key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices, query_sketch,
              query_states, rand_prj):
    """``qjl/qjl_kernel.py:30-50``: the same estimator with as many key heads as query heads."""
    if (query_states.dtype, rand_prj.dtype) not in _PAIRS:
        raise TypeError("Unsupported data types for QJL score calculation")
    return ops.qjl_gqa_score(key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices,
                             query_sketch, query_states, rand_prj)
