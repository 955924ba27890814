"""Drop-in for the reference module ``qjl/matmul.py``."""

from __future__ import annotations

import torch

from .. import ops


def cuda_quantized_bmm_dynamic(group_size: int, fA: torch.Tensor, qB: torch.Tensor,
                               scales: torch.Tensor, zeros: torch.Tensor, bits: int,
                               mqa: bool = False) -> torch.Tensor:
    """Same contract as ``qjl/matmul.py:4-35``: fA [B,nh,1,K] times the group-format operand
    qB [B,nh',K,N*bits/32] with scales/zeros [B,nh',K,N/g]; returns [B,nh,1,N] in fA.dtype.

    nh' may be nh (operands expanded with ``repeat_kv_quant`` as the reference does), any
    divisor of nh (GQA; the kernel maps q head j to KV head j // (nh/nh')), or 1 with
    ``mqa=True``.  Unlike the reference, ``bits == 1`` is supported and no transposed copy of
    the packed operand is made.
    """
    assert len(fA.shape) == 4 and len(qB.shape) == 4
    assert bits in [1, 2, 4]
    if fA.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("Unsupported dtype for tensor fA. Expected float16 or bfloat16.")
    if mqa:
        assert qB.shape[1] == 1
    return ops.qbmm(group_size, fA, qB, scales, zeros, bits)
