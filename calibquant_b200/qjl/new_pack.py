"""Drop-in for the reference module ``qjl/new_pack.py``.

``triton_quantize_and_pack_along_last_dim`` keeps the reference's name, arguments and
return layout (``qjl/new_pack.py:53-82``) so existing call sites keep working; the work is
done by one CUDA kernel (``cq_pack_last_dim``), not Triton.
"""

from __future__ import annotations

import torch

from .. import ops


def triton_quantize_and_pack_along_last_dim(data: torch.Tensor, group_size: int, bit: int):
    """data [B,nh,D,T] -> (code int32 [B,nh,D,T*bit/32], scale [B,nh,D,T/g], mn [B,nh,D,T/g])."""
    assert len(data.shape) == 4
    assert data.shape[-1] % group_size == 0
    return ops.pack_last_dim(data, group_size, bit)


def quantize_and_pack_k_per_channel(k: torch.Tensor, group_size: int, bit: int):
    """K given token-major [B,nh,T,D] -> per-channel pack, i.e. the result of the call above on
    ``k.transpose(2, 3).contiguous()`` without making that copy."""
    return ops.pack_k_per_channel(k, group_size, bit)
