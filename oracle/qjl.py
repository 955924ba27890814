"""CPU restatement (PyTorch, fp32) of the reference's QJL sign-sketch kernels.  Test infrastructure only.

* ``qjl_quant``      <- ``qjl/csrc/qjl_quant_kernel.cu:53-168`` (``quantize_with_outliers_kernel``):
  per token, sign bits of the projections of the inlier and of the outlier channels, packed LSB-first
  eight per byte (``1 << (wIdx % 8)``, ``:147-148``), and the 2-norm of the outlier channels (``:128-166``).
  The same arithmetic is spelled out in torch in ``qjl/qjl_utils.py:46-73`` (``qjl_qunatize``).
* ``qjl_gqa_score``  <- ``qjl/csrc/qjl_gqa_score_kernel.cu:40-180`` (``calc_gqa_score_kernel``): the
  estimator ``sqrt(pi/2)/s |k_in| <sgn(S k_in), S q_in> + sqrt(pi/2)/s_o |k_out| <sgn(S k_out), S q_out>``
  (``:170-177``), with ``S q_out`` rebuilt from the group's outlier channels (``:118-127``).
* ``build_groups``   <- ``qjl/qjl_utils.py:115-134`` (grouping, top-k outlier channels by group norm).

Parity pinned on a GPU: the reference has no test vectors for these kernels, so ``oracle/build_ref.py`` builds
the two reference extensions unchanged and ``tests/test_gpu_ref_pin_qjl.py`` compares this file (and the library)
with their outputs on seeded inputs.  This file follows the kernel sources line by line.  One deliberate difference: ``|k_in|`` uses
``max(|k|^2 - |k_out|^2, 0)`` where the kernel takes the square root of the raw difference.
"""

from __future__ import annotations

import math

import torch


def pack_bits(bits: torch.Tensor) -> torch.Tensor:
    """bool [..., s] -> uint8 [..., s/8], bit p%8 of byte p/8."""
    b = bits.reshape(*bits.shape[:-1], -1, 8).to(torch.int32)
    w = (b << torch.arange(8, dtype=torch.int32)).sum(-1)
    return w.to(torch.uint8)


def unpack_bits(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., n] -> bool [..., 8n]."""
    b = (packed.to(torch.int32).unsqueeze(-1) >> torch.arange(8, dtype=torch.int32)) & 1
    return b.reshape(*packed.shape[:-1], -1).bool()


def outlier_mask(outlier_indices: torch.Tensor, dim: int) -> torch.Tensor:
    """uint8 [B,H,n,oc] -> float [B,H,n,dim] with ones at the outlier channels."""
    m = torch.zeros(*outlier_indices.shape[:3], dim)
    return m.scatter_(-1, outlier_indices.long(), 1.0)


def sketches(key_states, outlier_indices, rand_prj):
    """fp32 projections of the inlier and outlier parts: two tensors [B,H,n,G,s]."""
    k = key_states.float()
    m = outlier_mask(outlier_indices, k.shape[-1]).unsqueeze(-2)
    p = rand_prj.float()
    return torch.einsum("bhngd,sd->bhngs", k * (1 - m), p), torch.einsum("bhngd,sd->bhngs", k * m, p)


def qjl_quant(key_states, outlier_indices, rand_prj, outlier_sketch_dim):
    """key_states [B,H,n,G,D], outlier_indices uint8 [B,H,n,oc], rand_prj [s,D] ->
    (key_quant uint8 [B,H,n,G,s/8], key_outlier_quant uint8 [B,H,n,G,s_o/8], outlier_norms [B,H,n,G])."""
    sk_in, sk_out = sketches(key_states, outlier_indices, rand_prj)
    m = outlier_mask(outlier_indices, key_states.shape[-1]).unsqueeze(-2)
    norms = (key_states.float() * m).pow(2).sum(-1).sqrt().to(key_states.dtype)
    return pack_bits(sk_in > 0), pack_bits(sk_out[..., :outlier_sketch_dim] > 0), norms


def qjl_gqa_score(key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices, query_sketch,
                  query_states, rand_prj):
    """-> fp32 [B,Hq,n*G,1].  query_states [B,Hq,1,D]; query_sketch [B,Hq,1,s]; rand_prj [D,s]."""
    B, Hkv, n, G, _ = key_quant.shape
    Hq, D = query_states.shape[1], query_states.shape[-1]
    rep = Hq // Hkv
    s, so = key_quant.shape[-1] * 8, key_outlier_quant.shape[-1] * 8
    q = query_states.float().reshape(B, Hkv, rep, D)
    qs = query_sketch.float().reshape(B, Hkv, rep, s)
    m = outlier_mask(outlier_indices, D)                                   # [B,Hkv,n,D]
    q_out = torch.einsum("bhrd,bhnd,ds->bhnrs", q, m, rand_prj.float())     # sketch of q on the outlier channels
    q_in = qs.unsqueeze(2) - q_out
    sgn = unpack_bits(key_quant).float() * 2 - 1                            # [B,Hkv,n,G,s]
    sgn_o = unpack_bits(key_outlier_quant).float() * 2 - 1
    inner = torch.einsum("bhngs,bhnrs->bhrng", sgn, q_in)
    outer = torch.einsum("bhngs,bhnrs->bhrng", sgn_o, q_out[..., :so])
    no = key_outlier_norm.float()
    ni = (key_norm.float().pow(2) - no.pow(2)).clamp_min(0).sqrt()
    c = math.sqrt(math.pi / 2)
    score = c / s * ni.unsqueeze(2) * inner + c / so * no.unsqueeze(2) * outer
    return score.reshape(B, Hq, n * G, 1)


def build_groups(key_states, group_size, outliers_count):
    """[B,H,T,D] (T a multiple of group_size) -> (groups [B,H,n,G,D], outlier_indices uint8 [B,H,n,oc],
    key norms [B,H,n,G]) as ``QJLKeyQuantizer.build_sketch`` forms them."""
    B, H, T, D = key_states.shape
    groups = key_states.reshape(B, H, T // group_size, group_size, D)
    _, idx = groups.float().norm(dim=-2).topk(outliers_count, dim=-1)
    return groups, idx.to(torch.uint8), groups.float().norm(dim=-1).to(key_states.dtype)
