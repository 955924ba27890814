"""Oracle for the CalibQuant uint8 format (test infrastructure).

Restates on CPU:

* ``quant``           <- ``calibquant.py:24-42`` (min-max over tokens with a clip factor)
* ``encode``          <- ``calibquant.py:114-137`` (uint8, most-significant field first)
* ``fused_kernel``    <- ``calibquant.py:54-111``  (scores = weights . LUT[code], fp16 out)
* ``fused_kernel_wv`` <- ``calibquant.py:192-276`` (out = weights . LUT[code], fp16 out)
* ``prefill_quantize`` <- ``patch_internvl.py:288-339``
* ``decode_attention`` <- ``patch_internvl.py:356-436`` (post-scaling, bias, calibration)

The reference recovers code indices through ``torch.unique`` of the first 10 000
quantized values (``patch_internvl.py:318-329``).  Its lookup table then maps
index -> quantized level, so ``LUT[index]`` equals the quantized level itself
whenever every level occurs in that sample.  This oracle (and the CUDA path) use
the identity table ``LUT[c] = c``, which is that same function.
"""

from __future__ import annotations

import math

import torch

from .group_format import repeat_kv, calibrate


def quant(x, bits, per_channel=False, scale=1, post_scale=False):
    """x [B,T,H,D]; per_channel reduces over dim 1 (tokens). Every op in x.dtype."""
    levels = 2 ** bits - 1
    if per_channel:
        x_min = x.amin(dim=1, keepdim=True) * scale
        x_max = x.amax(dim=1, keepdim=True) * scale
    else:
        x_min = x.min() * scale
        x_max = x.max() * scale
    s = (x_max - x_min) / levels
    zp = -x_min / s
    x_q = torch.round(torch.clamp(x / s + zp, 0, levels))
    if post_scale:
        return x_q, s, zp
    return s * (x_q - zp), s, zp


def encode(codes: torch.Tensor, bits: int, datum_per_elem: int) -> torch.Tensor:
    """Integer codes [B,H,T,D] -> uint8 [B,H,T,D*bits/8]; field i of a byte sits at
    bit offset bits*(datum_per_elem-1-i)."""
    B, H, T, D = codes.shape
    y = codes.to(torch.int64).reshape(B, H, T, D // datum_per_elem, datum_per_elem)
    shift = bits * (datum_per_elem - 1 - torch.arange(datum_per_elem))
    return (y << shift).sum(dim=-1).to(torch.uint8)


def decode_bytes(enc: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 [..., P] -> integer codes [..., P*8/bits] (int64)."""
    dpe = 8 // bits
    shift = bits * (dpe - 1 - torch.arange(dpe))
    c = (enc.to(torch.int64).unsqueeze(-1) >> shift) & (2 ** bits - 1)
    return c.reshape(*enc.shape[:-1], enc.shape[-1] * dpe)


def fused_kernel(lut, weights, enc, bits):
    """s[b,h,0,t] = sum_d weights[b,h,0,d]*lut[code[b,h,t,d]]; fp32 accumulate, fp16 out."""
    vals = lut.to(torch.float32)[decode_bytes(enc, bits)]               # [B,H,T,D]
    out = torch.matmul(weights.to(torch.float32), vals.transpose(2, 3))
    return out.to(torch.float16)


def fused_kernel_wv(lut, weights, enc, bits):
    """o[b,h,0,n] = sum_t weights[b,h,0,t]*lut[code[b,h,t,n]]; fp32 accumulate, fp16 out."""
    vals = lut.to(torch.float32)[decode_bytes(enc, bits)]               # [B,H,T,D]
    return torch.matmul(weights.to(torch.float32), vals).to(torch.float16)


def prefill_quantize(k_vis, v_vis, bits, clip_k, clip_v, n_rep):
    """k_vis, v_vis [B,T,Hkv,D] -> state dict as the reference keeps on the module.

    scale/zero-point come back as [B,Hq,1,D] (already repeated to q heads, as
    ``patch_internvl.py:300-309``); enc_* are uint8 [B,Hkv,T,D*bits/8].
    """
    dpe = 8 // bits
    vq, sv, zv = quant(v_vis, bits, per_channel=True, scale=clip_v, post_scale=True)
    kq, sk, zk = quant(k_vis, bits, per_channel=True, scale=clip_k, post_scale=True)
    rep = lambda t: repeat_kv(t.transpose(1, 2), n_rep)
    return {
        "scale_key": rep(sk), "zero_point_key": rep(zk),
        "scale_value": rep(sv), "zero_point_value": rep(zv),
        "enc_k": encode(kq.transpose(1, 2), bits, dpe),
        "enc_v": encode(vq.transpose(1, 2), bits, dpe),
    }


def decode_attention(q, state, k_fp, v_fp, bits, sys_len, normalize=None):
    """One decode step. q [B,Hq,1,D]; k_fp/v_fp [B,Hkv,T_fp,D] hold [sys | text].

    Returns o [B,Hq,1,D] in bfloat16 (the reference hard-codes that cast,
    ``patch_internvl.py:436``).
    """
    B, Hq, _, D = q.shape
    n_rep = Hq // k_fp.shape[1]
    if normalize is None:
        normalize = bits <= 2
    sd = math.sqrt(D)
    lut = torch.arange(2 ** bits, dtype=q.dtype)
    k = repeat_kv(k_fp, n_rep)
    v = repeat_kv(v_fp, n_rep)
    enc_k = repeat_kv(state["enc_k"], n_rep)
    enc_v = repeat_kv(state["enc_v"], n_rep)
    sk, zk = state["scale_key"], state["zero_point_key"]
    sv, zv = state["scale_value"], state["zero_point_value"]
    s_sys = torch.matmul(q, k[:, :, :sys_len].transpose(2, 3)) / sd
    s_txt = torch.matmul(q, k[:, :, sys_len:].transpose(2, 3)) / sd
    bias_k = torch.sum(sk * zk * q, dim=-1, keepdim=True) / sd
    s_vis = fused_kernel(lut, q * sk, enc_k, bits) / sd - bias_k
    if normalize:
        s_vis = calibrate(s_vis)
    t_vis = s_vis.shape[-1]
    att = torch.softmax(torch.cat([s_sys, s_vis, s_txt], dim=-1), dim=-1,
                        dtype=torch.float32).to(q.dtype)
    a_vis = att[..., sys_len:sys_len + t_vis]
    o_vis = fused_kernel_wv(lut.half(), a_vis.half(), enc_v, bits) * sv
    o_vis = o_vis - sv * zv * torch.sum(a_vis, dim=-1, keepdim=True)
    o = o_vis + torch.matmul(att[..., :sys_len], v[:, :, :sys_len]) \
        + torch.matmul(att[..., sys_len + t_vis:], v[:, :, sys_len:])
    return o.to(torch.bfloat16)
