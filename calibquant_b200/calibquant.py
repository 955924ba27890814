"""Drop-in for the reference module ``calibquant.py`` (the CalibQuant uint8 format).

Same names, arguments and results as the reference: ``quant`` (``calibquant.py:24-42``), ``encode``
(``:114-137``), ``fused_kernel`` (``:104-111``) and ``fused_kernel_wv`` (``:269-276``), plus the module
constants ``BITS_KV, SCALE_K, SCALE_V, DATA_TYPE``.  The work is done by CUDA kernels of
``libcalibquant_b200.so`` instead of eager torch / torch.compile / Triton; inputs must be CUDA tensors.
"""

from __future__ import annotations

import ctypes

import torch

from . import ops
from ._lib import check, lib
from .ops import _dtype_enum, _need_cuda, _ptr, _stream, _workspace

DATA_TYPE = torch.float16
BITS_KV = 1

if BITS_KV == 1:
    SCALE_V = 0.3
    SCALE_K = 0.5
else:
    SCALE_V = 1
    SCALE_K = 1


def _strides3(t):
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def _prep(x):
    if x.stride(3) != 1 or any(s % 8 for s in x.stride()[:3]) or x.data_ptr() % 16:
        x = x.contiguous()
    return x


def quant_params(x: torch.Tensor, bits: int, scale=1):
    """Per-channel (over tokens, dim 1) scale and zero point of ``quant``: both [B,1,H,D]."""
    _need_cuda(x)
    x = _prep(x)
    B, T, H, D = x.shape
    s = torch.empty((B, 1, H, D), dtype=x.dtype, device=x.device)
    zp = torch.empty_like(s)
    with torch.cuda.device(x.device):
        rc = lib().cq_calib_minmax(_ptr(x), B, T, H, D, _strides3(x), bits, float(scale), _dtype_enum(x),
                                   _ptr(s), _ptr(zp), _stream())
    check(rc, "cq_calib_minmax")
    return s, zp


def quant(x, bits, per_channel=False, scale=1, post_scale=False):
    """``quant(x [B,T,H,D], bits, per_channel=True, scale=clip, post_scale)`` ->
    ``(x_q or dequantized x, scale, zero_point)``.  ``per_channel=True`` (min/max over tokens per channel) is
    the mode the reference's attention forward uses (``patch_internvl.py:292,297``); ``per_channel=False``
    takes one scale and zero point for the whole tensor and returns them as 0-dim tensors."""
    _need_cuda(x)
    x = _prep(x)
    B, T, H, D = x.shape
    if per_channel:
        s, zp = quant_params(x, bits, scale)
        s_ret, zp_ret = s, zp
    else:
        # one scale for the whole tensor (calibquant.py:29-31): the two reductions and the four scalar ops run
        # as the reference writes them, the per-element pass is the same kernel with the scalars broadcast
        x_min, x_max = x.min() * scale, x.max() * scale
        s_ret = (x_max - x_min) / (2 ** bits - 1)
        zp_ret = -x_min / s_ret
        s = s_ret.to(x.dtype).expand(B, 1, H, D).contiguous()
        zp = zp_ret.to(x.dtype).expand(B, 1, H, D).contiguous()
    out = torch.empty((B, T, H, D), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib().cq_calib_quantize(_ptr(x), B, T, H, D, _strides3(x), bits, _dtype_enum(x), _ptr(s), _ptr(zp),
                                     0 if post_scale else 1, _ptr(out), None, _stream())
    check(rc, "cq_calib_quantize")
    return out, s_ret, zp_ret


def quant_encode(x, bits, scale=1):
    """Fused ``quant`` + ``encode``: x [B,T,H,D] -> (enc uint8 [B,H,T,D*bits/8], scale, zero_point)
    without materialising the codes (replaces ``patch_internvl.py:292-339`` per tensor)."""
    _need_cuda(x)
    x = _prep(x)
    B, T, H, D = x.shape
    s, zp = quant_params(x, bits, scale)
    enc = torch.empty((B, H, T, D * bits // 8), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib().cq_calib_quantize(_ptr(x), B, T, H, D, _strides3(x), bits, _dtype_enum(x), _ptr(s), _ptr(zp),
                                     0, None, _ptr(enc), _stream())
    check(rc, "cq_calib_quantize")
    return enc, s, zp


def encode(X: torch.Tensor, bits=BITS_KV, datum_per_elem=int(8 / BITS_KV)):
    """Integer codes [B,H,T,D] -> uint8 [B,H,T,D/datum_per_elem], most significant field first."""
    _need_cuda(X)
    assert datum_per_elem * bits == 8
    codes = X.to(torch.int64).contiguous()
    out = torch.empty((*X.shape[:-1], X.shape[-1] // datum_per_elem), dtype=torch.uint8, device=X.device)
    with torch.cuda.device(X.device):
        rc = lib().cq_calib_encode_i64(_ptr(codes), codes.numel(), bits, _ptr(out), _stream())
    check(rc, "cq_calib_encode_i64")
    return out


def fused_kernel(unique_values, weights, features_enc, BITS=BITS_KV, DATUM_PER_ELM=int(8 / BITS_KV)):
    """scores[b,h,0,t] = sum_d weights[b,h,0,d] * unique_values[code[b,h',t,d]] -> fp16 [B,Hq,1,T].
    ``features_enc`` may carry Hq heads (as the reference passes it) or the KV-head count."""
    _need_cuda(unique_values, weights, features_enc)
    B, Hq = weights.shape[0], weights.shape[1]
    He, T = features_enc.shape[1], features_enc.shape[2]
    w = weights.reshape(B, Hq, -1).contiguous()
    lut = unique_values.to(w.dtype).contiguous()
    enc = features_enc.contiguous()
    out = torch.empty((B, Hq, 1, T), dtype=torch.float16, device=w.device)
    with torch.cuda.device(w.device):
        rc = lib().cq_lut_scores(_ptr(lut), _ptr(w), _ptr(enc), _ptr(out), B, Hq, He, T, w.shape[-1], BITS,
                                 _dtype_enum(w), _stream())
    check(rc, "cq_lut_scores")
    return out


def fused_kernel_wv(unique_values, weights, features_enc, BITS=BITS_KV, DATUM_PER_ELM=int(8 / BITS_KV)):
    """out[b,h,0,n] = sum_t weights[b,h,0,t] * unique_values[code[b,h',t,n]] -> fp16 [B,Hq,1,D]."""
    _need_cuda(unique_values, weights, features_enc)
    B, Hq = weights.shape[0], weights.shape[1]
    He, T = features_enc.shape[1], features_enc.shape[2]
    D = features_enc.shape[3] * DATUM_PER_ELM
    w = weights.reshape(B, Hq, -1).contiguous()
    lut = unique_values.to(w.dtype).contiguous()
    enc = features_enc.contiguous()
    out = torch.empty((B, Hq, 1, D), dtype=torch.float16, device=w.device)
    nbytes = lib().cq_lut_out_workspace_bytes(B, Hq, T)
    ws = _workspace(nbytes + 256, w.device)
    with torch.cuda.device(w.device):
        rc = lib().cq_lut_out(_ptr(lut), _ptr(w), _ptr(enc), _ptr(out), B, Hq, He, T, D, BITS, _dtype_enum(w),
                              ctypes.c_void_p(ws.data_ptr() + 256), nbytes, _stream())
    check(rc, "cq_lut_out")
    return out


def decode_attention(q, state, k_fp, v_fp, bits, sys_len, normalize=None, mask=None, t_fp_dev=None):
    """Decode step of the reference's calibquant forward (``patch_internvl.py:356-436``) on the uint8
    format as ONE library call of four launches: post-scaling (scale folded into the query, zero point
    into a scalar bias), logit calibration, fp32 softmax, the two code products, the full-precision
    system/text segments.  ``state`` holds ``enc_k, enc_v`` [B,Hkv,T,D*bits/8] and ``scale_key,
    zero_point_key, scale_value, zero_point_value`` as [B,Hq,1,D] (the reference's repeated layout) or
    [B,1,Hkv,D] / [B,Hkv,1,D] (one row per KV head).  ``k_fp``/``v_fp`` [B,Hkv,T_fp,D] hold
    [system | text]; ``mask`` is the optional additive mask [B,1,1,T] over [system | visual | text].
    With ``t_fp_dev`` (int32 device scalar) the live number of full-precision tokens is read on the device and
    ``k_fp``/``v_fp`` are the whole pre-allocated buffers, so that a captured CUDA graph serves every step.
    Returns [B,Hq,1,D] in bfloat16 as the reference does."""
    from ._lib import U8DecodeArgs
    _need_cuda(q, k_fp, v_fp)
    B, Hq, _, D = q.shape
    Hkv, t_fp = k_fp.shape[1], k_fp.shape[2]
    normalize = (bits <= 2) if normalize is None else normalize
    enc_k, enc_v = state["enc_k"].contiguous(), state["enc_v"].contiguous()
    t_vis = enc_k.shape[2]
    params = [state[n] for n in ("scale_key", "zero_point_key", "scale_value", "zero_point_value")]
    hs = params[0].numel() // (B * D)
    if hs not in (Hq, Hkv) or any(p.numel() != B * hs * D or p.dtype != q.dtype for p in params):
        raise ValueError("scale / zero point must hold one row of D values per query head or per KV head")
    params = [p.contiguous() for p in params]
    for t in (k_fp, v_fp):
        if t_fp and (t.stride(3) != 1 or t.stride(2) != D):
            raise ValueError("k_fp / v_fp token rows must be contiguous")
    q3 = q.reshape(B, Hq, D).contiguous()
    mask2 = None
    if mask is not None:
        mask2 = mask.reshape(B, -1).to(q.dtype).contiguous()
        if mask2.shape[1] != t_vis + t_fp:
            raise ValueError(f"mask must cover {t_vis + t_fp} keys, got {mask2.shape[1]}")
    out = torch.empty((B, Hq, 1, D), dtype=torch.bfloat16, device=q.device)
    a = U8DecodeArgs(batch=B, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, t_vis=t_vis, t_fp=t_fp, t_sys=sys_len,
                     bits=bits, dtype=_dtype_enum(q), calibrate=int(bool(normalize)), n_scale_heads=hs, reserved=0,
                     q=q3.data_ptr(), enc_k=enc_k.data_ptr(), enc_v=enc_v.data_ptr(),
                     scale_key=params[0].data_ptr(), zero_point_key=params[1].data_ptr(),
                     scale_value=params[2].data_ptr(), zero_point_value=params[3].data_ptr(),
                     k_fp=k_fp.data_ptr() if t_fp else None, v_fp=v_fp.data_ptr() if t_fp else None,
                     fp_stride_b=k_fp.stride(0), fp_stride_h=k_fp.stride(1),
                     mask=mask2.data_ptr() if mask2 is not None else None,
                     mask_stride_b=mask2.stride(0) if mask2 is not None else 0, out=out.data_ptr(),
                     t_fp_dev=t_fp_dev.data_ptr() if t_fp_dev is not None else None)
    if k_fp.stride() != v_fp.stride():
        raise ValueError("k_fp and v_fp must share strides")
    nbytes = lib().cq_u8_decode_attn_workspace_bytes(ctypes.byref(a))
    if nbytes == 0:
        raise ValueError("cq_u8_decode_attn rejects this request (sizes, head counts or more than 51200 keys)")
    ws = _workspace(nbytes + 256, q.device)
    with torch.cuda.device(q.device):
        rc = lib().cq_u8_decode_attn(ctypes.byref(a), ctypes.c_void_p(ws.data_ptr() + 256), nbytes, _stream())
    check(rc, "cq_u8_decode_attn")
    return out


def decode_attention_unfused(q, state, k_fp, v_fp, bits, sys_len, normalize=None):
    """The same step as the reference writes it: eager torch around ``fused_kernel`` and
    ``fused_kernel_wv``.  Kept as a cross-check of ``decode_attention``."""
    import math
    from .patch_internvl import repeat_kv
    n_rep = q.shape[1] // k_fp.shape[1]
    normalize = (bits <= 2) if normalize is None else normalize
    sd = math.sqrt(q.shape[-1])
    lut = torch.arange(2 ** bits, dtype=q.dtype, device=q.device)
    k, v = repeat_kv(k_fp, n_rep), repeat_kv(v_fp, n_rep)
    sk, zk, sv, zv = state["scale_key"], state["zero_point_key"], state["scale_value"], state["zero_point_value"]
    s_sys = torch.matmul(q, k[:, :, :sys_len].transpose(2, 3)) / sd
    s_txt = torch.matmul(q, k[:, :, sys_len:].transpose(2, 3)) / sd
    bias_k = torch.sum(sk * zk * q, dim=-1, keepdim=True) / sd
    s_vis = fused_kernel(lut, q * sk, state["enc_k"], bits, 8 // bits) / sd - bias_k
    if normalize:
        cur_max = s_vis.amax(dim=(2, 3), keepdim=True)
        cur_min = s_vis.amin(dim=(2, 3), keepdim=True)
        s_vis = (s_vis - cur_min) / (cur_max - cur_min + 1e-8) * ((cur_max + (-3)) - cur_min) + cur_min
    t_vis = s_vis.shape[-1]
    att = torch.softmax(torch.cat([s_sys, s_vis, s_txt], dim=-1), dim=-1, dtype=torch.float32).to(q.dtype)
    a_vis = att[..., sys_len:sys_len + t_vis]
    o_vis = fused_kernel_wv(lut.half(), a_vis.half().contiguous(), state["enc_v"], bits, 8 // bits) * sv
    o_vis = o_vis - sv * zv * torch.sum(a_vis, dim=-1, keepdim=True)
    o = o_vis + torch.matmul(att[..., :sys_len], v[:, :, :sys_len]) + torch.matmul(att[..., sys_len + t_vis:], v[:, :, sys_len:])
    return o.to(torch.bfloat16)
