"""Oracle for the group-wise (KIVI-style) int32 format (test infrastructure).

Restates on CPU, with the same per-operation rounding the reference gets from
running dtype-typed torch ops, the following reference pieces:

* ``quantize_and_pack_last_dim``  <- ``qjl/new_pack.py:53-82`` (+ kernels :7-50)
* ``qbmm``                        <- ``qjl/matmul.py:4-35`` and the arithmetic of
                                    ``qjl/csrc/quantization.cu:108-123``
* ``repeat_kv``                   <- ``qjl/qjl_utils.py:6-11``, ``patch_internvl.py:97-106``
* ``calibrate``                   <- ``patch_internvl.py:376-385``
* ``decode_attention``            <- the decode step ``patch_internvl.py:556-592``
                                    with the calibration of ``:376-385`` on the
                                    visual logits when bits <= 2

Format facts (all from ``qjl/new_pack.py``): groups are ``group_size`` consecutive
elements of the last dim; ``mn``/``mx`` keep the data dtype; ``scale = (mx-mn)/(2^b-1)``;
``code = round_half_even(clamp((x-mn)/scale, 0, 2^b-1))``; 32/b codes per int32,
element i of a word in bits [i*b, (i+1)*b) (least significant first).

One deliberate difference: a constant group (mx == mn) makes the reference divide
0/0 and convert NaN to an integer, whose value is platform-defined.  Here (and in
the CUDA kernel) such a group gets code 0; its dequantized value ``0*0 + mn`` is
still exact.
"""

from __future__ import annotations

import math

import torch


def quantize_and_pack_last_dim(data: torch.Tensor, group_size: int, bit: int):
    """(code int32 [B,nh,R,L*bit/32], scale [B,nh,R,L/g], mn [B,nh,R,L/g])."""
    assert data.dim() == 4
    B, nh, R, L = data.shape
    assert L % group_size == 0
    fpi = 32 // bit
    assert L % fpi == 0
    levels = 2 ** bit - 1
    x = data.reshape(B * nh * R, L // group_size, group_size)
    mn = x.amin(dim=-1)
    mx = x.amax(dim=-1)
    scale = (mx - mn) / levels                 # two rounded ops in data dtype
    y = x - mn.unsqueeze(-1)                   # rounded
    constant = (mx == mn).unsqueeze(-1)
    safe = torch.where(constant.squeeze(-1), torch.ones_like(scale), scale)
    y = y / safe.unsqueeze(-1)                 # rounded, IEEE division
    y = y.clamp(0, levels).round()             # round half to even
    codes = torch.where(constant, torch.zeros_like(y), y).to(torch.int64)
    codes = codes.reshape(B * nh * R, L // fpi, fpi)
    shifts = torch.arange(fpi, dtype=torch.int64) * bit
    words = (codes << shifts).sum(dim=-1)      # disjoint bit fields: sum == OR
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    shp = (B, nh, R, L // group_size)
    return words.reshape(B, nh, R, L // fpi), scale.reshape(shp), mn.reshape(shp)


def unpack_codes(code: torch.Tensor, bit: int) -> torch.Tensor:
    """int32 words [..., W] -> integer codes [..., W*32/bit] (int64)."""
    fpi = 32 // bit
    w = code.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(fpi, dtype=torch.int64) * bit
    c = (w.unsqueeze(-1) >> shifts) & (2 ** bit - 1)
    return c.reshape(*code.shape[:-1], code.shape[-1] * fpi)


def dequantize(code, scale, mn, bit, group_size):
    """fp32 ``scale*code + mn`` (``qjl/csrc/quantization.cu:117``)."""
    c = unpack_codes(code, bit).to(torch.float32)
    s = scale.to(torch.float32).repeat_interleave(group_size, dim=-1)
    z = mn.to(torch.float32).repeat_interleave(group_size, dim=-1)
    return s * c + z


def qbmm(group_size, fA, qB, scales, zeros, bits):
    """out[b,h,m,n] = sum_k fA[b,h,m,k] * (scales[b,h,k,n/g]*code[b,h,k,n] + zeros[b,h,k,n/g]).

    fp32 accumulation, result cast to ``fA.dtype`` (``quantization.cu:116-129``).
    Valid for bits in {1,2,4}; the reference itself cannot run bits == 1.
    """
    w = dequantize(qB, scales, zeros, bits, group_size)       # [B,nh,K,N] fp32
    return torch.matmul(fA.to(torch.float32), w).to(fA.dtype)


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B,Hkv,S,X] -> [B,Hkv*n_rep,S,X]; q head j reads KV head j // n_rep."""
    if n_rep == 1:
        return x
    B, H, S, X = x.shape
    return x[:, :, None].expand(B, H, n_rep, S, X).reshape(B, H * n_rep, S, X)


def calibrate(s_vis: torch.Tensor) -> torch.Tensor:
    """Logit calibration of the visual scores, every op rounded to ``s_vis.dtype``.

    Per (batch, q head): remap [min, max] affinely onto [min, max-3].
    """
    cur_max = s_vis.amax(dim=(2, 3), keepdim=True)
    cur_min = s_vis.amin(dim=(2, 3), keepdim=True)
    tgt_max = cur_max + (-3)
    tgt_min = cur_min + 0
    n = (s_vis - cur_min) / (cur_max - cur_min + 1e-8)
    return n * (tgt_max - tgt_min) + tgt_min


def decode_attention(q, k_pack, v_pack, k_sys, k_txt, v_sys, v_txt, bits,
                     group_size=32, calibrated=None, return_parts=False):
    """One decode step of attention over ``[sys | visual(quantized) | text]``.

    q [B,Hq,1,D]; k_pack = (code [B,Hkv,D,Tv*b/32], scale, mn [B,Hkv,D,Tv/g]) -- K
    quantized per channel; v_pack = (code [B,Hkv,Tv,D*b/32], scale, mn [B,Hkv,Tv,D/g])
    -- V per token; k_sys/k_txt/v_sys/v_txt [B,Hkv,*,D] in q.dtype.
    Returns o [B,Hq,1,D] in q.dtype.
    """
    B, Hq, _, D = q.shape
    n_rep = Hq // k_sys.shape[1]
    if calibrated is None:
        calibrated = bits <= 2                      # patch_internvl.py:191
    rep = lambda t: repeat_kv(t, n_rep)
    sqrt_d = math.sqrt(D)
    kc, ks, kmn = k_pack
    vc, vs, vmn = v_pack
    t_vis = vc.shape[2]
    s_vis = qbmm(group_size, q, rep(kc), rep(ks), rep(kmn), bits)       # [B,Hq,1,Tv]
    s_sys = torch.matmul(q, rep(k_sys).transpose(2, 3))
    s_txt = torch.matmul(q, rep(k_txt).transpose(2, 3))
    s_vis, s_sys, s_txt = s_vis / sqrt_d, s_sys / sqrt_d, s_txt / sqrt_d
    if calibrated:
        s_vis = calibrate(s_vis)
    n_sys = s_sys.shape[-1]
    logits = torch.cat([s_sys, s_vis, s_txt], dim=-1)
    att = torch.softmax(logits, dim=-1, dtype=torch.float32).to(q.dtype)
    att_vis = att[..., n_sys:n_sys + t_vis]
    o = qbmm(group_size, att_vis, rep(vc), rep(vs), rep(vmn), bits)
    o = o + (torch.matmul(att[..., n_sys + t_vis:], rep(v_txt))
             + torch.matmul(att[..., :n_sys], rep(v_sys)))
    if return_parts:
        return o, logits, att
    return o


def decode_attention_from_fp(q, k, v, t_vis, bits, sys_len, group_size=32, calibrated=None):
    """Quantize the visual span of fp K/V ([B,Hkv,T,D]) and run ``decode_attention``."""
    k_sys, k_vis, k_txt = (k[:, :, :sys_len], k[:, :, sys_len:sys_len + t_vis],
                           k[:, :, sys_len + t_vis:])
    v_sys, v_vis, v_txt = (v[:, :, :sys_len], v[:, :, sys_len:sys_len + t_vis],
                           v[:, :, sys_len + t_vis:])
    k_pack = quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), group_size, bits)
    v_pack = quantize_and_pack_last_dim(v_vis.contiguous(), group_size, bits)
    o = decode_attention(q, k_pack, v_pack, k_sys, k_txt, v_sys, v_txt, bits,
                         group_size, calibrated)
    return o, k_pack, v_pack
