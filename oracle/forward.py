"""Oracle for the patched attention forward (test infrastructure).

CPU restatement of ``forward_internlm2_calibquant`` (``patch_internvl.py:141-484``) with the
quantized state in the group format or (``kv_format="uint8"``) in the reference's own byte format
(``:288-339`` prefill, ``:356-436`` decode), and of the decode arithmetic of ``forward_internlm2_qjl``
(``:544-600``) with per-channel group-quantized keys.  Weights are passed in explicitly; all
tensor ops run in the weight dtype on CPU, the attention core in the oracle functions of
``group_format`` / ``prefill``.
"""

from __future__ import annotations

import math

import torch

from . import calibquant_format as cqf
from . import group_format as gf
from . import prefill as pf


def rope_tables(head_dim, base, seq_len, dtype):
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32)
    emb = torch.cat([torch.outer(t, inv)] * 2, dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x, cos, sin, position_ids):
    """x [B,H,q,D]; ``copy.mul_(cos)`` then ``addcmul_(rotate_half(x), sin)`` as
    ``patch_internvl.py:118-137``."""
    c = cos[position_ids].unsqueeze(1)
    s = sin[position_ids].unsqueeze(1)
    return torch.addcmul(x * c, rotate_half(x), s)


class AttentionOracle:
    """One attention layer: prefill once, then decode steps; mirrors the module state of the
    reference (fp cache of system+text tokens, quantized visual span kept on the object)."""

    def __init__(self, wqkv, wo, n_heads, n_kv_heads, head_dim=128, rope_base=1e6, bits=1, sys_len=41,
                 group_size=32, calibrate=None, kv_format="group"):
        self.kv_format = kv_format
        self.wqkv, self.wo = wqkv, wo
        self.hq, self.hkv, self.d = n_heads, n_kv_heads, head_dim
        self.n_rep = n_heads // n_kv_heads
        self.base, self.bits, self.sys_len, self.g = rope_base, bits, sys_len, group_size
        self.calibrate = (bits <= 2) if calibrate is None else calibrate

    def _qkv(self, h, position_ids, kv_len):
        B, T, _ = h.shape
        qkv = torch.nn.functional.linear(h, self.wqkv).view(B, T, self.hkv, self.n_rep + 2, self.d)
        q = qkv[..., : self.n_rep, :].reshape(B, T, self.hq, self.d).transpose(1, 2)
        k = qkv[..., -2, :].transpose(1, 2)
        v = qkv[..., -1, :].transpose(1, 2)
        cos, sin = rope_tables(self.d, self.base, kv_len, h.dtype)
        return apply_rope(q, cos, sin, position_ids), apply_rope(k, cos, sin, position_ids), v

    def prefill(self, h, image_token_num):
        B, T, _ = h.shape
        pos = torch.arange(T).unsqueeze(0).expand(B, T)
        q, k, v = self._qkv(h, pos, T)
        s0, s1 = self.sys_len, self.sys_len + image_token_num
        self.t_vis = image_token_num
        if self.kv_format == "uint8":
            clip_k, clip_v = (0.5, 0.3) if self.bits == 1 else (1, 1)        # patch_internvl.py:22-27
            self.u8 = cqf.prefill_quantize(k[:, :, s0:s1].transpose(1, 2), v[:, :, s0:s1].transpose(1, 2), self.bits,
                                           clip_k, clip_v, self.n_rep)
        self.k_pack = gf.quantize_and_pack_last_dim(k[:, :, s0:s1].transpose(2, 3).contiguous(), self.g, self.bits)
        self.v_pack = gf.quantize_and_pack_last_dim(v[:, :, s0:s1].contiguous(), self.g, self.bits)
        self.k_fp = torch.cat([k[:, :, :s0], k[:, :, s1:]], dim=2)
        self.v_fp = torch.cat([v[:, :, :s0], v[:, :, s1:]], dim=2)
        self.pos = T
        o = pf.causal_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return torch.nn.functional.linear(o.reshape(B, T, self.hq * self.d), self.wo)

    def decode(self, h):
        B = h.shape[0]
        pos = torch.full((B, 1), self.pos, dtype=torch.long)
        q, k, v = self._qkv(h, pos, self.pos + 1)
        self.pos += 1
        self.k_fp = torch.cat([self.k_fp, k], dim=2)
        self.v_fp = torch.cat([self.v_fp, v], dim=2)
        s = self.sys_len
        if self.kv_format == "uint8":
            o = cqf.decode_attention(q, self.u8, self.k_fp, self.v_fp, self.bits, s, normalize=self.calibrate).to(h.dtype)
            return torch.nn.functional.linear(o.transpose(1, 2).reshape(B, 1, self.hq * self.d), self.wo)
        o = gf.decode_attention(q, self.k_pack, self.v_pack, self.k_fp[:, :, :s], self.k_fp[:, :, s:],
                                self.v_fp[:, :, :s], self.v_fp[:, :, s:], self.bits, self.g,
                                calibrated=self.calibrate)
        return torch.nn.functional.linear(o.transpose(1, 2).reshape(B, 1, self.hq * self.d), self.wo)
