"""Seeded synthetic K/V/q generator (test infrastructure).

Stands in for real InternVL2.5 image+prompt KV caches: the reference evaluates on
no dataset inside its repository, so shapes come from its own constants
(41 system-prompt tokens, ``patch_internvl.py:30``; 13 image tiles,
``infer.py:168,216``) and values from a fixed distribution: K, V ~ N(0,1), K
multiplied by a per-channel lognormal(0,1) factor so that a few channels are
outliers (the property per-channel K quantization is designed for), q ~ N(0,1).

Everything is drawn in fp32 from one ``torch.Generator('cpu')`` in a fixed order
and then cast, so any (seed, shape) can be regenerated bit-identically anywhere.
"""

from __future__ import annotations

import torch

SYS_LEN = 41  # patch_internvl.py:30 (SPROMPT_LEN)


def make_kvq(batch, n_q_heads, n_kv_heads, t_total, head_dim=128, seed=0,
             dtype=torch.float16):
    """Return (K [B,Hkv,T,D], V [B,Hkv,T,D], q [B,Hq,1,D]) in ``dtype`` on CPU.

    Draw order: K, V, channel factor f (lognormal), q.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    k = torch.randn(batch, n_kv_heads, t_total, head_dim, generator=g)
    v = torch.randn(batch, n_kv_heads, t_total, head_dim, generator=g)
    f = torch.exp(torch.randn(head_dim, generator=g))
    q = torch.randn(batch, n_q_heads, 1, head_dim, generator=g)
    return (k * f).to(dtype), v.to(dtype), q.to(dtype)


def row_seed(seed, row):
    """Per-batch-row seed for large configurations, so one row can be rebuilt alone."""
    return seed * 1_000_003 + row


def split_spans(x, t_vis, sys_len=SYS_LEN):
    """Split [B,H,T,D] along T into (sys, visual, text) following the reference's
    token layout ``[sys | visual | text]`` (``patch_internvl.py:268-273``)."""
    return x[:, :, :sys_len], x[:, :, sys_len:sys_len + t_vis], x[:, :, sys_len + t_vis:]
