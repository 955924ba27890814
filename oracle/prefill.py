"""Oracle for dense causal prefill attention (test infrastructure).

The reference delegates prefill attention to the third-party flash_attn library
(``patch_internvl.py:464-468`` through InternVL's ``_flash_attention_forward``, and
``:606-609``), in 1024-query chunks against the growing K/V prefix, which is just
causal attention.  flash_attn is not part of the reference tree and needs a GPU, so
this file restates the published definition -- softmax(Q K^T / sqrt(D) + causal
mask) V with GQA head sharing -- in fp32.  The reference has no test or vector for it;
where the flash_attn package is installed and runs on the test GPU,
``tests/test_gpu_prefill.py::test_against_the_flash_attn_library`` pins this file and the
library's kernel to ``flash_attn_func(causal=True)`` on seeded tensors.
"""

from __future__ import annotations

import math

import torch


def causal_attention(q, k, v):
    """q [B,T,Hq,D], k/v [B,T,Hkv,D] (flash_attn layout) -> o [B,T,Hq,D] in q.dtype."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    n_rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)                               # [B,Hq,T,D]
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(n_rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(n_rep, dim=1)
    s = torch.matmul(qf, kf.transpose(2, 3)) / math.sqrt(D)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    o = torch.matmul(torch.softmax(s, dim=-1), vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)
