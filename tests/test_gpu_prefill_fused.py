"""Prefill split + rotary embedding + cache fill in one launch, and the strided per-token V pack.

The launch replaces, for a whole prompt, the QKV split, `apply_rotary_pos_emb` and the concatenations
that build the full-precision system+text cache (patch_internvl.py:214-260, :281-284); the strided V
pack replaces `pack_last_dim(v[:, :, s0:s1].contiguous())` (:271).  Both are checked bit for bit
against the unfused composition in torch + the existing pack kernels (tolerance: none).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tables(T, D, dtype):
    inv = 1.0 / (1000000.0 ** (torch.arange(0, D, 2, dtype=torch.float32, device="cuda") / D))
    f = torch.outer(torch.arange(T, dtype=torch.float32, device="cuda"), inv)
    emb = torch.cat([f, f], -1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("B,T,Hkv,n_rep,s0,n_vis", [(2, 333, 2, 4, 7, 256), (1, 1100, 8, 4, 35, 1024),
                                                   (3, 64, 1, 6, 0, 64), (2, 40, 2, 1, 5, 0)])
def test_fused_prefill_matches_unfused(dtype, bits, B, T, Hkv, n_rep, s0, n_vis):
    from calibquant_b200 import ops
    from calibquant_b200.patch_internvl import apply_rotary_pos_emb
    D = 128
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + T)
    qkv = (torch.randn(B, T, Hkv * (n_rep + 2) * D, generator=g, device="cuda") * 1.5).to(dtype)
    cos, sin = _tables(T + 5, D, dtype)
    pos = torch.arange(T, device="cuda").unsqueeze(0).expand(B, T).contiguous()
    if B > 1:
        pos = pos.clone()
        pos[1] += 3                                   # rows need not share positions

    v5 = qkv.view(B, T, Hkv, n_rep + 2, D)
    q_ref = v5[..., :n_rep, :].reshape(B, T, Hkv * n_rep, D).transpose(1, 2)
    k_ref, v_ref = v5[..., -2, :].transpose(1, 2), v5[..., -1, :].transpose(1, 2)
    q_ref, k_ref = apply_rotary_pos_emb(q_ref, k_ref, cos, sin, pos)
    s1 = s0 + n_vis
    k_text = torch.cat([k_ref[:, :, :s0], k_ref[:, :, s1:]], 2)
    v_text = torch.cat([v_ref[:, :, :s0], v_ref[:, :, s1:]], 2)

    cap = T - n_vis + 9
    kc = torch.full((B, Hkv, cap, D), float("nan"), dtype=dtype, device="cuda")
    vc = torch.full_like(kc, float("nan"))
    q, k, v = ops.prefill_rope_split(qkv, cos, sin, pos, Hkv, n_rep, kc, vc, s0, n_vis)
    bits_of = lambda t: t.contiguous().view(torch.int16)
    assert torch.equal(bits_of(q), bits_of(q_ref.transpose(1, 2)))
    assert torch.equal(bits_of(k), bits_of(k_ref.transpose(1, 2)))
    assert torch.equal(bits_of(v), bits_of(v_ref.transpose(1, 2)))
    assert torch.equal(bits_of(kc[:, :, :T - n_vis]), bits_of(k_text))
    assert torch.equal(bits_of(vc[:, :, :T - n_vis]), bits_of(v_text))
    assert torch.isnan(kc[:, :, T - n_vis:].float()).all()           # rows past the prompt stay untouched

    if n_vis:
        want_k = ops.pack_k_per_channel(k_ref[:, :, s0:s1], 32, bits)
        got_k = ops.pack_k_per_channel(k.transpose(1, 2)[:, :, s0:s1], 32, bits)
        want_v = ops.pack_last_dim(v_ref[:, :, s0:s1].contiguous(), 32, bits)
        got_v = ops.pack_v_per_token(v.transpose(1, 2)[:, :, s0:s1], 32, bits)
        for a, b in zip(want_k + want_v, got_k + got_v):
            assert a.shape == b.shape
            assert torch.equal(a.view(torch.int32) if a.dtype == torch.int32 else a.view(torch.int16),
                               b.view(torch.int32) if b.dtype == torch.int32 else b.view(torch.int16))


def test_default_positions_and_no_cache():
    from calibquant_b200 import ops
    B, T, Hkv, n_rep, D = 2, 50, 2, 4, 128
    qkv = torch.randn(B, T, Hkv * (n_rep + 2) * D, device="cuda").half()
    cos, sin = _tables(T, D, torch.float16)
    pos = torch.arange(T, device="cuda").unsqueeze(0).expand(B, T).contiguous()
    a = ops.prefill_rope_split(qkv, cos, sin, pos, Hkv, n_rep)
    b = ops.prefill_rope_split(qkv, cos, sin, None, Hkv, n_rep)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_rejects_bad_span():
    from calibquant_b200 import ops
    qkv = torch.randn(1, 8, 2 * 6 * 128, device="cuda").half()
    cos, sin = _tables(8, 128, torch.float16)
    kc = torch.empty(1, 2, 16, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        ops.prefill_rope_split(qkv, cos, sin, None, 2, 4, kc, kc.clone(), 4, 8)   # span runs past the prompt
