"""Decode-step glue kernels (QKV split + RoPE + cache append, residual add + RMSNorm, SwiGLU)
against the torch ops they replace, through the C ABI."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]


def _rope_tables(seq, dim, dtype, base=1e6):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    emb = torch.cat([torch.outer(torch.arange(seq, dtype=torch.float32), inv)] * 2, dim=-1)
    return emb.cos().to(dtype).cuda(), emb.sin().to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("counter_on_device", [False, True])
def test_rope_split_append_bit_exact(dtype, counter_on_device):
    from calibquant_b200 import ops
    from calibquant_b200.patch_internvl import apply_rotary_pos_emb
    B, Hkv, n_rep, D, cap, length = 3, 2, 4, 128, 24, 17
    g = torch.Generator().manual_seed(5)
    qkv = (torch.randn(B, 1, Hkv * (n_rep + 2) * D, generator=g) * 2).to(dtype).cuda()
    cos, sin = _rope_tables(600, D, dtype)
    pos = torch.tensor([[5], [333], [599]], dtype=torch.int64, device="cuda")
    kc = torch.randn(B, Hkv, cap, D, generator=g).to(dtype).cuda()
    vc = torch.randn(B, Hkv, cap, D, generator=g).to(dtype).cuda()
    kc_ref, vc_ref = kc.clone(), vc.clone()

    v5 = qkv.view(B, 1, Hkv, n_rep + 2, D)
    q_ref = v5[..., :n_rep, :].reshape(B, 1, Hkv * n_rep, D).transpose(1, 2)
    k_ref, v_ref = v5[..., -2, :].transpose(1, 2), v5[..., -1, :].transpose(1, 2)
    q_ref, k_ref = apply_rotary_pos_emb(q_ref, k_ref, cos, sin, pos)
    kc_ref[:, :, length] = k_ref[:, :, 0]
    vc_ref[:, :, length] = v_ref[:, :, 0]

    if counter_on_device:
        live = torch.tensor([length + 1], dtype=torch.int32, device="cuda")   # counts the new token
        q = ops.rope_split_append(qkv, cos, sin, pos, Hkv, n_rep, kc, vc, t_fp_dev=live)
    else:
        q = ops.rope_split_append(qkv, cos, sin, pos, Hkv, n_rep, kc, vc, append_index=length)
    assert q.shape == (B, Hkv * n_rep, 1, D)
    assert torch.equal(q, q_ref)
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)


def test_rope_split_append_full_cache_writes_nothing():
    from calibquant_b200 import ops
    B, Hkv, n_rep, D, cap = 1, 1, 4, 128, 8
    qkv = torch.randn(B, 1, Hkv * (n_rep + 2) * D).half().cuda()
    cos, sin = _rope_tables(16, D, torch.float16)
    pos = torch.zeros(B, 1, dtype=torch.int64, device="cuda")
    kc = torch.zeros(B, Hkv, cap, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    live = torch.tensor([cap + 1], dtype=torch.int32, device="cuda")
    ops.rope_split_append(qkv, cos, sin, pos, Hkv, n_rep, kc, vc, t_fp_dev=live)
    assert not kc.any() and not vc.any()
    with pytest.raises(ValueError):
        ops.rope_split_append(qkv, cos, sin, pos, Hkv, n_rep, kc, vc, append_index=cap)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [512, 4096, 6144])
def test_add_rmsnorm_matches_torch(dtype, hidden):
    from calibquant_b200 import ops
    from calibquant_b200.internlm2 import RMSNorm
    g = torch.Generator().manual_seed(hidden)
    h = torch.randn(5, 1, hidden, generator=g).to(dtype).cuda()
    d = (torch.randn(5, 1, hidden, generator=g) * 0.5).to(dtype).cuda()
    norm = RMSNorm(hidden, 1e-5).to(dtype).cuda()
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype))
        h_ref = h + d
        x_ref = norm(h_ref)
        x_plain_ref = norm(h)
    x_plain = ops.add_rmsnorm(h.clone(), None, norm.weight.detach(), 1e-5)
    h_io = h.clone()
    x = ops.add_rmsnorm(h_io, d, norm.weight.detach(), 1e-5)
    assert torch.equal(h_io, h_ref)                      # the residual stream is bit-exact
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    for got, ref in ((x, x_ref), (x_plain, x_plain_ref)):
        # fp32 sum of squares in a different order: at most one rounding step apart, on few elements
        assert (got.float() - ref.float()).abs().le(ref.float().abs() * 2 * ulp + 1e-6).all()
        assert (got != ref).float().mean() < 0.02
    # bare residual add
    h_io2 = h.clone()
    assert ops.add_rmsnorm(h_io2, d, None, 1e-5, normalize=False) is None
    assert torch.equal(h_io2, h_ref)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_matches_torch(dtype):
    from calibquant_b200 import ops
    g = torch.Generator().manual_seed(11)
    a = (torch.randn(16, 1, 14336, generator=g) * 3).to(dtype).cuda()
    b = torch.randn(16, 1, 14336, generator=g).to(dtype).cuda()
    ref = torch.nn.functional.silu(a) * b
    got = ops.swiglu(a, b)
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert (got.float() - ref.float()).abs().le(ref.float().abs() * 2 * ulp + 1e-7).all()
    assert (got != ref).float().mean() < 1e-3            # exp may differ in the last fp32 bit


def test_fused_step_equals_layerwise_step():
    """forward_step_fused (fused elementwise blocks) against forward_step on the same caches."""
    import os
    from calibquant_b200 import patch_internvl as pi
    from calibquant_b200.internlm2 import ChatModelShell, GraphedDecoder, InternLM2Config, init_weights_
    cfg = InternLM2Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=1,
                          intermediate_size=1024, num_hidden_layers=2, vocab_size=128)
    shell = ChatModelShell(cfg).half()
    init_weights_(shell, 3, std=0.05)
    pi.patch_model(shell, "calibquant")
    shell.cuda()
    lm = shell.language_model
    g = torch.Generator().manual_seed(4)
    T, t_vis, n_new = 41 + 256 + 7, 256, 5
    emb = (torch.randn(2, T, 512, generator=g) * 0.3).half().cuda()
    os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
    pos = torch.arange(T, device="cuda").unsqueeze(0).expand(2, T)
    out = {}
    for fused in (False, True):
        with torch.no_grad():
            logits, past = lm.forward_step(emb, pos, None)
        dec = GraphedDecoder(lm, past, logits[:, -1].argmax(-1), T, n_new, fused=fused)
        out[fused] = dec.run(n_new - 1).clone()
        dec.close()
    assert torch.equal(out[False], out[True])
