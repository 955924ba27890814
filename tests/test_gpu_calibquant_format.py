"""CalibQuant uint8 format: quant / encode / fused_kernel / fused_kernel_wv drop-ins and the decode
composition vs the CPU oracle and the fixtures recorded from the reference itself.

quant / encode: bit-exact.  LUT products: fp32 accumulation in another order than the reference's
reduction, so <= 1 fp16 ulp per element (as the oracle itself vs the reference).  Decode: rel-L2
<= 1e-2 (the reference's output is bfloat16)."""

import os

import pytest
import torch

from oracle import calibquant_format as cqf
from oracle import generator
from gpu_util import bits_equal, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cq():
    from calibquant_b200 import calibquant as _cq
    return _cq


@pytest.fixture(scope="module")
def golden(golden_dir):
    return torch.load(os.path.join(golden_dir, "calibquant.pt"))


def _ulp_diff(a, b):
    return (a.cpu().view(torch.int16).int() - b.cpu().view(torch.int16).int()).abs()


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_golden_quant_encode_and_lut_kernels(cq, golden, bits):
    c = golden[f"b{bits}"]
    dpe = 8 // bits
    kq, sk, zk = cq.quant(c["k"].cuda(), bits, per_channel=True, scale=c["clip_k"], post_scale=True)
    vq, sv, zv = cq.quant(c["v"].cuda(), bits, per_channel=True, scale=c["clip_v"], post_scale=True)
    for mine, ref in ((kq, c["kq"]), (sk, c["sk"]), (zk, c["zk"]), (vq, c["vq"]), (sv, c["sv"]), (zv, c["zv"])):
        assert bits_equal(mine, ref)
    assert torch.equal(cq.encode(kq.transpose(1, 2).to(torch.int64), bits, dpe).cpu(), c["enc_k"])
    enc_v, sv2, zv2 = cq.quant_encode(c["v"].cuda(), bits, scale=c["clip_v"])
    assert torch.equal(enc_v.cpu(), c["enc_v"]) and bits_equal(sv2, c["sv"]) and bits_equal(zv2, c["zv"])
    lut = torch.arange(2 ** bits, dtype=torch.float16, device="cuda")
    s = cq.fused_kernel(lut, c["w_k"].cuda(), c["enc_k"].cuda(), bits, dpe)          # KV-head count enc
    o = cq.fused_kernel_wv(lut, c["w_v"].cuda(), c["enc_v"].cuda(), bits, dpe)
    # fp32 sums in another order, on the tensor core (whose fp32 accumulation truncates): within one fp16
    # rounding step of the reference's value plus 2e-5 of the sum of the terms' magnitudes (the second term
    # only matters where the terms cancel)
    codes_k = cqf.decode_bytes(c["enc_k"], bits).float().repeat_interleave(4, 1)
    codes_v = cqf.decode_bytes(c["enc_v"], bits).float().repeat_interleave(4, 1)
    mag_s = torch.einsum("bhd,bhtd->bht", c["w_k"][:, :, 0].float().abs(), codes_k).unsqueeze(2)
    mag_o = torch.einsum("bht,bhtd->bhd", c["w_v"][:, :, 0].float().abs(), codes_v).unsqueeze(2)
    for mine, ref, mag in ((s, c["scores"], mag_s), (o, c["out_v"], mag_o)):
        assert mine.shape == ref.shape and mine.dtype == torch.float16
        err = (mine.cpu().float() - ref.float()).abs()
        assert (err <= ref.float().abs() * 2.0 ** -10 + 2e-5 * mag).all()
    # enc expanded to the query heads, as the reference passes it
    rep = c["enc_k"][:, :, None].expand(-1, -1, 4, -1, -1).reshape(1, 8, *c["enc_k"].shape[2:]).contiguous()
    s_rep = cq.fused_kernel(lut, c["w_k"].cuda(), rep.cuda(), bits, dpe)
    assert ((s_rep.cpu().float() - s.cpu().float()).abs() <= s.cpu().float().abs() * 2.0 ** -10 + 2e-5 * mag_s).all()


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quant_dequant_paths(cq, bits, dtype):
    k, v, _ = generator.make_kvq(2, 8, 2, 130, seed=bits, dtype=dtype)
    x = k.transpose(1, 2).contiguous()                     # [B,T,H,D]
    ref_q = cqf.quant(x, bits, per_channel=True, scale=0.5, post_scale=True)
    ref_d = cqf.quant(x, bits, per_channel=True, scale=0.5, post_scale=False)
    got_q = cq.quant(x.cuda(), bits, per_channel=True, scale=0.5, post_scale=True)
    got_d = cq.quant(x.cuda(), bits, per_channel=True, scale=0.5, post_scale=False)
    for a, b in zip(got_q + got_d, ref_q + ref_d):
        assert bits_equal(a, b)
    # strided input: the [B,T,H,D] view of a [B,H,T,D] cache
    got_s = cq.quant(k.cuda().transpose(1, 2), bits, per_channel=True, scale=0.5, post_scale=True)
    assert bits_equal(got_s[0], ref_q[0])
    # per_channel=False: one scale and zero point for the whole tensor, returned as 0-dim tensors
    for post in (True, False):
        ref_t = cqf.quant(x, bits, per_channel=False, scale=0.5, post_scale=post)
        got_t = cq.quant(x.cuda(), bits, per_channel=False, scale=0.5, post_scale=post)
        assert got_t[1].dim() == 0 and got_t[2].dim() == 0
        for a, b in zip(got_t, ref_t):
            assert bits_equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T", [1000, 4096 + 40])
def test_quant_long_spans(cq, dtype, T):
    """Spans long enough for the sliced min/max reduction (token axis cut over many CTAs, ragged last
    slice), contiguous and as the [B,T,H,D] view of a [B,H,T,D] cache: bit-exact scale, zero point, codes
    and bytes."""
    k, _, _ = generator.make_kvq(2, 8, 2, T, seed=T % 97, dtype=dtype)
    x = k.transpose(1, 2).contiguous()                     # [B,T,H,D]
    ref = cqf.quant(x, 1, per_channel=True, scale=0.5, post_scale=True)
    for src in (x.cuda(), k.cuda().transpose(1, 2)):
        got = cq.quant(src, 1, per_channel=True, scale=0.5, post_scale=True)
        for a, b in zip(got, ref):
            assert bits_equal(a, b)
    enc, s, z = cq.quant_encode(x.cuda(), 2, scale=1)
    ref2 = cqf.quant(x, 2, per_channel=True, scale=1, post_scale=True)
    assert bits_equal(s, ref2[1]) and bits_equal(z, ref2[2])
    assert torch.equal(enc.cpu(), cqf.encode(ref2[0].transpose(1, 2).to(torch.int64), 2, 4))


@pytest.mark.parametrize("bits", [1, 2])
def test_quant_with_a_constant_channel(cq, bits):
    """A channel that is constant over the span has scale 0 (the reference divides by it): the kernel
    then computes that (batch, head) with the per-element arithmetic; every other channel stays bit-exact."""
    k, _, _ = generator.make_kvq(1, 8, 2, 300, seed=5)
    x = k.transpose(1, 2).contiguous()                     # [B,T,H,D]
    x[:, :, 1, 7] = 0.25
    ref = cqf.quant(x, bits, per_channel=True, scale=1, post_scale=True)
    got = cq.quant(x.cuda(), bits, per_channel=True, scale=1, post_scale=True)
    keep = torch.ones(128, dtype=torch.bool)
    keep[7] = False
    for a, b in zip(got, ref):
        a, b = a.cpu(), b
        assert bits_equal(a[:, :, 0], b[:, :, 0])
        assert bits_equal(a[:, :, 1][..., keep], b[:, :, 1][..., keep])
    assert float(got[1][0, 0, 1, 7]) == 0.0                # the degenerate scale itself


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_decode_composition(cq, bits):
    """Full decode step in the uint8 format against the oracle of patch_internvl.py:356-436."""
    sys_len, t_vis, t_txt, n_rep = 41, 416, 30, 4
    k, v, q = generator.make_kvq(2, 8, 2, sys_len + t_vis + t_txt, seed=30 + bits)
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis)
    clip_k, clip_v = (0.5, 0.3) if bits == 1 else (1, 1)
    ref_state = cqf.prefill_quantize(k_vis.transpose(1, 2), v_vis.transpose(1, 2), bits, clip_k, clip_v, n_rep)
    k_fp, v_fp = torch.cat([k_sys, k_txt], 2), torch.cat([v_sys, v_txt], 2)
    ref = cqf.decode_attention(q, ref_state, k_fp, v_fp, bits, sys_len)
    from calibquant_b200.patch_internvl import repeat_kv
    enc_k, sk, zk = cq.quant_encode(k_vis.cuda().transpose(1, 2), bits, scale=clip_k)
    enc_v, sv, zv = cq.quant_encode(v_vis.cuda().transpose(1, 2), bits, scale=clip_v)
    assert torch.equal(enc_k.cpu(), ref_state["enc_k"]) and torch.equal(enc_v.cpu(), ref_state["enc_v"])
    rep = lambda t: repeat_kv(t.transpose(1, 2), n_rep)
    state = {"enc_k": enc_k, "enc_v": enc_v, "scale_key": rep(sk), "zero_point_key": rep(zk),
             "scale_value": rep(sv), "zero_point_value": rep(zv)}
    out = cq.decode_attention(q.cuda(), state, k_fp.cuda(), v_fp.cuda(), bits, sys_len)
    assert out.dtype == torch.bfloat16 and out.shape == ref.shape
    assert rel_l2(out, ref) <= 1e-2, rel_l2(out, ref)


def _step_inputs(bits, B, Hq, Hkv, sys_len, t_vis, t_txt, dtype, seed):
    k, v, q = generator.make_kvq(B, Hq, Hkv, sys_len + t_vis + t_txt, seed=seed)
    k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
    clip_k, clip_v = (0.5, 0.3) if bits == 1 else (1, 1)
    state = cqf.prefill_quantize(k_vis.transpose(1, 2), v_vis.transpose(1, 2), bits, clip_k, clip_v, Hq // Hkv)
    return q, state, torch.cat([k_sys, k_txt], 2), torch.cat([v_sys, v_txt], 2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [1, 2, 4])
def test_fused_step_larger_shape_and_kv_head_scales(cq, bits, dtype):
    """The one-call step at 32 query heads on 8 KV heads and 4 096 visual tokens, against the oracle
    (tolerance 1e-2 rel-L2, the bar of the step) and against the eager composition around the two code
    products (2e-3: same arithmetic, different summation order); scale / zero point given once per query
    head (the reference's layout) and once per KV head must agree bit for bit."""
    sys_len, t_vis, t_txt, B, Hq, Hkv = 41, 4096, 77, 2, 32, 8
    q, state, k_fp, v_fp = _step_inputs(bits, B, Hq, Hkv, sys_len, t_vis, t_txt, dtype, seed=70 + bits)
    ref = cqf.decode_attention(q, state, k_fp, v_fp, bits, sys_len)
    dev = {n: t.cuda() for n, t in state.items()}
    out = cq.decode_attention(q.cuda(), dev, k_fp.cuda(), v_fp.cuda(), bits, sys_len)
    assert out.dtype == torch.bfloat16 and out.shape == ref.shape
    assert rel_l2(out, ref) <= 1e-2, rel_l2(out, ref)
    eager = cq.decode_attention_unfused(q.cuda(), dev, k_fp.cuda(), v_fp.cuda(), bits, sys_len)
    assert rel_l2(out, eager.cpu()) <= 4e-3, rel_l2(out, eager.cpu())
    per_kv = dict(dev)
    for n in ("scale_key", "zero_point_key", "scale_value", "zero_point_value"):
        per_kv[n] = dev[n][:, ::Hq // Hkv].contiguous()                   # [B,Hkv,1,D]
    out2 = cq.decode_attention(q.cuda(), per_kv, k_fp.cuda(), v_fp.cuda(), bits, sys_len)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_fused_step_mask_and_empty_spans(cq):
    """An additive mask that removes keys must equal the step on the remaining keys' probabilities
    (checked against the oracle with the same mask); no full-precision tokens and no visual tokens are
    both legal requests."""
    bits, sys_len, t_vis, t_txt = 2, 41, 512, 20
    q, state, k_fp, v_fp = _step_inputs(bits, 1, 8, 2, sys_len, t_vis, t_txt, torch.float16, seed=91)
    dev = {n: t.cuda() for n, t in state.items()}
    mask = torch.zeros(1, 1, 1, sys_len + t_vis + t_txt, dtype=torch.float16)
    mask[..., 5:9] = -60000.0
    mask[..., sys_len + 100:sys_len + 140] = -60000.0
    out = cq.decode_attention(q.cuda(), dev, k_fp.cuda(), v_fp.cuda(), bits, sys_len, mask=mask.cuda())
    # oracle with the mask: the same composition with the mask added before the softmax
    import math
    from oracle.group_format import repeat_kv, calibrate
    n_rep, sd = 4, math.sqrt(128)
    lut = torch.arange(2 ** bits, dtype=q.dtype)
    k, v = repeat_kv(k_fp, n_rep), repeat_kv(v_fp, n_rep)
    s_sys = torch.matmul(q, k[:, :, :sys_len].transpose(2, 3)) / sd
    s_txt = torch.matmul(q, k[:, :, sys_len:].transpose(2, 3)) / sd
    bias = torch.sum(state["scale_key"] * state["zero_point_key"] * q, dim=-1, keepdim=True) / sd
    s_vis = calibrate(cqf.fused_kernel(lut, q * state["scale_key"], repeat_kv(state["enc_k"], n_rep), bits) / sd - bias)
    att = torch.softmax(torch.cat([s_sys, s_vis, s_txt], -1) + mask, dim=-1, dtype=torch.float32).to(q.dtype)
    a_vis = att[..., sys_len:sys_len + t_vis]
    o = cqf.fused_kernel_wv(lut.half(), a_vis.half(), repeat_kv(state["enc_v"], n_rep), bits) * state["scale_value"]
    o = o - state["scale_value"] * state["zero_point_value"] * a_vis.sum(-1, keepdim=True)
    o = o + torch.matmul(att[..., :sys_len], v[:, :, :sys_len]) + torch.matmul(att[..., sys_len + t_vis:], v[:, :, sys_len:])
    assert rel_l2(out, o.to(torch.bfloat16)) <= 1e-2
    # no full-precision tokens
    empty = torch.empty(1, 2, 0, 128, dtype=torch.float16)
    ref = cqf.decode_attention(q, state, empty, empty, bits, 0)
    out = cq.decode_attention(q.cuda(), dev, empty.cuda(), empty.cuda(), bits, 0)
    assert rel_l2(out, ref) <= 1e-2
    # no visual tokens: plain attention over the full-precision tokens
    none = {n: t[:, :, :0].cuda() if n.startswith("enc") else t.cuda() for n, t in state.items()}
    out = cq.decode_attention(q.cuda(), none, k_fp.cuda(), v_fp.cuda(), bits, sys_len)
    att = torch.softmax((torch.matmul(q, k.transpose(2, 3)) / sd).float(), -1).to(q.dtype)
    assert rel_l2(out, torch.matmul(att, v).to(torch.bfloat16)) <= 1e-2


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("T", [130, 1024 + 72])
@pytest.mark.parametrize("lut_kind", ["identity", "affine", "arbitrary"])
def test_lut_kernels_ragged_lengths_and_luts(cq, bits, T, lut_kind):
    """The two LUT products on lengths that are not multiples of their tile sizes, with the identity
    LUT, a general affine one (both served by the tensor-core kernels) and an arbitrary one (scalar
    path inside the same kernels); 8 query heads on 2 code heads."""
    g = torch.Generator().manual_seed(100 * bits + T)
    dpe = 8 // bits
    codes = torch.randint(0, 2 ** bits, (1, 2, T, 128), generator=g)
    enc = cqf.encode(codes, bits, dpe)
    n = 2 ** bits
    lut = {"identity": torch.arange(n).float(),
           "affine": 0.75 - 0.5 * torch.arange(n).float(),
           "arbitrary": torch.tensor([0.5, -1.0, 3.0, 0.25, 2.0, -0.75, 1.5, 4.0, -2.0, 0.0, 1.0, 2.5, -3.0, 0.125, 6.0, -0.5])[:n]
           }[lut_kind].half()
    w_k = torch.randn(1, 8, 1, 128, generator=g).half()
    w_v = torch.softmax(torch.randn(1, 8, 1, T, generator=g), -1).half()
    s = cq.fused_kernel(lut.cuda(), w_k.cuda(), enc.cuda(), bits, dpe)
    o = cq.fused_kernel_wv(lut.cuda(), w_v.cuda(), enc.cuda(), bits, dpe)
    vals = lut.float()[codes].repeat_interleave(4, dim=1)                 # [1,8,T,128]
    ref_s = torch.einsum("bhd,bhtd->bht", w_k[:, :, 0].float(), vals).unsqueeze(2)
    ref_o = torch.einsum("bht,bhtd->bhd", w_v[:, :, 0].float(), vals).unsqueeze(2)
    assert s.shape == (1, 8, 1, T) and o.shape == (1, 8, 1, 128)
    assert torch.allclose(s.cpu().float(), ref_s, rtol=2e-3, atol=2e-3)
    assert torch.allclose(o.cpu().float(), ref_o, rtol=2e-3, atol=2e-3)
