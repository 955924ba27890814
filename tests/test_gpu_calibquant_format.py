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
    for mine, ref in ((s, c["scores"]), (o, c["out_v"])):
        assert mine.shape == ref.shape and mine.dtype == torch.float16
        assert _ulp_diff(mine, ref).max() <= 1
    # enc expanded to the query heads, as the reference passes it
    rep = c["enc_k"][:, :, None].expand(-1, -1, 4, -1, -1).reshape(1, 8, *c["enc_k"].shape[2:]).contiguous()
    assert torch.equal(cq.fused_kernel(lut, c["w_k"].cuda(), rep.cuda(), bits, dpe), s)


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
    with pytest.raises(NotImplementedError):
        cq.quant(x.cuda(), bits)


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
