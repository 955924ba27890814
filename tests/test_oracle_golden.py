"""The CPU oracle must reproduce, bit for bit, what the reference's own functions
returned when they were executed to build the fixtures (tests/golden/make_golden.py)."""

import os

import pytest
import torch

from oracle import calibquant_format as cqf
from oracle import group_format as gf


def _bits_equal(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape
    if a.dtype in (torch.float16, torch.bfloat16):
        return torch.equal(a.view(torch.int16), b.view(torch.int16))
    return torch.equal(a, b)


@pytest.fixture(scope="module")
def new_pack_golden(golden_dir):
    return torch.load(os.path.join(golden_dir, "new_pack.pt"))


@pytest.fixture(scope="module")
def calibquant_golden(golden_dir):
    return torch.load(os.path.join(golden_dir, "calibquant.pt"))


@pytest.mark.parametrize("layout", ["k", "v"])
@pytest.mark.parametrize("dname", ["f16", "bf16"])
@pytest.mark.parametrize("bit", [1, 2, 4])
def test_pack_matches_reference(new_pack_golden, layout, dname, bit):
    case = new_pack_golden[f"{layout}_{dname}_b{bit}"]
    code, scale, mn = gf.quantize_and_pack_last_dim(case["data"], 32, bit)
    assert _bits_equal(code, case["code"])
    assert _bits_equal(scale, case["scale"])
    assert _bits_equal(mn, case["mn"])


@pytest.mark.parametrize("bit", [1, 2, 4])
def test_unpack_roundtrip(new_pack_golden, bit):
    case = new_pack_golden[f"v_f16_b{bit}"]
    codes = gf.unpack_codes(case["code"], bit)
    assert codes.min() >= 0 and codes.max() <= 2 ** bit - 1
    deq = gf.dequantize(case["code"], case["scale"], case["mn"], bit, 32)
    err = (deq - case["data"].float()).abs()
    step = case["scale"].float().repeat_interleave(32, dim=-1)
    assert (err <= 0.5 * step + 1e-2 * step + 1e-3).all()


@pytest.mark.parametrize("bit", [1, 2, 4])
def test_calibquant_quant_encode(calibquant_golden, bit):
    c = calibquant_golden[f"b{bit}"]
    kq, sk, zk = cqf.quant(c["k"], bit, per_channel=True, scale=c["clip_k"], post_scale=True)
    vq, sv, zv = cqf.quant(c["v"], bit, per_channel=True, scale=c["clip_v"], post_scale=True)
    for mine, ref in ((kq, c["kq"]), (sk, c["sk"]), (zk, c["zk"]),
                      (vq, c["vq"]), (sv, c["sv"]), (zv, c["zv"])):
        assert _bits_equal(mine, ref)
    dpe = 8 // bit
    assert torch.equal(cqf.encode(kq.transpose(1, 2), bit, dpe), c["enc_k"])
    assert torch.equal(cqf.encode(vq.transpose(1, 2), bit, dpe), c["enc_v"])
    assert torch.equal(cqf.decode_bytes(c["enc_k"], bit), kq.transpose(1, 2).to(torch.int64))


def test_encode_known_bytes():
    # MSB-first packing: 8 one-bit fields 1,0,0,1,1,1,1,0 -> 0b10011110; 2-bit 2,1,0,2 -> 0b10010010
    one = torch.tensor([1, 0, 0, 1, 1, 1, 1, 0]).view(1, 1, 1, 8)
    two = torch.tensor([2, 1, 0, 2]).view(1, 1, 1, 4)
    assert cqf.encode(one, 1, 8).item() == 158
    assert cqf.encode(two, 2, 4).item() == 146


@pytest.mark.parametrize("bit", [1, 2, 4])
def test_calibquant_fused_kernels(calibquant_golden, bit):
    c = calibquant_golden[f"b{bit}"]
    lut = torch.arange(2 ** bit, dtype=torch.float16)
    rep = lambda t: gf.repeat_kv(t, 4)
    s = cqf.fused_kernel(lut, c["w_k"], rep(c["enc_k"]), bit)
    o = cqf.fused_kernel_wv(lut, c["w_v"], rep(c["enc_v"]), bit)
    # fp32 accumulation order differs between the Triton reduction and a matmul:
    # agree to one fp16 ulp on every element, exactly on nearly all of them.
    for mine, ref in ((s, c["scores"]), (o, c["out_v"])):
        assert mine.dtype == ref.dtype == torch.float16 and mine.shape == ref.shape
        ulp = (mine.view(torch.int16).int() - ref.view(torch.int16).int()).abs()
        assert ulp.max() <= 1
        assert (ulp == 0).float().mean() > 0.98
