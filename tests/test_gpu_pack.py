"""Quantize+pack kernels vs the CPU oracle: codes, scales and minima must be bit-identical."""

import os

import pytest
import torch

from oracle import generator
from oracle import group_format as gf
from gpu_util import bits_equal, mismatch_count

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from calibquant_b200 import ops as _ops
    return _ops


def _check(pack, ref):
    names = ("code", "scale", "mn")
    for n, a, b in zip(names, pack, ref):
        assert bits_equal(a, b), f"{n}: {mismatch_count(a, b)} mismatches of {b.numel()}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [1, 2, 4])
def test_golden_fixtures(ops, golden_dir, dtype, bits):
    g = torch.load(os.path.join(golden_dir, "new_pack.pt"))
    dn = "f16" if dtype == torch.float16 else "bf16"
    for layout in ("k", "v"):
        c = g[f"{layout}_{dn}_b{bits}"]
        _check(ops.pack_last_dim(c["data"].cuda(), 32, bits), (c["code"], c["scale"], c["mn"]))
    ck = g[f"k_{dn}_b{bits}"]
    k_tok_major = ck["data"].transpose(2, 3).contiguous().cuda()       # back to [B,H,T,D]
    _check(ops.pack_k_per_channel(k_tok_major, 32, bits), (ck["code"], ck["scale"], ck["mn"]))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [1, 2, 4])
def test_config0_shapes(ops, dtype, bits):
    """Config-0 generator: B=1, 8 KV heads, 3328 visual tokens, D=128, outlier K channels."""
    k, v, _ = generator.make_kvq(1, 32, 8, 4096, seed=0, dtype=dtype)
    _, k_vis, _ = generator.split_spans(k, 3328)
    _, v_vis, _ = generator.split_spans(v, 3328)
    ref_v = gf.quantize_and_pack_last_dim(v_vis.contiguous(), 32, bits)
    ref_k = gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), 32, bits)
    _check(ops.pack_last_dim(v_vis.contiguous().cuda(), 32, bits), ref_v)
    _check(ops.pack_last_dim(k_vis.transpose(2, 3).contiguous().cuda(), 32, bits), ref_k)
    # strided view of the full cache, transpose fused
    _check(ops.pack_k_per_channel(k.cuda()[:, :, 41:41 + 3328], 32, bits), ref_k)


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_edge_cases(ops, bits):
    g = torch.Generator().manual_seed(3)
    # smallest legal input, ragged tile (T not a multiple of the kernels' tiles), tiny/huge values
    for shape in ((1, 1, 1, 32), (1, 2, 3, 96), (2, 1, 5, 160)):
        x = (torch.randn(*shape, generator=g) * 4).half()
        _check(ops.pack_last_dim(x.cuda(), 32, bits), gf.quantize_and_pack_last_dim(x, 32, bits))
    x = torch.randn(1, 2, 160, 128, generator=g).half()                 # T=160: 1.25 tiles of 128
    _check(ops.pack_k_per_channel(x.cuda(), 32, bits),
           gf.quantize_and_pack_last_dim(x.transpose(2, 3).contiguous(), 32, bits))
    x = torch.randn(1, 1, 4, 64, generator=g).half()
    x[..., :32] *= 1e-4                                                  # subnormal range/scale
    x[0, 0, 1, 32:] *= 2000                                              # large magnitudes
    x[0, 0, 2, :32] = 1.25                                               # constant group
    x[0, 0, 3, 32:] = 0.0                                                # all-zero group
    _check(ops.pack_last_dim(x.cuda(), 32, bits), gf.quantize_and_pack_last_dim(x, 32, bits))


def test_empty_and_bad_inputs(ops):
    e = torch.zeros(0, 2, 4, 64, dtype=torch.float16, device="cuda")
    code, scale, mn = ops.pack_last_dim(e, 32, 1)
    assert code.shape == (0, 2, 4, 2) and scale.shape == (0, 2, 4, 2)
    x = torch.zeros(1, 1, 1, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        ops.pack_last_dim(x, 32, 3)
    with pytest.raises(AssertionError):
        ops.pack_last_dim(torch.zeros(1, 1, 1, 48, dtype=torch.float16, device="cuda"), 32, 1)
    with pytest.raises(TypeError):
        ops.pack_last_dim(x.float(), 32, 1)


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_many_values_bit_exact(ops, bits):
    """Broad sweep (8.4 M elements, several magnitudes) to exercise rounding corner cases."""
    g = torch.Generator().manual_seed(100 + bits)
    x = torch.randn(4, 8, 2048, 128, generator=g)
    x = (x * torch.exp(2 * torch.randn(4, 8, 2048, 1, generator=g))).half()
    _check(ops.pack_last_dim(x.cuda(), 32, bits), gf.quantize_and_pack_last_dim(x, 32, bits))


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_full_size_properties(ops, bits):
    """Config-1 size (B=8, 8 heads, T=32768): too big for the oracle in a test, so check
    size-independent properties on device: the dequantised value is within half a step of the
    input, scale/mn equal the group range/min, and the K-layout kernel agrees with the generic
    one on the transposed tensor."""
    torch.manual_seed(5)
    x = torch.randn(8, 8, 32768, 128, device="cuda", dtype=torch.float16)
    code, scale, mn = ops.pack_last_dim(x, 32, bits)
    xg = x.view(8, 8, 32768, 4, 32)
    assert torch.equal(mn, xg.amin(-1))
    assert torch.equal(scale, (xg.amax(-1) - xg.amin(-1)) / (2 ** bits - 1))
    fpi = 32 // bits
    shifts = (torch.arange(fpi, device="cuda", dtype=torch.int32) * bits)
    c = ((code.unsqueeze(-1) >> shifts) & (2 ** bits - 1)).reshape(8, 8, 32768, 4, 32)
    deq = c.float() * scale.float().unsqueeze(-1) + mn.float().unsqueeze(-1)
    err = (deq - xg.float()).abs()
    assert bool((err <= 0.51 * scale.float().unsqueeze(-1) + 2e-3 * xg.float().abs() + 1e-6).all())
    del c, deq, err
    sub = x[:2]
    a = ops.pack_k_per_channel(sub, 32, bits)
    b = ops.pack_last_dim(sub.transpose(2, 3).contiguous(), 32, bits)
    for u, w in zip(a, b):
        assert bits_equal(u, w)


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_rounding_break_points(ops, bits):
    """Adversarial groups: for every fp16 mantissa of the group range (three binades) the
    elements are the fp16 neighbours of each decision threshold (k + 0.5) * scale, i.e. exactly the
    inputs where an inexact quotient would flip a code."""
    levels = 2 ** bits - 1
    mant = torch.arange(1024, dtype=torch.float32)
    groups = []
    for exp in (-3, 0, 5):
        rng = ((1 + mant / 1024) * 2.0 ** exp).half()                 # group max (min is 0)
        scale = (rng / levels).float()                                 # what the kernel will derive
        for k in range(levels):
            thr = ((k + 0.5) * scale).half()
            bits16 = thr.view(torch.int16).to(torch.int32)
            cand = torch.stack([(bits16 + o).to(torch.int16).view(torch.float16) for o in range(-15, 15)], dim=1)
            cand = torch.minimum(cand, rng[:, None])                   # stay inside [0, max]
            cand = torch.maximum(cand, torch.zeros_like(cand))
            g = torch.cat([torch.zeros(1024, 1, dtype=torch.float16), rng[:, None], cand], dim=1)
            groups.append(g)                                           # [1024, 32]
    x = torch.cat(groups, dim=0).reshape(1, 1, -1, 32).contiguous()
    _check(ops.pack_last_dim(x.cuda(), 32, bits), gf.quantize_and_pack_last_dim(x, 32, bits))
    xb = x.to(torch.bfloat16)
    _check(ops.pack_last_dim(xb.cuda(), 32, bits), gf.quantize_and_pack_last_dim(xb, 32, bits))
