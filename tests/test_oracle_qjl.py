"""CPU checks of the QJL oracle: known-answer packing, and that the estimator it restates does what
the method claims (an unbiased, strongly correlated estimate of q.k)."""

import math

import torch

from oracle import qjl


def test_pack_bits_is_lsb_first():
    bits = torch.zeros(16, dtype=torch.bool)
    bits[0] = bits[3] = bits[9] = True
    assert qjl.pack_bits(bits).tolist() == [0b00001001, 0b00000010]
    assert torch.equal(qjl.unpack_bits(qjl.pack_bits(bits)), bits)


def test_quant_known_answer():
    """Identity-like projection: the sign bits are the signs of the key channels, split by the mask."""
    keys = torch.tensor([1.0, -2.0, 3.0, -4.0] + [0.0] * 124).half().view(1, 1, 1, 1, 128)
    proj = torch.eye(128)[:32]                               # projection p reads channel p
    idx = torch.tensor([2, 3], dtype=torch.uint8).view(1, 1, 1, 2)
    kq, koq, norms = qjl.qjl_quant(keys, idx, proj, 32)
    assert kq.shape == (1, 1, 1, 1, 4) and kq[0, 0, 0, 0].tolist() == [0b0001, 0, 0, 0]      # channel 0 positive, inlier
    assert koq[0, 0, 0, 0].tolist() == [0b0100, 0, 0, 0]                                     # channel 2 positive, outlier
    assert float(norms) == 5.0                                                               # sqrt(3^2 + 4^2)


def test_estimator_tracks_the_inner_product():
    g = torch.Generator().manual_seed(0)
    B, Hkv, rep, T, D, s = 1, 2, 4, 256, 128, 256
    k = (torch.randn(B, Hkv, T, D, generator=g) * torch.exp(0.5 * torch.randn(D, generator=g))).half()
    q = torch.randn(B, Hkv * rep, 1, D, generator=g).half()
    S = torch.randn(D, s, generator=g)
    groups, idx, knorm = qjl.build_groups(k, 32, 32)
    kq, koq, onorm = qjl.qjl_quant(groups, idx, S.t().contiguous(), s)
    est = qjl.qjl_gqa_score(kq, koq, knorm, onorm, idx, q.float() @ S, q, S).reshape(B, Hkv, rep, T)
    exact = torch.einsum("bhrd,bhtd->bhrt", q.float().reshape(B, Hkv, rep, D), k.float())
    corr = torch.corrcoef(torch.stack([est.flatten(), exact.flatten()]))[0, 1]
    assert corr > 0.8        # s = 256 sign bits per key: ~0.85 on this data
    # unbiased up to noise: the regression slope of the estimate on the truth is close to one
    slope = (est * exact).sum() / (exact * exact).sum()
    assert abs(float(slope) - 1) < 0.1
    assert math.isfinite(float(est.abs().max()))
