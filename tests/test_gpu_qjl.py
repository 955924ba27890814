"""QJL sign-sketch kernels against the CPU oracle, through the reference-shaped API.

Bars: the packed sign bits are byte data derived from fp32 sums, so they must equal the oracle's
wherever the sum is not within rounding distance of zero (checked: every mismatching bit has
|projection| < 1e-3 of the row's typical magnitude, and fewer than 0.1 % mismatch); outlier norms
within one rounding step of the data dtype; scores computed from the *same* bits within 1e-4
(fp32 arithmetic, different summation order)."""

import os

import pytest
import torch

from oracle import qjl as oq
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu


def _data(B, Hkv, rep, T, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    k = (torch.randn(B, Hkv, T, 128, generator=g) * torch.exp(0.5 * torch.randn(128, generator=g))).to(dtype)
    q = torch.randn(B, Hkv * rep, 1, 128, generator=g).to(dtype)
    return k, q


def _sketch(seed=7):
    from calibquant_b200.qjl.qjl_utils import QJLSketch
    return QJLSketch((128, 256), 256, device=torch.device("cuda"),
                     rng=torch.Generator(device="cuda").manual_seed(seed), rot=True)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("proj_same_dtype", [False, True])
def test_quant_matches_oracle(dtype, proj_same_dtype):
    from calibquant_b200.qjl import qjl_kernel
    sk = _sketch()
    k, _ = _data(2, 2, 4, 160, dtype, seed=1)
    groups, idx, _ = oq.build_groups(k, 32, 32)
    proj = sk.proj_dir_quant.to(dtype) if proj_same_dtype else sk.proj_dir_quant
    kq, koq, norms = qjl_kernel.qjl_quant(groups.cuda(), idx.cuda(), proj, 256)
    r_kq, r_koq, r_norms = oq.qjl_quant(groups, idx, proj.cpu(), 256)
    assert kq.shape == r_kq.shape == (2, 2, 5, 32, 32) and koq.shape == r_koq.shape and kq.dtype == torch.uint8
    sk_in, sk_out = oq.sketches(groups, idx, proj.cpu())
    for got, ref, val in ((kq, r_kq, sk_in), (koq, r_koq, sk_out)):
        diff = oq.unpack_bits(got.cpu()) != oq.unpack_bits(ref)
        assert diff.float().mean() < 1e-3
        assert (val[diff].abs() < 1e-3 * val.abs().mean()).all()       # only sums at rounding distance of zero
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert (norms.cpu().float() - r_norms.float()).abs().le(r_norms.float() * ulp + 1e-6).all()


@pytest.mark.parametrize("dtype,rep", [(torch.float16, 4), (torch.bfloat16, 4), (torch.float16, 6), (torch.float16, 1)])
def test_score_matches_oracle_on_the_same_bits(dtype, rep):
    from calibquant_b200.qjl import qjl_kernel
    sk = _sketch(3)
    k, q = _data(2, 2, rep, 96, dtype, seed=2)
    groups, idx, knorm = oq.build_groups(k, 32, 32)
    kq, koq, onorm = qjl_kernel.qjl_quant(groups.cuda(), idx.cuda(), sk.proj_dir_quant, 256)
    qs = torch.matmul(q.cuda().float(), sk.proj_dir_score)
    got = qjl_kernel.qjl_gqa_score(kq, koq, knorm.cuda(), onorm, idx.cuda(), qs, q.cuda(), sk.proj_dir_score)
    ref = oq.qjl_gqa_score(kq.cpu(), koq.cpu(), knorm, onorm.cpu(), idx, qs.cpu(), q, sk.proj_dir_score.cpu())
    assert got.shape == ref.shape == (2, 2 * rep, 96, 1) and got.dtype == torch.float32
    assert rel_l2(got, ref) <= 1e-4


@pytest.mark.parametrize("sketch_dim,outlier_dim,T,rep", [(256, 128, 352, 4), (256, 128, 352, 8), (128, 128, 288, 4),
                                                         (96, 64, 96, 4), (224, 32, 64, 6)])
def test_score_sketch_sizes_and_group_counts(sketch_dim, outlier_dim, T, rep):
    """Outlier sketches shorter than the inlier one, group counts that are not a multiple of what one CTA
    walks (tensor-core kernel: sketch dims multiples of 128), and sketch dims only the CUDA-core kernel takes."""
    from calibquant_b200.qjl import qjl_kernel
    from calibquant_b200.qjl.qjl_utils import QJLSketch
    sk = QJLSketch((128, sketch_dim), outlier_dim, device=torch.device("cuda"),
                   rng=torch.Generator(device="cuda").manual_seed(5), rot=True)
    k, q = _data(1, 2, rep, T, torch.float16, seed=9)
    groups, idx, knorm = oq.build_groups(k, 32, 8)
    kq, koq, onorm = qjl_kernel.qjl_quant(groups.cuda(), idx.cuda(), sk.proj_dir_quant, outlier_dim)
    assert kq.shape[-1] == sketch_dim // 8 and koq.shape[-1] == outlier_dim // 8
    qs = torch.matmul(q.cuda().float(), sk.proj_dir_score)
    got = qjl_kernel.qjl_gqa_score(kq, koq, knorm.cuda(), onorm, idx.cuda(), qs, q.cuda(), sk.proj_dir_score)
    ref = oq.qjl_gqa_score(kq.cpu(), koq.cpu(), knorm, onorm.cpu(), idx, qs.cpu(), q, sk.proj_dir_score.cpu())
    assert got.shape == ref.shape == (1, 2 * rep, T, 1)
    assert rel_l2(got, ref) <= 1e-4


def test_key_quantizer_streaming_and_estimate_quality():
    """build_sketch / update_sketch / attention_score of the sketch-backed quantizer: shapes, the fp
    residual that flushes every buffer_size keys, and an estimate that tracks q.k."""
    from calibquant_b200.qjl.qjl_utils import QJLKeyQuantizer
    sk = _sketch(11)
    k, q = _data(1, 2, 4, 300, torch.float16, seed=4)
    kq = QJLKeyQuantizer(sk, 32, 128, 32, 2)
    kq.build_sketch(k.cuda())
    assert kq.seq_len == 300 and kq.key_residual.shape[2] == 300 % 128
    assert kq.key_states_quant.shape == (1, 2, 8, 32, 32) and kq.outlier_indices.shape == (1, 2, 8, 32)
    s = kq.attention_score(q.cuda())
    assert s.shape == (1, 8, 1, 300) and s.dtype == torch.float32
    exact = torch.einsum("bhrd,bhtd->bhrt", q.float().reshape(1, 2, 4, 128), k.float()).reshape(1, 8, 1, 300)
    assert torch.allclose(s[..., 256:].cpu(), exact[..., 256:], rtol=2e-3, atol=2e-2)        # residual keys are exact
    corr = torch.corrcoef(torch.stack([s[..., :256].cpu().flatten(), exact[..., :256].flatten()]))[0, 1]
    assert corr > 0.8
    g = torch.Generator().manual_seed(9)
    for _ in range(128 - 44):
        kq.update_sketch(torch.randn(1, 2, 1, 128, generator=g).half().cuda())
    assert kq.key_residual is None and kq.seq_len == 384 and kq.key_states_quant.shape[2] == 12
    assert kq.attention_score(q.cuda()).shape == (1, 8, 1, 384)


def test_dtype_errors_and_empty():
    from calibquant_b200.qjl import qjl_kernel
    sk = _sketch()
    k = torch.randn(1, 1, 1, 32, 128, device="cuda")
    idx = torch.zeros(1, 1, 1, 32, dtype=torch.uint8, device="cuda")
    with pytest.raises(TypeError):
        qjl_kernel.qjl_quant(k, idx, sk.proj_dir_quant, 256)                       # fp32 keys
    with pytest.raises(TypeError):
        qjl_kernel.qjl_quant(k.half(), idx, sk.proj_dir_quant.bfloat16(), 256)     # mixed 16-bit types
    kq, koq, n = qjl_kernel.qjl_quant(k.half()[:, :, :0], idx[:, :, :0], sk.proj_dir_quant, 256)
    assert kq.shape == (1, 1, 0, 32, 32) and n.numel() == 0


def test_qjl_forward_with_sketch_runs_close_to_full_precision():
    """patch_model(..., "qjl") with the sign sketch: the decode step must stay close to the layer run
    with exact keys (the estimator is noisy by design, so the bar is loose)."""
    from calibquant_b200 import patch_internvl as pi
    from calibquant_b200.internlm2 import ChatModelShell, InternLM2Config, init_weights_
    cfg = InternLM2Config(hidden_size=1024, num_attention_heads=8, num_key_value_heads=2,
                          intermediate_size=256, num_hidden_layers=1, vocab_size=64)
    shell = ChatModelShell(cfg).half()
    init_weights_(shell, 5, std=0.05)
    shell.cuda()
    pi.patch_model(shell, "qjl", k_bits=2, v_bits=4, buffer_size=128)
    try:
        attn = shell.language_model.model.layers[0].attention
        t_vis, t_txt, B = 256, 9, 1
        T = 41 + t_vis + t_txt
        g = torch.Generator().manual_seed(3)
        h = (torch.randn(B, T + 1, 1024, generator=g) * 0.5).half().cuda()
        os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
        pos = torch.arange(T + 1, device="cuda").unsqueeze(0)
        full, _, _ = attn(h, position_ids=pos, use_cache=False)                   # exact attention over T+1 tokens
        _, _, past = attn(h[:, :T], position_ids=pos[:, :T], use_cache=True)
        assert type(past[1]).__name__ == "QJLKeyQuantizer" and past[1].key_states_quant is not None
        out, _, past = attn(h[:, T:], position_ids=pos[:, T:], past_key_value=past, use_cache=True)
        assert out.shape == (B, 1, 1024) and torch.isfinite(out.float()).all()
        assert rel_l2(out, full[:, T:]) <= 0.35
    finally:
        pi.patch_model(shell, "calibquant")
