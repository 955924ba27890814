"""Prefill attention vs the fp32 oracle (softmax(QK^T/sqrt(D) + causal) V with GQA).

Tolerance: rel-L2 <= 5e-3 (fp16) / 1e-2 (bf16): the probabilities are rounded to the 16-bit type
before the PV product, as in any flash-attention kernel."""

import pytest
import torch

from oracle import prefill as oracle_prefill
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from calibquant_b200 import ops as _ops
    return _ops


def _qkv(B, T, Hq, Hkv, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, Hq, 128, generator=g).to(dtype)
    k = torch.randn(B, T, Hkv, 128, generator=g).to(dtype)
    v = torch.randn(B, T, Hkv, 128, generator=g).to(dtype)
    return q, k, v


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 5e-3), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("T", [1, 63, 64, 65, 200, 1024 + 41])
def test_matches_oracle(ops, dtype, tol, T):
    q, k, v = _qkv(2, T, 8, 2, dtype, seed=T)
    ref = oracle_prefill.causal_attention(q, k, v)
    out = ops.prefill_attention(q.cuda(), k.cuda(), v.cuda())
    assert out.shape == ref.shape and out.dtype == dtype
    assert rel_l2(out, ref) <= tol, rel_l2(out, ref)


def test_n_rep_6_and_strided_views(ops):
    """48q/8kv grouping, and q/k/v given as slices of one fused projection output (the layout the
    patched forward produces), i.e. non-trivial head/token strides."""
    B, T, Hkv, n_rep = 1, 300, 2, 6
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, T, Hkv, n_rep + 2, 128, generator=g).half()
    q = qkv[:, :, :, :n_rep].reshape(B, T, Hkv * n_rep, 128)
    k, v = qkv[:, :, :, -2], qkv[:, :, :, -1]
    ref = oracle_prefill.causal_attention(q, k, v)
    d = qkv.cuda()
    out = ops.prefill_attention(d[:, :, :, :n_rep].reshape(B, T, Hkv * n_rep, 128), d[:, :, :, -2], d[:, :, :, -1])
    assert rel_l2(out, ref) <= 5e-3


def test_first_token_is_v0_and_causality(ops):
    q, k, v = _qkv(1, 130, 4, 1, torch.float16, seed=9)
    out = ops.prefill_attention(q.cuda(), k.cuda(), v.cuda()).cpu()
    assert torch.allclose(out[0, 0].float(), v[0, 0].float().expand(4, 128), atol=2e-3)
    k2, v2 = k.clone(), v.clone()
    k2[:, 100:] = 7.0          # changing later keys/values must not change earlier outputs
    v2[:, 100:] = -3.0
    out2 = ops.prefill_attention(q.cuda(), k2.cuda(), v2.cuda()).cpu()
    assert torch.equal(out[:, :100], out2[:, :100])


def test_large_property(ops):
    """Config-2 sized sequence (3392 tokens, 32q/8kv): oracle on a slice of heads only."""
    q, k, v = _qkv(1, 3392, 32, 8, torch.bfloat16, seed=21)
    out = ops.prefill_attention(q.cuda(), k.cuda(), v.cuda()).cpu()
    ref = oracle_prefill.causal_attention(q[:, :, :4], k[:, :, :1], v[:, :, :1])
    assert rel_l2(out[:, :, :4], ref) <= 1e-2
    assert torch.isfinite(out.float()).all()


def test_status_word_clean_and_general_kernel_agrees(ops):
    """No bounded wait of the tensor-core kernel may have timed out during this module, and the
    warp-MMA kernel must agree with the oracle too.  It serves what a TMA tensor map cannot describe: here
    K and V broadcast over the batch (batch stride 0, as ``expand`` makes them)."""
    from calibquant_b200 import _lib
    assert _lib.lib().cq_prefill_status() == 0
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, 333, 8, 128, generator=g).half()
    k = torch.randn(1, 333, 2, 128, generator=g).half()
    v = torch.randn(1, 333, 2, 128, generator=g).half()
    kd, vd = k.cuda().expand(2, -1, -1, -1), v.cuda().expand(2, -1, -1, -1)
    assert kd.stride(0) == 0
    o = ops.prefill_attention(q.cuda(), kd, vd)
    ref = oracle_prefill.causal_attention(q, k.expand(2, -1, -1, -1), v.expand(2, -1, -1, -1))
    assert rel_l2(o, ref) <= 5e-3
    assert _lib.lib().cq_prefill_status() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 5e-3), (torch.bfloat16, 1e-2)])
def test_growing_logits_force_row_rescales(ops, dtype, tol):
    """Keys whose norm grows along the sequence make the row maximum jump by far more than 2^8
    between key tiles, so the lazily rescaled accumulator path runs on most rows and tiles; a few
    rows also see a *falling* maximum (stale reference kept)."""
    B, T, Hq, Hkv = 1, 700, 4, 2
    g = torch.Generator().manual_seed(21)
    q = (torch.randn(B, T, Hq, 128, generator=g) * 3).to(dtype)
    ramp = torch.linspace(0.2, 4.0, T).view(1, T, 1, 1)
    ramp[:, 300:420] *= 0.1
    k = (torch.randn(B, T, Hkv, 128, generator=g) * ramp).to(dtype)
    v = torch.randn(B, T, Hkv, 128, generator=g).to(dtype)
    ref = oracle_prefill.causal_attention(q, k, v)
    out = ops.prefill_attention(q.cuda(), k.cuda(), v.cuda())
    assert torch.isfinite(out.float()).all()
    assert rel_l2(out, ref) <= tol, rel_l2(out, ref)


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 5e-3), (torch.bfloat16, 1e-2)])
def test_against_the_flash_attn_library(ops, dtype, tol):
    """The reference's prefill is a call into the third-party flash_attn package (patch_internvl.py:464-468,
    :606-609).  Where that package is installed and has kernels for this GPU, its causal attention on the same
    seeded tensors pins both the library's prefill kernel and the fp32 oracle; otherwise the test is skipped."""
    try:
        from flash_attn import flash_attn_func
    except Exception as e:                      # not installed / not importable here
        pytest.skip(f"flash_attn not importable: {type(e).__name__}")
    q, k, v = _qkv(2, 700, 8, 2, dtype, seed=33)
    try:
        ref = flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=True)
        torch.cuda.synchronize()
    except Exception as e:                      # e.g. no kernel image for this architecture
        pytest.skip(f"flash_attn cannot run on this GPU: {type(e).__name__}: {str(e)[:80]}")
    out = ops.prefill_attention(q.cuda(), k.cuda(), v.cuda())
    assert rel_l2(out, ref.cpu()) <= tol
    assert rel_l2(oracle_prefill.causal_attention(q, k, v), ref.cpu()) <= tol
