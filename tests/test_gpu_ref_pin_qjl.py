"""The QJL kernels and their CPU oracle against the reference's own CUDA kernels.

``oracle/build_ref.py`` compiles the reference's ``qjl/csrc/qjl_quant_kernel.cu`` and
``qjl_gqa_score_kernel.cu`` (unchanged) into ``oracle/_ref/cuda_qjl_quant.so`` and ``cuda_qjl_gqa_score.so``.
This test runs them on the GPU with the arguments the reference's dispatcher passes
(``qjl/qjl_kernel.py:7-28, 52-72``) and compares, on the same seeded inputs,

* the packed sign bits and outlier norms of ``cq_qjl_quant`` and of ``oracle.qjl.qjl_quant``: bits equal except
  where the projected sum is at rounding distance of zero (fewer than 0.1 %), norms within one rounding step;
* the scores of ``cq_qjl_gqa_score`` and of ``oracle.qjl.qjl_gqa_score`` computed from the reference's own bits:
  rel-L2 <= 1e-4 (fp32 arithmetic, different summation order).

Shapes stay inside what the reference kernels can take: 4 query heads per KV head (``GQA_GROUP_SIZE``,
``qjl_gqa_score_kernel.cu:8``), at most 32 outlier channels (``shared_outlier_ind[32]``, ``:95``), sketch
dimensions that are multiples of 256, groups of 32 keys.  The reference launches its quantizer on a stream of its
own that nothing waits for (``qjl_quant_kernel.cu:219-220``): the test synchronises the device around it.
Skipped when the extensions have not been built (the reference checkout is needed for that).
"""

import importlib.util
import os

import pytest
import torch

from oracle import qjl as oq
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _load(name):
    path = os.path.join(_REF, name + ".so")
    if not os.path.exists(path):
        pytest.skip(f"oracle/_ref/{name}.so not built (python oracle/build_ref.py needs the reference checkout)")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref_quant():
    return _load("cuda_qjl_quant")


@pytest.fixture(scope="module")
def ref_score():
    return _load("cuda_qjl_gqa_score")


def _suffix(t, proj):
    a = {torch.float16: "half", torch.bfloat16: "bf16", torch.float32: "float"}[t.dtype]
    b = {torch.float16: "half", torch.bfloat16: "bf16", torch.float32: "float"}[proj.dtype]
    return f"{a}_{b}"


def _inputs(dtype, n_outliers, seed):
    from calibquant_b200.qjl.qjl_utils import QJLSketch
    sk = QJLSketch((128, 256), 256, device=torch.device("cuda"),
                   rng=torch.Generator(device="cuda").manual_seed(seed), rot=True)
    g = torch.Generator().manual_seed(seed)
    k = (torch.randn(2, 2, 160, 128, generator=g) * torch.exp(0.5 * torch.randn(128, generator=g))).to(dtype)
    q = torch.randn(2, 8, 1, 128, generator=g).to(dtype)
    groups, idx, knorm = oq.build_groups(k, 32, n_outliers)          # [B,H,n,32,128], uint8 [B,H,n,count], [B,H,n,32]
    return sk, groups, idx, knorm, q


def _ref_quant(ext, groups, idx, proj, outlier_dim):
    torch.cuda.synchronize()
    fn = getattr(ext, "qjl_quant_" + _suffix(groups, proj))
    out = fn(groups.contiguous(), idx.contiguous(), proj.contiguous(), outlier_dim)
    torch.cuda.synchronize()                       # the reference's private stream
    return out


@pytest.mark.parametrize("dtype,proj_dtype", [(torch.float16, torch.float32), (torch.float16, torch.float16),
                                              (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("n_outliers", [8, 32])
def test_quantizer_bits_and_norms(ref_quant, dtype, proj_dtype, n_outliers):
    from calibquant_b200.qjl import qjl_kernel
    sk, groups, idx, _, _ = _inputs(dtype, n_outliers, seed=11)
    proj = sk.proj_dir_quant.to(proj_dtype)
    r_kq, r_koq, r_norm = _ref_quant(ref_quant, groups.cuda(), idx.cuda(), proj, 256)
    kq, koq, norm = qjl_kernel.qjl_quant(groups.cuda(), idx.cuda(), proj, 256)
    o_kq, o_koq, o_norm = oq.qjl_quant(groups, idx, proj.cpu(), 256)
    assert r_kq.shape == kq.shape == o_kq.shape and r_koq.shape == koq.shape == o_koq.shape
    sk_in, sk_out = oq.sketches(groups, idx, proj.cpu())
    for name, got in (("library", (kq.cpu(), koq.cpu())), ("oracle", (o_kq, o_koq))):
        for bits, ref_bits, val in ((got[0], r_kq.cpu(), sk_in), (got[1], r_koq.cpu(), sk_out)):
            diff = oq.unpack_bits(bits) != oq.unpack_bits(ref_bits)
            assert diff.float().mean() < 1e-3, (name, float(diff.float().mean()))
            assert (val[diff].abs() < 1e-3 * val.abs().mean()).all(), name   # only sums at rounding distance of zero
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    for name, n in (("library", norm.cpu()), ("oracle", o_norm)):
        assert (n.float() - r_norm.cpu().float()).abs().le(r_norm.cpu().float() * 2 * ulp + 1e-6).all(), name


@pytest.mark.parametrize("dtype,proj_dtype", [(torch.float16, torch.float32), (torch.bfloat16, torch.float32),
                                              (torch.float16, torch.float16)])
@pytest.mark.parametrize("n_outliers", [8, 32])
def test_scores_from_the_references_bits(ref_quant, ref_score, dtype, proj_dtype, n_outliers):
    from calibquant_b200.qjl import qjl_kernel
    sk, groups, idx, knorm, q = _inputs(dtype, n_outliers, seed=12)
    r_kq, r_koq, r_norm = _ref_quant(ref_quant, groups.cuda(), idx.cuda(), sk.proj_dir_quant.to(proj_dtype), 256)
    proj_s = sk.proj_dir_score.to(proj_dtype).contiguous()
    qs = torch.matmul(q.cuda().float(), sk.proj_dir_score).contiguous()          # fp32 query sketch [B,Hq,1,256]
    args = (r_kq, r_koq, knorm.cuda().contiguous(), r_norm, idx.cuda().contiguous(), qs, q.cuda().contiguous(), proj_s)
    torch.cuda.synchronize()
    ref = getattr(ref_score, "qjl_gqa_score_cuda_" + _suffix(q, proj_s))(*args)
    torch.cuda.synchronize()
    got = qjl_kernel.qjl_gqa_score(*args)
    orc = oq.qjl_gqa_score(*(a.cpu() for a in args))
    assert ref.shape == got.shape == orc.shape == (2, 8, 160, 1)
    assert rel_l2(got, ref.cpu()) <= 1e-4, rel_l2(got, ref.cpu())
    assert rel_l2(orc, ref.cpu()) <= 1e-4, rel_l2(orc, ref.cpu())
