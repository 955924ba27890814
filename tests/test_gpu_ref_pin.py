"""The CPU oracle and cq_qbmm against the reference's own CUDA kernel for the quantized product.

``oracle/build_ref.py`` compiles the reference's ``qjl/csrc/quantization.cu`` (unchanged) into
``oracle/_ref/quantization.so``; this test runs it on the GPU through the layout transforms of the
reference's Python wrapper (``qjl/matmul.py:12-22``: activations flattened to [B*nh, 1, K], the packed
operand and its scales / zeros transposed to [B*nh, N/.., K]) and compares, on the same seeded operands,
with ``oracle.group_format.qbmm`` (what every other parity test is measured against) and with the
library's ``cq_qbmm``.  Only 2 and 4 bits and one query row: the reference kernel keeps ``psum[16]``
(``quantization.cu:89``), too few for the 32 codes of a 1-bit word, and ignores rows beyond the first.
Skipped when the extension has not been built (the reference checkout is needed for that).
"""

import importlib.util
import os

import pytest
import torch

from oracle import generator
from oracle import group_format as gf
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu

_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "quantization.so")


@pytest.fixture(scope="module")
def ref_ext():
    if not os.path.exists(_SO):
        pytest.skip("oracle/_ref/quantization.so not built (python oracle/build_ref.py needs the reference checkout)")
    spec = importlib.util.spec_from_file_location("quantization", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _reference_bmm(ext, group_size, fA, qB, scales, zeros, bits):
    """The call sequence of qjl/matmul.py:4-35 (operands already expanded to the query heads)."""
    B, nh, M, K = fA.shape
    a = fA.view(-1, M, K).contiguous()
    w = qB.reshape(-1, K, qB.shape[-1]).transpose(1, 2).contiguous()
    s = scales.view(B * nh, scales.shape[-2], scales.shape[-1]).transpose(1, 2).contiguous()
    z = zeros.view(B * nh, zeros.shape[-2], zeros.shape[-1]).transpose(1, 2).contiguous()
    fn = {torch.float16: ext.batchedQuantizedMultiplyAccumulate_half,
          torch.bfloat16: ext.batchedQuantizedMultiplyAccumulate_bf16}[fA.dtype]
    torch.cuda.synchronize()               # the kernel is launched on the legacy default stream
    out = fn(a, w, s, z, bits, group_size, nh, False)
    torch.cuda.synchronize()
    return out.view(B, nh, out.shape[-2], out.shape[-1])


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantized_product_against_the_reference_kernel(ref_ext, bits, dtype):
    from calibquant_b200 import ops
    B, Hq, Hkv, T = 2, 8, 2, 1280
    k, v, q = generator.make_kvq(B, Hq, Hkv, T, seed=60 + bits, dtype=dtype)
    kp = gf.quantize_and_pack_last_dim(k.transpose(2, 3).contiguous(), 32, bits)   # K per channel: [B,Hkv,128,T/..]
    vp = gf.quantize_and_pack_last_dim(v.contiguous(), 32, bits)                   # V per token:   [B,Hkv,T,128/..]
    rep = lambda t: gf.repeat_kv(t, Hq // Hkv)
    g = torch.Generator().manual_seed(7)
    att = torch.softmax(torch.randn(B, Hq, 1, T, generator=g) * 2, -1).to(dtype)
    for name, fA, pack in (("q.K", q, kp), ("att.V", att, vp)):
        exp = [rep(t).cuda().contiguous() for t in pack]
        ref = _reference_bmm(ref_ext, 32, fA.cuda(), exp[0], exp[1], exp[2], bits).cpu()
        oracle = gf.qbmm(32, fA, rep(pack[0]), rep(pack[1]), rep(pack[2]), bits)
        ours = ops.qbmm(32, fA.cuda(), *[t.cuda() for t in pack], bits).cpu()
        # the oracle restates the kernel's arithmetic (fp32 dequantise, fp32 accumulate, one rounding): only
        # the summation order and the kernel's fast-math FMA contraction differ, a fraction of an ulp
        tol_oracle = 3e-4 if dtype == torch.float16 else 2e-3
        assert rel_l2(oracle, ref) <= tol_oracle, (name, rel_l2(oracle, ref))
        # cq_qbmm: the tolerance of the product's own tests
        tol_ours = 2e-3 if dtype == torch.float16 else 4e-3
        assert rel_l2(ours, ref) <= tol_ours, (name, rel_l2(ours, ref))
        mism = float((oracle.view(torch.int16) != ref.view(torch.int16)).float().mean())
        assert mism <= 0.05, (name, mism)          # almost all values bit-equal, the rest one ulp apart


@pytest.mark.parametrize("bits", [2, 4])
def test_decode_composition_with_the_reference_kernel(ref_ext, bits):
    """The decode step of patch_internvl.py:556-592 composed around the reference's kernel for both
    products (scores and attn.V), against oracle.group_format.decode_attention and the fused step."""
    import math
    from calibquant_b200 import ops
    B, Hq, Hkv, t_vis, t_txt, sys_len = 1, 8, 2, 1024, 23, generator.SYS_LEN
    k, v, q = generator.make_kvq(B, Hq, Hkv, sys_len + t_vis + t_txt, seed=80 + bits)
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
    kp = gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), 32, bits)
    vp = gf.quantize_and_pack_last_dim(v_vis.contiguous(), 32, bits)
    rep = lambda t: gf.repeat_kv(t, Hq // Hkv)
    dev = lambda ts: [rep(t).cuda().contiguous() for t in ts]
    sd = math.sqrt(128)
    qd = q.cuda()
    s_vis = _reference_bmm(ref_ext, 32, qd, *dev(kp), bits) / sd
    s_sys = torch.matmul(qd, rep(k_sys).cuda().transpose(2, 3)) / sd
    s_txt = torch.matmul(qd, rep(k_txt).cuda().transpose(2, 3)) / sd
    if bits <= 2:
        s_vis = gf.calibrate(s_vis)
    att = torch.softmax(torch.cat([s_sys, s_vis, s_txt], -1), -1, dtype=torch.float32).to(q.dtype)
    ns = sys_len
    o = _reference_bmm(ref_ext, 32, att[..., ns:ns + t_vis].contiguous(), *dev(vp), bits)
    o = o + (torch.matmul(att[..., ns + t_vis:], rep(v_txt).cuda()) + torch.matmul(att[..., :ns], rep(v_sys).cuda()))
    o = o.cpu()
    oracle = gf.decode_attention(q, kp, vp, k_sys, k_txt, v_sys, v_txt, bits)
    assert rel_l2(oracle, o) <= 5e-3, rel_l2(oracle, o)
    k_fp, v_fp = torch.cat([k_sys, k_txt], 2).cuda(), torch.cat([v_sys, v_txt], 2).cuda()
    ours = ops.decode_attention(qd, [t.cuda() for t in kp], [t.cuda() for t in vp], k_fp, v_fp, sys_len, bits).cpu()
    assert rel_l2(ours, o) <= 1e-2, rel_l2(ours, o)
