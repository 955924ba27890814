"""cq_qbmm_static: the quantized product for callers that cannot allocate device memory.

A serving process that has given all remaining HBM to its KV-cache pool (so cudaMalloc would
fail) or that must not stall its other streams (cudaMalloc synchronises the device) calls this
entry point instead of cq_qbmm: the fp32 scratch is a fixed 8 MiB array inside the library.
The test drives it through the C ABI only (ctypes, raw device pointers), twice in a row with
different inputs -- the array is shared and keeps the previous call's contents, so the second
call would expose any dependence on stale scratch -- and requires bit-identical outputs to
cq_qbmm, which runs the same kernels on a caller-provided workspace, and agreement with the CPU
oracle.  The shapes cover the three routes of the product: the general kernels, the score kernel
(128 reduction rows) and the attn.V kernels (128 output columns, the route that really parks its
partial sums in the array).  It also checks that a problem beyond the fixed capacity is refused
and that the array's status word reads clean.  This file sorts last on purpose.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _case(seed, B, Hq, Hkv, K, N, bits):
    from oracle import group_format as gf
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(B, Hkv, K, N, generator=g).half()
    code, scale, mn = gf.quantize_and_pack_last_dim(w, 32, bits)
    a = torch.softmax(torch.randn(B, Hq, 1, K, generator=g) * 2, -1).half()
    rep = lambda t: gf.repeat_kv(t, Hq // Hkv)
    want = gf.qbmm(32, a, rep(code), rep(scale), rep(mn), bits).reshape(B, Hq, N)
    return a.cuda(), code.cuda(), scale.cuda(), mn.cuda(), want


def test_static_scratch_matches_workspace_variant_twice():
    from calibquant_b200 import _lib
    lib = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.cq_qbmm_static_capacity_bytes() == 8 << 20
    # general kernels (K not a multiple of 256), score kernel (K = 128), attn.V kernels (N = 128, K % 256 = 0)
    shapes = [(11, 2, 8, 2, 700, 128, 1), (12, 1, 12, 2, 128, 2048, 2), (13, 2, 8, 2, 512, 128, 1),
              (14, 1, 8, 2, 1536, 128, 2)]
    cases = []
    for seed, B, Hq, Hkv, K, N, bits in shapes:                           # references first
        a, code, scale, mn, want = _case(seed, B, Hq, Hkv, K, N, bits)
        need = lib.cq_qbmm_workspace_bytes(B, Hq, K, N)
        assert 0 < need <= 8 << 20
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        ref = torch.empty(B, Hq, N, dtype=torch.float16, device="cuda")
        rc = lib.cq_qbmm(_p(a), _p(code), _p(scale), _p(mn), _p(ref), B, Hq, Hkv, K, N, 32, bits,
                         _lib.CQ_DTYPE_F16, _p(ws), need, stream)
        assert rc == _lib.CQ_OK
        assert lib.cq_workspace_status(_p(ws), stream) == _lib.CQ_OK
        err = float((ref.cpu().double() - want.double()).norm() / want.double().norm())
        assert err <= 2e-3, err                                           # the tolerance of the product's own tests
        cases.append((a, code, scale, mn, ref, torch.full_like(ref, float("nan")),
                      (B, Hq, Hkv, K, N, bits)))
    for a, code, scale, mn, ref, out, (B, Hq, Hkv, K, N, bits) in cases:  # two static calls in a row
        rc = lib.cq_qbmm_static(_p(a), _p(code), _p(scale), _p(mn), _p(out), B, Hq, Hkv, K, N, 32,
                                bits, _lib.CQ_DTYPE_F16, stream)
        assert rc == _lib.CQ_OK, lib.cq_status_string(rc)
    torch.cuda.synchronize()
    assert lib.cq_qbmm_static_status(stream) == _lib.CQ_OK
    for a, code, scale, mn, ref, out, dims in cases:
        assert torch.isfinite(out.float()).all()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))   # tolerance: bit-identical


def test_static_scratch_rejects_oversized_problem():
    from calibquant_b200 import _lib
    lib = _lib.lib()
    # 32 chunks * 64 rows * 4096 columns * 4 B = 32 MiB > 8 MiB: refused before touching memory
    B, Hq, Hkv, K, N = 2, 32, 8, 8192, 4096
    assert lib.cq_qbmm_workspace_bytes(B, Hq, K, N) > lib.cq_qbmm_static_capacity_bytes()
    dummy = torch.zeros(16, dtype=torch.float16, device="cuda")
    rc = lib.cq_qbmm_static(_p(dummy), _p(dummy), _p(dummy), _p(dummy), _p(dummy), B, Hq, Hkv, K, N,
                            32, 1, _lib.CQ_DTYPE_F16, None)
    assert rc == _lib.CQ_ERR_TOO_LARGE
    assert b"scratch" in lib.cq_status_string(rc)
