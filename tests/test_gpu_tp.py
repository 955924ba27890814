"""The peer-memory collectives of the tensor-parallel decode step, on one GPU.

``PeerComm.local_group`` makes the buffers of G ranks inside this process; the ranks of a collective then
run one after the other on one stream (all pushes, then all reduces), so no wait ever has to spin: what is
exercised is the slot addressing, the double buffering on the sequence number's parity, the device-side
advance of the sequence number over several collectives in a row, and the arithmetic of the fused
sum + residual + RMSNorm against plain torch.  (Ranks that really run at the same time are covered by the
two-GPU test.)"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_add_norm(res, parts, weight, eps):
    r = (res.float() + sum(p.float() for p in parts)).to(res.dtype)
    v = r.float()
    n = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(res.dtype)
    return r, weight * n


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_push_reduce_add_rmsnorm(world, dtype):
    from calibquant_b200 import tp
    dev = torch.device("cuda")
    B, hidden = 16, 4096
    comms = tp.PeerComm.local_group(world, B * hidden * 2, dev)
    try:
        g = torch.Generator(device=dev).manual_seed(1)
        weight = (1 + 0.1 * torch.randn(hidden, generator=g, device=dev)).to(dtype)
        res = [torch.randn(B, 1, hidden, generator=g, device=dev).to(dtype) for _ in range(world)]
        want_res = res[0].clone()
        for r in range(1, world):
            res[r].copy_(res[0])
        for it in range(5):                       # five collectives in a row: both parities, advancing numbers
            parts = [(torch.randn(B, 1, hidden, generator=g, device=dev) * 0.3).to(dtype) for _ in range(world)]
            for r in range(world):
                comms[r].push(parts[r])
            want_res, want_out = _ref_add_norm(want_res, parts, weight, 1e-5)
            for r in range(world):
                out = comms[r].reduce_add_rmsnorm(res[r], weight, 1e-5)
                assert torch.equal(res[r], want_res), (it, r)
                assert float((out.float() - want_out.float()).abs().max()) <= 2e-2 * float(want_out.float().abs().max())
        # the bare sum (no norm), then a gather
        parts = [(torch.randn(B, 1, hidden, generator=g, device=dev)).to(dtype) for _ in range(world)]
        for r in range(world):
            comms[r].push(parts[r])
        want_res, _ = _ref_add_norm(want_res, parts, weight, 1e-5)
        for r in range(world):
            assert comms[r].reduce_add_rmsnorm(res[r], None, 1e-5, normalize=False) is None
            assert torch.equal(res[r], want_res)
        small = [torch.randn(B, 2, generator=g, device=dev) for _ in range(world)]
        for r in range(world):
            comms[r].push(small[r])
        for r in range(world):
            got = comms[r].gather(small[r])
            assert torch.equal(got, torch.stack(small))
        assert all(c.status() == 0 for c in comms)
    finally:
        for c in comms:
            c.close()


def test_fused_allreduce_with_one_rank():
    """The one-launch collective with a single rank (no peer to wait for): residual += partial, then the norm.
    With more ranks its CTAs wait for their peers' CTAs, which only separate GPUs can run at the same time:
    that is the two-GPU test's part."""
    from calibquant_b200 import tp
    dev = torch.device("cuda")
    B, hidden = 16, 4096
    comm = tp.PeerComm.local_group(1, B * hidden * 2, dev)[0]
    try:
        g = torch.Generator(device=dev).manual_seed(3)
        weight = (1 + 0.1 * torch.randn(hidden, generator=g, device=dev)).to(torch.bfloat16)
        res = torch.randn(B, 1, hidden, generator=g, device=dev).to(torch.bfloat16)
        want_res = res.clone()
        for _ in range(3):
            part = (torch.randn(B, 1, hidden, generator=g, device=dev) * 0.3).to(torch.bfloat16)
            want_res, want_out = _ref_add_norm(want_res, [part], weight, 1e-5)
            out = comm.allreduce_add_rmsnorm(part, res, weight, 1e-5)
            assert torch.equal(res, want_res)
            assert float((out.float() - want_out.float()).abs().max()) <= 2e-2 * float(want_out.float().abs().max())
        assert comm.status() == 0
    finally:
        comm.close()


def test_swiglu_packed_matches_two_tensor_form():
    from calibquant_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(2)
    gu = torch.randn(16, 1, 2 * 1792, generator=g, device="cuda").to(torch.bfloat16)
    want = ops.swiglu(gu[..., :1792].contiguous(), gu[..., 1792:].contiguous())
    assert torch.equal(ops.swiglu_packed(gu), want)


def test_argument_checks():
    from calibquant_b200 import _lib, tp
    lib = _lib.lib()
    assert lib.cq_comm_buffer_bytes(9, 1024) == 0
    assert lib.cq_comm_buffer_bytes(2, 1000) == 4096 + 256 + 2 * 2 * 1024
    comms = tp.PeerComm.local_group(2, 4096, torch.device("cuda"))
    try:
        x = torch.zeros(4096, dtype=torch.float16, device="cuda")          # 8192 bytes > the slot
        with pytest.raises(ValueError):
            comms[0].push(x)
    finally:
        for c in comms:
            c.close()
