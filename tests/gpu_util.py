"""Helpers shared by the GPU parity tests."""

import torch


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.cpu(), b.cpu()
    assert a.dtype == b.dtype and a.shape == b.shape, (a.dtype, b.dtype, a.shape, b.shape)
    if a.dtype in (torch.float16, torch.bfloat16):
        return torch.equal(a.view(torch.int16), b.view(torch.int16))
    return torch.equal(a, b)


def mismatch_count(a, b):
    a, b = a.cpu(), b.cpu()
    if a.dtype in (torch.float16, torch.bfloat16):
        a, b = a.view(torch.int16), b.view(torch.int16)
    return int((a != b).sum())


def rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    x, ref = x.detach().cpu().double(), ref.detach().cpu().double()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))
