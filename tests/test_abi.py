"""The C-ABI library must load and export every symbol that include/calibquant_b200.h declares
(no compute calls: this runs without a GPU)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "calibquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cq_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def handle():
    from calibquant_b200 import build
    path = build.build_library()
    return ctypes.CDLL(path)


def test_header_declares_entry_points():
    syms = _declared_symbols()
    for must in ("cq_pack_last_dim", "cq_pack_k_per_channel", "cq_qbmm", "cq_decode_attn",
                 "cq_decode_attn_workspace_bytes", "cq_decode_attn_host", "cq_decode_attn_host_workspace_bytes",
                 "cq_version", "cq_status_string"):
        assert must in syms


def test_library_exports_every_declared_symbol(handle):
    for name in _declared_symbols():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    from calibquant_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_symbols()


def test_version_and_status_strings(handle):
    handle.cq_status_string.restype = ctypes.c_char_p
    assert handle.cq_version() >= 100
    assert handle.cq_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert len(handle.cq_status_string(code)) > 3


def test_argument_validation_needs_no_gpu(handle):
    """Bad arguments are rejected on the host before any CUDA call."""
    from calibquant_b200 import _lib
    lib = _lib.lib()
    assert lib.cq_pack_last_dim(None, 1, 32, 32, 1, 0, None, None, None, None) == _lib.CQ_ERR_BAD_ARG
    assert lib.cq_pack_last_dim(None, 0, 32, 32, 1, 0, None, None, None, None) == _lib.CQ_OK   # empty
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    p16 = ctypes.c_void_p((p.value + 15) // 16 * 16)
    assert lib.cq_pack_last_dim(p16, 1, 32, 32, 3, 0, p16, p16, p16, None) == _lib.CQ_ERR_UNSUPPORTED
    assert lib.cq_pack_last_dim(p16, 1, 48, 32, 1, 0, p16, p16, p16, None) == _lib.CQ_ERR_UNSUPPORTED
    assert lib.cq_pack_last_dim(p16, 1, 32, 64, 1, 0, p16, p16, p16, None) == _lib.CQ_ERR_UNSUPPORTED
    assert lib.cq_pack_last_dim(p16, 1, 32, 32, 1, 7, p16, p16, p16, None) == _lib.CQ_ERR_BAD_ARG
    a = _lib.DecodeArgs()
    assert lib.cq_decode_attn_workspace_bytes(ctypes.byref(a)) == 0
    assert lib.cq_decode_attn(ctypes.byref(a), None, 0, None) == _lib.CQ_ERR_BAD_ARG
    a.batch, a.n_q_heads, a.n_kv_heads, a.head_dim = 1, 4, 1, 64
    a.t_vis, a.t_fp, a.bits, a.group_size = 32, 0, 1, 32
    a.q = a.out = a.k_code = a.k_scale = a.k_mn = a.v_code = a.v_scale = a.v_mn = p16.value
    assert lib.cq_decode_attn(ctypes.byref(a), None, 0, None) == _lib.CQ_ERR_UNSUPPORTED  # head_dim
    a.head_dim = 128
    assert lib.cq_decode_attn_workspace_bytes(ctypes.byref(a)) > 0
    assert lib.cq_decode_attn(ctypes.byref(a), None, 0, None) == _lib.CQ_ERR_WORKSPACE


def test_argument_validation_of_the_newer_entry_points(handle):
    """Prefill split + RoPE, strided V pack, the uint8-format decode step and the peer-buffer collectives reject bad
    arguments on the host, before any CUDA call."""
    from calibquant_b200 import _lib
    lib = _lib.lib()
    buf = ctypes.create_string_buffer(4096)
    p16 = ctypes.c_void_p((ctypes.cast(buf, ctypes.c_void_p).value + 15) // 16 * 16)
    # cq_prefill_rope_split: empty prompt is a no-op, null operands / a span past the prompt / odd strides are not
    args = lambda **kw: [kw.get("qkv", p16), kw.get("sb", 6 * 128 * 8), kw.get("st", 6 * 128), p16, p16, 64, None,
                         kw.get("batch", 1), kw.get("t_len", 8), 1, 4, kw.get("head_dim", 128), p16, p16, None, None,
                         0, 0, 0, kw.get("vis_start", 0), kw.get("vis_len", 0), 0, None]
    assert lib.cq_prefill_rope_split(*args(batch=0)) == _lib.CQ_OK
    assert lib.cq_prefill_rope_split(*args(qkv=None)) == _lib.CQ_ERR_BAD_ARG
    assert lib.cq_prefill_rope_split(*args(vis_start=4, vis_len=8)) == _lib.CQ_ERR_BAD_ARG
    assert lib.cq_prefill_rope_split(*args(st=6 * 128 + 4)) == _lib.CQ_ERR_BAD_ARG
    assert lib.cq_prefill_rope_split(*args(head_dim=64)) == _lib.CQ_ERR_UNSUPPORTED
    # cq_pack_v_per_token
    assert lib.cq_pack_v_per_token(p16, 0, 2, 8, 128, 0, 0, 0, 32, 1, 0, p16, p16, p16, None) == _lib.CQ_OK
    assert lib.cq_pack_v_per_token(None, 1, 2, 8, 128, 2048, 128, 256, 32, 1, 0, p16, p16, p16, None) == _lib.CQ_ERR_BAD_ARG
    assert lib.cq_pack_v_per_token(p16, 1, 2, 8, 128, 2048, 128, 256, 32, 3, 0, p16, p16, p16, None) == _lib.CQ_ERR_UNSUPPORTED
    assert lib.cq_pack_v_per_token(p16, 1, 2, 8, 128, 2044, 128, 256, 32, 1, 0, p16, p16, p16, None) == _lib.CQ_ERR_BAD_ARG
    # cq_u8_decode_attn
    a = _lib.U8DecodeArgs()
    assert lib.cq_u8_decode_attn_workspace_bytes(ctypes.byref(a)) == 0
    assert lib.cq_u8_decode_attn(ctypes.byref(a), None, 0, None) == _lib.CQ_ERR_BAD_ARG
    a.batch, a.n_q_heads, a.n_kv_heads, a.head_dim = 1, 4, 1, 128
    a.t_vis, a.t_fp, a.t_sys, a.bits, a.dtype, a.n_scale_heads = 64, 0, 0, 1, 0, 4
    for f in ("q", "out", "enc_k", "enc_v", "scale_key", "zero_point_key", "scale_value", "zero_point_value"):
        setattr(a, f, p16.value)
    assert lib.cq_u8_decode_attn_workspace_bytes(ctypes.byref(a)) > 0
    assert lib.cq_u8_decode_attn(ctypes.byref(a), None, 0, None) == _lib.CQ_ERR_WORKSPACE
    a.n_scale_heads = 3
    assert lib.cq_u8_decode_attn(ctypes.byref(a), None, 0, None) == _lib.CQ_ERR_BAD_ARG
    a.n_scale_heads, a.t_vis = 4, 60000                       # more keys than a shared-memory row holds
    assert lib.cq_u8_decode_attn(ctypes.byref(a), None, 0, None) == _lib.CQ_ERR_UNSUPPORTED
    # peer-buffer sizes
    assert lib.cq_comm_buffer_bytes(2, 8192) > 2 * 2 * 8192
    assert lib.cq_comm_buffer_bytes(0, 8192) == 0 or lib.cq_comm_buffer_bytes(9, 8192) == 0


def test_cpu_tensors_are_rejected():
    import torch
    from calibquant_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.pack_last_dim(torch.zeros(1, 1, 1, 32, dtype=torch.float16), 32, 1)
    # a host query is a legal input of the decode step (host-buffer entry point), a host cache is not
    z = torch.zeros(1, 4, 8, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.decode_attention(z[:, :, :1], None, None, z[:, :1], z[:, :1], 0, 1)
