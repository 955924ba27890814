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


def test_cpu_tensors_are_rejected():
    import torch
    from calibquant_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.pack_last_dim(torch.zeros(1, 1, 1, 32, dtype=torch.float16), 32, 1)
    # a host query is a legal input of the decode step (host-buffer entry point), a host cache is not
    z = torch.zeros(1, 4, 8, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.decode_attention(z[:, :, :1], None, None, z[:, :1], z[:, :1], 0, 1)
