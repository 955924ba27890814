"""ctypes binding of ``libcalibquant_b200.so`` (the C ABI declared in include/calibquant_b200.h).

There is no CPU fallback: if the library has not been built, or a call returns a
negative status, the caller gets an exception.
"""

from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libcalibquant_b200.so")

CQ_OK = 0
CQ_ERR_BAD_ARG = -1
CQ_ERR_UNSUPPORTED = -2
CQ_ERR_LAUNCH = -3
CQ_ERR_WORKSPACE = -4
CQ_ERR_TIMEOUT = -5
CQ_ERR_TOO_LARGE = -6

CQ_DTYPE_F16 = 0
CQ_DTYPE_BF16 = 1
CQ_DTYPE_F32 = 2

_c = ctypes
_vp, _i32, _i64, _sz = _c.c_void_p, _c.c_int32, _c.c_int64, _c.c_size_t


class DecodeArgs(_c.Structure):
    """Mirror of ``struct cq_decode_args``."""

    _fields_ = [
        ("batch", _i32), ("n_q_heads", _i32), ("n_kv_heads", _i32), ("head_dim", _i32),
        ("t_vis", _i32), ("t_fp", _i32), ("t_sys", _i32),
        ("bits", _i32), ("group_size", _i32), ("dtype", _i32),
        ("calibrate", _i32), ("reserved", _i32),
        ("q", _vp), ("k_code", _vp), ("k_scale", _vp), ("k_mn", _vp),
        ("v_code", _vp), ("v_scale", _vp), ("v_mn", _vp),
        ("k_fp", _vp), ("v_fp", _vp),
        ("fp_stride_b", _i64), ("fp_stride_h", _i64),
        ("mask", _vp), ("mask_stride_b", _i64),
        ("out", _vp),
        ("t_fp_dev", _vp),
    ]


class U8DecodeArgs(_c.Structure):
    """Mirror of ``struct cq_u8_decode_args``."""

    _fields_ = [
        ("batch", _i32), ("n_q_heads", _i32), ("n_kv_heads", _i32), ("head_dim", _i32),
        ("t_vis", _i32), ("t_fp", _i32), ("t_sys", _i32),
        ("bits", _i32), ("dtype", _i32), ("calibrate", _i32), ("n_scale_heads", _i32), ("reserved", _i32),
        ("q", _vp), ("enc_k", _vp), ("enc_v", _vp),
        ("scale_key", _vp), ("zero_point_key", _vp), ("scale_value", _vp), ("zero_point_value", _vp),
        ("k_fp", _vp), ("v_fp", _vp),
        ("fp_stride_b", _i64), ("fp_stride_h", _i64),
        ("mask", _vp), ("mask_stride_b", _i64),
        ("out", _vp),
        ("t_fp_dev", _vp),
    ]


# name -> (restype, argtypes); every symbol include/calibquant_b200.h declares.
SIGNATURES = {
    "cq_version": (_c.c_int, []),
    "cq_status_string": (_c.c_char_p, [_c.c_int]),
    "cq_pack_last_dim": (_c.c_int, [_vp, _i64, _i64, _c.c_int, _c.c_int, _c.c_int, _vp, _vp, _vp, _vp]),
    "cq_pack_k_per_channel": (_c.c_int, [_vp, _c.c_int, _c.c_int, _i64, _c.c_int, _i64, _i64, _i64,
                                         _c.c_int, _c.c_int, _c.c_int, _vp, _vp, _vp, _vp]),
    "cq_pack_v_per_token": (_c.c_int, [_vp, _c.c_int, _c.c_int, _i64, _c.c_int, _i64, _i64, _i64,
                                       _c.c_int, _c.c_int, _c.c_int, _vp, _vp, _vp, _vp]),
    "cq_qbmm_workspace_bytes": (_sz, [_c.c_int, _c.c_int, _i64, _i64]),
    "cq_qbmm": (_c.c_int, [_vp, _vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _c.c_int, _i64, _i64,
                           _c.c_int, _c.c_int, _c.c_int, _vp, _sz, _vp]),
    "cq_qbmm_static_capacity_bytes": (_sz, []),
    "cq_qbmm_static": (_c.c_int, [_vp, _vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _c.c_int, _i64, _i64,
                                  _c.c_int, _c.c_int, _c.c_int, _vp]),
    "cq_prefill_attn": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                   _c.POINTER(_i64), _c.POINTER(_i64), _c.POINTER(_i64), _c.POINTER(_i64),
                                   _c.c_int, _vp]),
    "cq_prefill_status": (_c.c_int, []),
    "cq_calib_minmax": (_c.c_int, [_vp, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_i64), _c.c_int,
                                   _c.c_float, _c.c_int, _vp, _vp, _vp]),
    "cq_calib_quantize": (_c.c_int, [_vp, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_i64), _c.c_int,
                                     _c.c_int, _vp, _vp, _c.c_int, _vp, _vp, _vp]),
    "cq_calib_encode_i64": (_c.c_int, [_vp, _i64, _c.c_int, _vp, _vp]),
    "cq_lut_scores": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                 _c.c_int, _c.c_int, _vp]),
    "cq_lut_out_workspace_bytes": (_sz, [_c.c_int, _c.c_int, _c.c_int]),
    "cq_lut_out": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                              _c.c_int, _c.c_int, _vp, _sz, _vp]),
    "cq_u8_decode_attn_workspace_bytes": (_sz, [_c.POINTER(U8DecodeArgs)]),
    "cq_u8_decode_attn": (_c.c_int, [_c.POINTER(U8DecodeArgs), _vp, _sz, _vp]),
    "cq_rope_split_append": (_c.c_int, [_vp, _i64, _vp, _vp, _c.c_int, _vp, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                        _vp, _vp, _vp, _i64, _i64, _c.c_int, _c.c_int, _vp, _c.c_int, _vp]),
    "cq_prefill_rope_split": (_c.c_int, [_vp, _i64, _i64, _vp, _vp, _c.c_int, _vp, _c.c_int, _c.c_int, _c.c_int,
                                         _c.c_int, _c.c_int, _vp, _vp, _vp, _vp, _i64, _i64, _c.c_int, _c.c_int,
                                         _c.c_int, _c.c_int, _vp]),
    "cq_add_rmsnorm": (_c.c_int, [_vp, _vp, _vp, _vp, _i64, _c.c_int, _c.c_float, _c.c_int, _vp]),
    "cq_swiglu": (_c.c_int, [_vp, _vp, _vp, _i64, _c.c_int, _vp]),
    "cq_swiglu_packed": (_c.c_int, [_vp, _vp, _i64, _i64, _c.c_int, _vp]),
    "cq_comm_buffer_bytes": (_sz, [_c.c_int, _sz]),
    "cq_comm_alloc": (_c.c_int, [_sz, _c.POINTER(_vp), _vp]),
    "cq_comm_open": (_c.c_int, [_vp, _c.POINTER(_vp)]),
    "cq_comm_close": (_c.c_int, [_vp]),
    "cq_comm_free": (_c.c_int, [_vp]),
    "cq_comm_status": (_c.c_int, [_vp, _vp]),
    "cq_comm_push": (_c.c_int, [_vp, _sz, _c.POINTER(_vp), _c.c_int, _c.c_int, _sz, _vp]),
    "cq_comm_reduce_add_rmsnorm": (_c.c_int, [_vp, _c.c_int, _sz, _vp, _vp, _vp, _i64, _c.c_int, _c.c_float,
                                              _c.c_int, _vp]),
    "cq_comm_gather": (_c.c_int, [_vp, _c.c_int, _sz, _vp, _sz, _vp]),
    "cq_comm_allreduce_add_rmsnorm": (_c.c_int, [_vp, _c.POINTER(_vp), _c.c_int, _c.c_int, _sz, _vp, _vp, _vp, _i64,
                                                 _c.c_int, _c.c_float, _c.c_int, _vp]),
    "cq_qjl_quant": (_c.c_int, [_vp, _vp, _vp, _c.c_int, _i64, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                _c.c_int, _vp, _vp, _vp, _vp]),
    "cq_qjl_gqa_score": (_c.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                    _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _vp, _vp]),
    "cq_decode_attn_workspace_bytes": (_sz, [_c.POINTER(DecodeArgs)]),
    "cq_decode_attn": (_c.c_int, [_c.POINTER(DecodeArgs), _vp, _sz, _vp]),
    "cq_decode_attn_profile": (_c.c_int, [_c.POINTER(DecodeArgs), _vp, _sz, _vp, _c.POINTER(_c.c_float)]),
    "cq_workspace_status": (_c.c_int, [_vp, _vp]),
    "cq_host_status_word": (_c.POINTER(_c.c_int), []),
    "cq_qbmm_static_status": (_c.c_int, [_vp]),
    "cq_decode_attn_host_workspace_bytes": (_sz, [_c.POINTER(DecodeArgs)]),
    "cq_decode_attn_host": (_c.c_int, [_c.POINTER(DecodeArgs), _vp, _vp, _vp, _sz, _vp]),
}

_lib = None


class CalibQuantError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        text = lib().cq_status_string(status).decode()
        super().__init__(f"{where}: status {status} ({text})")


def lib():
    """Load the shared library once; raise if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m calibquant_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        handle = _c.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, where: str):
    """Map a negative status to the exception type the reference raises for that failure:
    assertion-like argument/shape problems -> AssertionError/ValueError-compatible
    ``ValueError``; everything else -> ``CalibQuantError``."""
    if status == CQ_OK:
        return
    if status in (CQ_ERR_BAD_ARG, CQ_ERR_UNSUPPORTED):
        text = lib().cq_status_string(status).decode()
        raise ValueError(f"{where}: status {status} ({text})")
    raise CalibQuantError(status, where)
