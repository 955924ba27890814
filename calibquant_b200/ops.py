"""Tensor-level entry points over the C ABI.

torch is used here for device memory and streams only: every function hands raw
device pointers of CUDA tensors to ``libcalibquant_b200.so`` on torch's current
stream.  CPU tensors are rejected -- there is no fallback implementation.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import DecodeArgs, check, lib

_DTYPES = {torch.float16: _lib.CQ_DTYPE_F16, torch.bfloat16: _lib.CQ_DTYPE_BF16}


def _dtype_enum(t: torch.Tensor) -> int:
    if t.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float16 or bfloat16")
    return _DTYPES[t.dtype]


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("calibquant_b200 runs on CUDA tensors only (no CPU fallback)")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


class _OnDevice:
    """Make ``device`` current for the duration of a call; a no-op (no driver calls) when it already is."""

    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx, self.prev = device.index, None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


_workspaces = {}
_decode_ws_bytes = {}      # problem extents -> bytes, so a decode loop asks the library once


def _workspace(nbytes: int, device, stream_handle=None) -> torch.Tensor:
    """Grow-only scratch buffer per (device, stream), zeroed when created: its first word is
    the sticky device status the decode kernels set when a bounded wait runs out."""
    # A capture reuses the buffer an eager warm-up call created (a fixed address the replays can use).  A buffer
    # that has to be created while a CUDA graph is being captured lives in that graph's memory pool: it is kept
    # for captures only, eager calls on the same stream never see it.
    stream = torch.cuda.current_stream(device).cuda_stream if stream_handle is None else stream_handle
    capturing = bool(torch.cuda.is_current_stream_capturing())
    key = (device.index, stream, False)
    buf = _workspaces.get(key)
    if capturing and (buf is None or buf.numel() < nbytes):
        key = (device.index, stream, True)
        buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        new = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)
        if buf is not None:
            new[:4].copy_(buf[:4])      # a sticky status survives the regrowth
        _workspaces[key] = buf = new
    return buf


def device_status(device=None) -> int:
    """Sticky status word of the current stream's decode workspace (0 = no device-side wait has
    timed out since the workspace was created).  Synchronises the stream."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    stream = torch.cuda.current_stream(device).cuda_stream
    status = 0
    for capturing in (False, True):
        buf = _workspaces.get((device.index, stream, capturing))
        if buf is not None and status == 0:
            status = int(buf[:4].view(torch.int32).item())
    return status


def pack_last_dim(data: torch.Tensor, group_size: int, bits: int):
    """Group-wise quantize + pack along the last dim of a 4-D tensor.

    Returns (code int32 [B,nh,R,L*bits/32], scale [B,nh,R,L/g], mn [B,nh,R,L/g]).
    """
    _need_cuda(data)
    assert data.dim() == 4
    B, nh, R, L = data.shape
    assert L % group_size == 0
    data = data.contiguous()
    rows = B * nh * R
    code = torch.empty((B, nh, R, L * bits // 32), dtype=torch.int32, device=data.device)
    scale = torch.empty((B, nh, R, L // group_size), dtype=data.dtype, device=data.device)
    mn = torch.empty_like(scale)
    with torch.cuda.device(data.device):
        rc = lib().cq_pack_last_dim(_ptr(data), rows, L, group_size, bits, _dtype_enum(data),
                                    _ptr(code), _ptr(scale), _ptr(mn), _stream())
    check(rc, "cq_pack_last_dim")
    return code, scale, mn


def pack_k_per_channel(k: torch.Tensor, group_size: int, bits: int):
    """Per-channel quantize + pack of K given as [B,H,T,D] (any batch/head/token strides,
    channels contiguous), as if ``pack_last_dim(k.transpose(2,3).contiguous())``.

    Returns (code [B,H,D,T*bits/32], scale [B,H,D,T/g], mn [B,H,D,T/g]).
    """
    _need_cuda(k)
    assert k.dim() == 4
    B, H, T, D = k.shape
    assert T % group_size == 0
    if k.stride(3) != 1 or any(s % 8 for s in k.stride()[:3]) or k.data_ptr() % 16:
        k = k.contiguous()
    code = torch.empty((B, H, D, T * bits // 32), dtype=torch.int32, device=k.device)
    scale = torch.empty((B, H, D, T // group_size), dtype=k.dtype, device=k.device)
    mn = torch.empty_like(scale)
    with torch.cuda.device(k.device):
        rc = lib().cq_pack_k_per_channel(_ptr(k), B, H, T, D, k.stride(0), k.stride(1), k.stride(2),
                                         group_size, bits, _dtype_enum(k),
                                         _ptr(code), _ptr(scale), _ptr(mn), _stream())
    check(rc, "cq_pack_k_per_channel")
    return code, scale, mn


def pack_v_per_token(v: torch.Tensor, group_size: int, bits: int):
    """Per-token quantize + pack of V given as [B,H,T,D] through its strides (channels contiguous),
    as ``pack_last_dim(v.contiguous())`` without the copy.

    Returns (code [B,H,T,D*bits/32], scale [B,H,T,D/g], mn [B,H,T,D/g]).
    """
    _need_cuda(v)
    assert v.dim() == 4
    B, H, T, D = v.shape
    if v.stride(3) != 1 or any(s % 8 for s in v.stride()[:3]) or v.data_ptr() % 16:
        v = v.contiguous()
    code = torch.empty((B, H, T, D * bits // 32), dtype=torch.int32, device=v.device)
    scale = torch.empty((B, H, T, D // group_size), dtype=v.dtype, device=v.device)
    mn = torch.empty_like(scale)
    with torch.cuda.device(v.device):
        rc = lib().cq_pack_v_per_token(_ptr(v), B, H, T, D, v.stride(0), v.stride(1), v.stride(2),
                                       group_size, bits, _dtype_enum(v),
                                       _ptr(code), _ptr(scale), _ptr(mn), _stream())
    check(rc, "cq_pack_v_per_token")
    return code, scale, mn


def qbmm(group_size: int, fA: torch.Tensor, qB: torch.Tensor, scales: torch.Tensor,
         zeros: torch.Tensor, bits: int) -> torch.Tensor:
    """out[b,h,0,n] = sum_k fA[b,h,0,k]*(scales*code+zeros)[b,h//n_rep,k,n].

    fA [B,Hq,1,K]; qB [B,Hkv,K,N*bits/32]; scales, zeros [B,Hkv,K,N/g].  Hkv may equal Hq
    (operands already expanded, as the reference passes them) or divide it (GQA).
    """
    _need_cuda(fA, qB, scales, zeros)
    assert fA.dim() == 4 and qB.dim() == 4
    B, Hq, M, K = fA.shape
    if M != 1:
        raise ValueError("only M == 1 (one query row) is implemented")
    Hkv = qB.shape[1]
    N = qB.shape[-1] * (32 // bits)
    fA, qB = fA.contiguous(), qB.contiguous()
    scales, zeros = scales.contiguous(), zeros.contiguous()
    out = torch.empty((B, Hq, 1, N), dtype=fA.dtype, device=fA.device)
    nbytes = lib().cq_qbmm_workspace_bytes(B, Hq, K, N)
    ws = _workspace(nbytes, fA.device)      # its first word is the status word device_status() reads
    with torch.cuda.device(fA.device):
        rc = lib().cq_qbmm(_ptr(fA), _ptr(qB), _ptr(scales), _ptr(zeros), _ptr(out), B, Hq, Hkv,
                           K, N, group_size, bits, _dtype_enum(fA), _ptr(ws), ws.numel(), _stream())
    check(rc, "cq_qbmm")
    return out


def decode_attention(q, k_pack, v_pack, k_fp, v_fp, t_sys, bits, group_size=32,
                     calibrate=None, mask=None, out=None, t_fp=None, t_fp_dev=None, _prepare=False, _profile=None):
    """One decode step over [sys | visual (quantized) | text].

    q [B,Hq,1,D] or [B,Hq,D]; k_pack/v_pack = (code, scale, mn) in the group format (K per
    channel, V per token) or None when there are no quantized tokens; k_fp/v_fp [B,Hkv,T_fp,D]
    (token rows contiguous; batch/head strides free) hold the system tokens followed by the
    text tokens; ``t_fp`` limits how many of their rows are valid (default: all).
    ``mask``: optional additive [B, T_fp+T_vis] in key order [sys | visual | text].
    Returns o with q's shape.

    A ``q`` in host memory selects the host-buffer entry point: the query is copied in, the result
    lands in ``out`` (a host tensor; page-locked memory is written by the kernel itself) and the call
    returns once it is there.
    """
    host = not q.is_cuda
    dev = (k_fp if k_fp is not None else k_pack[0]).device
    _need_cuda(*(() if host else (q,)), k_fp, v_fp, mask, *(k_pack or ()), *(v_pack or ()))
    shape = q.shape
    B, Hq, D = shape[0], shape[1], shape[-1]
    q2 = q.reshape(B, Hq, D).contiguous()
    Hkv = k_fp.shape[1] if k_fp is not None else k_pack[0].shape[1]
    a = DecodeArgs()
    a.batch, a.n_q_heads, a.n_kv_heads, a.head_dim = B, Hq, Hkv, D
    a.bits, a.group_size, a.dtype = bits, group_size, _dtype_enum(q)
    a.calibrate = int(bits <= 2 if calibrate is None else calibrate)
    if not host:
        a.q = q2.data_ptr()
    keep = [q2]
    if k_pack is not None and k_pack[0].numel() > 0:
        kc, ks, kmn = (t.contiguous() for t in k_pack)
        vc, vs, vmn = (t.contiguous() for t in v_pack)
        keep += [kc, ks, kmn, vc, vs, vmn]
        a.t_vis = vc.shape[2]
        a.k_code, a.k_scale, a.k_mn = kc.data_ptr(), ks.data_ptr(), kmn.data_ptr()
        a.v_code, a.v_scale, a.v_mn = vc.data_ptr(), vs.data_ptr(), vmn.data_ptr()
    else:
        a.t_vis = 0
    if k_fp is not None and k_fp.shape[2] > 0:
        for t in (k_fp, v_fp):
            if t.stride(3) != 1 or t.stride(2) != D:
                raise ValueError("k_fp/v_fp token rows must be contiguous ([.., T, D] with stride D)")
        if k_fp.stride() != v_fp.stride():
            raise ValueError("k_fp and v_fp must share strides")
        a.t_fp = k_fp.shape[2] if t_fp is None else t_fp
        a.k_fp, a.v_fp = k_fp.data_ptr(), v_fp.data_ptr()
        a.fp_stride_b, a.fp_stride_h = k_fp.stride(0), k_fp.stride(1)
    else:
        a.t_fp = 0
    a.t_sys = min(t_sys, a.t_fp)
    if t_fp_dev is not None:      # int32 device scalar: live token count, a.t_fp is the capacity
        assert t_fp_dev.dtype == torch.int32 and t_fp_dev.is_cuda
        keep.append(t_fp_dev)
        a.t_fp_dev = t_fp_dev.data_ptr()
    if mask is not None:
        mask = mask.reshape(B, -1)
        if mask.dtype != q.dtype or mask.stride(1) != 1:
            mask = mask.to(q.dtype).contiguous()
        if mask.shape[1] != a.t_vis + a.t_fp:
            raise ValueError(f"Attention mask should cover {a.t_vis + a.t_fp} keys, but covers {mask.shape[1]}")
        keep.append(mask)
        a.mask, a.mask_stride_b = mask.data_ptr(), mask.stride(0)
    if out is None:
        out = torch.empty((B, Hq, D), dtype=q.dtype, pin_memory=True) if host else \
            torch.empty((B, Hq, D), dtype=q.dtype, device=dev)
    if host:
        if out.is_cuda or not out.is_contiguous() or out.dtype != q.dtype or out.numel() != B * Hq * D:
            raise ValueError("with q in host memory, out must be a contiguous host tensor of q's size and dtype")
    else:
        a.out = out.data_ptr()
    ref = ctypes.byref(a)
    aligned = all((ptr or 0) % 16 == 0 for ptr in (a.q, a.k_code, a.k_scale, a.k_mn, a.v_code, a.v_scale, a.v_mn,
                                                   a.k_fp, a.v_fp))      # decides which kernels serve the call
    key = (B, Hq, Hkv, D, a.t_vis, a.t_fp, bits, group_size, a.dtype, a.mask is not None, a.t_fp_dev is not None,
           a.k_code is not None, aligned, host)
    nbytes = _decode_ws_bytes.get(key)
    if nbytes is None:
        if len(_decode_ws_bytes) > 4096:      # a long generation adds one entry per text-cache length
            _decode_ws_bytes.clear()
        size_fn = lib().cq_decode_attn_host_workspace_bytes if host else lib().cq_decode_attn_workspace_bytes
        nbytes = _decode_ws_bytes[key] = size_fn(ref)
    handle = torch.cuda.current_stream(dev).cuda_stream      # looked up once per call
    if host:
        ws = _workspace(max(nbytes, 256), dev, handle)
        fn, ws_ptr, ws_n, st = lib().cq_decode_attn_host, _ptr(ws), ws.numel() if nbytes else 0, ctypes.c_void_p(handle)
        if _prepare:
            n_el = B * Hq * D

            def run(q_host, out_host):
                if q_host.is_cuda or out_host.is_cuda or q_host.dtype != q.dtype or out_host.dtype != q.dtype or \
                        q_host.numel() != n_el or out_host.numel() != n_el or \
                        not (q_host.is_contiguous() and out_host.is_contiguous()):
                    raise ValueError("prepared decode step: q_host/out_host must be contiguous host tensors of the "
                                     "prepared size and dtype")
                with _OnDevice(dev):
                    rc = fn(ref, q_host.data_ptr(), out_host.data_ptr(), ws_ptr, ws_n, st)
                if rc:
                    check(rc, "cq_decode_attn_host")
                return out_host
            run._keep = (a, keep, ws)      # the argument block holds raw pointers into these
            return run
        with _OnDevice(dev):
            rc = fn(ref, ctypes.c_void_p(q2.data_ptr()), ctypes.c_void_p(out.data_ptr()), ws_ptr, ws_n, st)
        check(rc, "cq_decode_attn_host")
        return out.reshape(shape)
    if nbytes == 0:      # the size query refused the arguments: let the call itself say why
        rc = lib().cq_decode_attn(ref, None, 0, ctypes.c_void_p(handle))
        check(rc if rc else _lib.CQ_ERR_WORKSPACE, "cq_decode_attn")
    ws = _workspace(nbytes, dev, handle)
    with _OnDevice(dev):
        if _profile is not None:      # a ctypes float[4]: per-launch milliseconds of this step
            rc = lib().cq_decode_attn_profile(ref, _ptr(ws), ws.numel(), ctypes.c_void_p(handle), _profile)
        else:
            rc = lib().cq_decode_attn(ref, _ptr(ws), ws.numel(), ctypes.c_void_p(handle))
    check(rc, "cq_decode_attn")
    return out.reshape(shape)


def decode_attention_profile(*args, **kw):
    """One decode step as :func:`decode_attention` runs it, timed launch by launch with CUDA events.
    Returns (out, {"scores": ms, "attn_v": ms, "attn_v_fp": ms, "combine": ms}).  Synchronises."""
    ms = (ctypes.c_float * 4)()
    out = decode_attention(*args, _profile=ms, **kw)
    return out, dict(zip(("scores", "attn_v", "attn_v_fp", "combine"), (float(v) for v in ms)))


def prepare_host_decode(q_host, k_pack, v_pack, k_fp, v_fp, t_sys, bits, **kw):
    """Decode step prepared once for a serving loop that keeps the cache fixed between calls and holds
    the query and the result in host memory: returns ``step(q_host, out_host) -> out_host``, one C call
    (``cq_decode_attn_host``) per step on the stream that was current here.  ``q_host`` gives shape and
    dtype; arguments as for :func:`decode_attention`.  The cache tensors' addresses
    are baked in: the caller keeps them alive and in place (their contents may change)."""
    if q_host.is_cuda:
        raise ValueError("prepare_host_decode wants the query in host memory")
    return decode_attention(q_host, k_pack, v_pack, k_fp, v_fp, t_sys, bits, _prepare=True, **kw)


def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out=None) -> torch.Tensor:
    """Causal attention over unquantized K/V in the flash_attn layout.

    q [B,T,Hq,D], k/v [B,T,Hkv,D] (any batch/token/head strides that are multiples of 8 elements,
    channels contiguous) -> o [B,T,Hq,D] in q.dtype.
    """
    _need_cuda(q, k, v)
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]

    def ok(t):
        return t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0

    q, k, v = (t if ok(t) else t.contiguous() for t in (q, k, v))
    if out is None:
        out = torch.empty((B, T, Hq, D), dtype=q.dtype, device=q.device)
    arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    with torch.cuda.device(q.device):
        rc = lib().cq_prefill_attn(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, T, Hq, Hkv, D,
                                   arr(q), arr(k), arr(v), arr(out), _dtype_enum(q), _stream())
    check(rc, "cq_prefill_attn")
    return out


def prefill_rope_split(qkv, cos, sin, position_ids, n_kv_heads, n_rep, k_cache=None, v_cache=None,
                       vis_start=0, vis_len=0):
    """A whole prompt: split the ``wqkv`` output ``qkv`` [B,T,Hkv*(n_rep+2)*D], rotate queries and keys
    with the ``cos``/``sin`` tables [S,D] at ``position_ids`` [B,T] (None: 0..T-1) in one launch.

    Returns (q [B,T,Hq,D], k [B,T,Hkv,D], v [B,T,Hkv,D]); ``v`` is a strided view into ``qkv``.  When
    the fp caches ``k_cache``/``v_cache`` [B,Hkv,capacity,D] are given, every token outside
    ``[vis_start, vis_start+vis_len)`` is also written there (rotated key, value), the tokens after the
    span following the ones before it."""
    _need_cuda(qkv, cos, sin)
    B, T = qkv.shape[0], qkv.shape[1]
    D = cos.shape[-1]
    per_tok = n_kv_heads * (n_rep + 2) * D
    if qkv.dim() != 3 or qkv.shape[2] != per_tok:
        raise ValueError(f"qkv must be [B,T,{per_tok}], got {tuple(qkv.shape)}")
    if qkv.stride(2) != 1 or qkv.stride(0) % 8 or qkv.stride(1) % 8 or qkv.data_ptr() % 16:
        qkv = qkv.contiguous()
    if cos.dtype != qkv.dtype or sin.dtype != qkv.dtype:
        raise TypeError("qkv and rotary tables must share one dtype")
    cos, sin = cos.contiguous(), sin.contiguous()
    pos = None
    if position_ids is not None:
        pos = position_ids.reshape(-1, T)
        if pos.shape[0] == 1 and B > 1:
            pos = pos.expand(B, T)
        if pos.dtype != torch.int64 or pos.shape[0] != B:
            raise ValueError("position_ids must be int64 [B,T]")
        pos = pos.contiguous()
    if (k_cache is None) != (v_cache is None):
        raise ValueError("give both caches or neither")
    cap = sb = sh = 0
    if k_cache is not None:
        for t in (k_cache, v_cache):
            if t.dtype != qkv.dtype or t.stride(3) != 1 or t.stride(2) != D:
                raise ValueError("caches must be [B,Hkv,capacity,D] of the data dtype with contiguous token rows")
        if k_cache.stride() != v_cache.stride():
            raise ValueError("k_cache and v_cache must share strides")
        cap, sb, sh = k_cache.shape[2], k_cache.stride(0), k_cache.stride(1)
        if T - vis_len > cap:
            raise ValueError(f"{T - vis_len} full-precision tokens do not fit a cache of {cap}")
    q = torch.empty((B, T, n_kv_heads * n_rep, D), dtype=qkv.dtype, device=qkv.device)
    k = torch.empty((B, T, n_kv_heads, D), dtype=qkv.dtype, device=qkv.device)
    with torch.cuda.device(qkv.device):
        rc = lib().cq_prefill_rope_split(_ptr(qkv), qkv.stride(0), qkv.stride(1), _ptr(cos), _ptr(sin), cos.shape[0],
                                         _ptr(pos), B, T, n_kv_heads, n_rep, D, _ptr(q), _ptr(k), _ptr(k_cache),
                                         _ptr(v_cache), sb, sh, cap, int(vis_start), int(vis_len),
                                         _dtype_enum(qkv), _stream())
    check(rc, "cq_prefill_rope_split")
    v = qkv.view(B, T, n_kv_heads, n_rep + 2, D)[:, :, :, n_rep + 1]
    return q, k, v


def rope_split_append(qkv, cos, sin, position_ids, n_kv_heads, n_rep, k_cache, v_cache,
                      append_index=None, t_fp_dev=None):
    """One decode token per batch row: split the ``wqkv`` output ``qkv`` [B,1,Hkv*(n_rep+2)*D]
    (per KV head: n_rep query heads, key, value), rotate queries and key with the ``cos``/``sin``
    tables [S,D] at ``position_ids`` [B,1], and write the rotated key and the value into the fp caches
    ``k_cache``/``v_cache`` [B,Hkv,capacity,D] at token ``append_index`` -- or at ``t_fp_dev - 1`` when
    the live token count is the int32 device scalar ``t_fp_dev`` (which then already counts the new
    token).  Returns the rotated queries [B,Hq,1,D]."""
    _need_cuda(qkv, cos, sin, position_ids, k_cache, v_cache)
    B = qkv.shape[0]
    D = cos.shape[-1]
    qkv2 = qkv.reshape(B, -1)
    if qkv2.stride(1) != 1:
        qkv2 = qkv2.contiguous()
    if qkv2.shape[1] != n_kv_heads * (n_rep + 2) * D:
        raise ValueError(f"qkv rows must hold {n_kv_heads * (n_rep + 2) * D} elements, got {qkv2.shape[1]}")
    if cos.dtype != qkv.dtype or sin.dtype != qkv.dtype or k_cache.dtype != qkv.dtype:
        raise TypeError("qkv, rotary tables and caches must share one dtype")
    cos, sin = cos.contiguous(), sin.contiguous()
    pos = position_ids.reshape(-1)
    if pos.dtype != torch.int64 or pos.numel() != B:
        raise ValueError("position_ids must be int64 with one position per batch row")
    pos = pos.contiguous()
    for t in (k_cache, v_cache):
        if t.stride(3) != 1 or t.stride(2) != D:
            raise ValueError("cache token rows must be contiguous ([.., T, D] with stride D)")
    if k_cache.stride() != v_cache.stride():
        raise ValueError("k_cache and v_cache must share strides")
    if (append_index is None) == (t_fp_dev is None):
        raise ValueError("give exactly one of append_index and t_fp_dev")
    if t_fp_dev is not None:
        assert t_fp_dev.dtype == torch.int32 and t_fp_dev.is_cuda
    q_out = torch.empty((B, n_kv_heads * n_rep, 1, D), dtype=qkv.dtype, device=qkv.device)
    with torch.cuda.device(qkv.device):
        rc = lib().cq_rope_split_append(_ptr(qkv2), qkv2.stride(0), _ptr(cos), _ptr(sin), cos.shape[0], _ptr(pos),
                                        B, n_kv_heads, n_rep, D, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                        k_cache.stride(0), k_cache.stride(1), k_cache.shape[2],
                                        0 if append_index is None else int(append_index), _ptr(t_fp_dev),
                                        _dtype_enum(qkv), _stream())
    check(rc, "cq_rope_split_append")
    return q_out


def add_rmsnorm(residual, delta, weight, eps, out=None, normalize=True):
    """``residual += delta`` in place (skipped when ``delta`` is None), then RMSNorm of the rows of
    ``residual`` [..., hidden] scaled by ``weight``.  Returns the normalised tensor (None when
    ``normalize`` is False: the bare residual add)."""
    _need_cuda(residual, delta, weight)
    hidden = residual.shape[-1]
    if not residual.is_contiguous() or (delta is not None and not delta.is_contiguous()):
        raise ValueError("residual and delta must be contiguous")
    if delta is not None and (delta.shape != residual.shape or delta.dtype != residual.dtype):
        raise ValueError("delta must match residual in shape and dtype")
    if normalize:
        if weight.dtype != residual.dtype or weight.numel() != hidden:
            raise ValueError("weight must hold `hidden` values of the data dtype")
        weight = weight.contiguous()
        if out is None:
            out = torch.empty_like(residual)
    rows = residual.numel() // hidden if hidden else 0
    with torch.cuda.device(residual.device):
        rc = lib().cq_add_rmsnorm(_ptr(delta), _ptr(residual), _ptr(weight) if normalize else None,
                                  _ptr(out) if normalize else None, rows, hidden, float(eps),
                                  _dtype_enum(residual), _stream())
    check(rc, "cq_add_rmsnorm")
    return out if normalize else None


def swiglu(gate, up, out=None):
    """``silu(gate) * up`` with torch's two roundings (the activation, then the product)."""
    _need_cuda(gate, up)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must match in shape and dtype")
    gate, up = gate.contiguous(), up.contiguous()
    if out is None:
        out = torch.empty_like(gate)
    with torch.cuda.device(gate.device):
        rc = lib().cq_swiglu(_ptr(gate), _ptr(up), _ptr(out), gate.numel(), _dtype_enum(gate), _stream())
    check(rc, "cq_swiglu")
    return out


def swiglu_packed(gate_up, out=None):
    """``silu(gate) * up`` for ``gate_up`` [..., 2n] holding the gate columns first, then the up columns (the
    output of one GEMM against stacked ``w1`` / ``w3`` weights).  Returns [..., n]."""
    _need_cuda(gate_up)
    n2 = gate_up.shape[-1]
    if n2 % 2 or not gate_up.is_contiguous():
        raise ValueError("gate_up must be contiguous with an even last dimension")
    n = n2 // 2
    rows = gate_up.numel() // n2 if n2 else 0
    if out is None:
        out = torch.empty((*gate_up.shape[:-1], n), dtype=gate_up.dtype, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        rc = lib().cq_swiglu_packed(_ptr(gate_up), _ptr(out), rows, n, _dtype_enum(gate_up), _stream())
    check(rc, "cq_swiglu_packed")
    return out


def _proj_dtype_enum(proj, data):
    if proj.dtype == torch.float32:
        return _lib.CQ_DTYPE_F32
    if proj.dtype == data.dtype:
        return _dtype_enum(data)
    raise TypeError("Unsupported data types for QJL: the projection must be float32 or match the keys")


def qjl_quant(key_states, outlier_indices, rand_prj, outlier_sketch_dim):
    """QJL sign sketch of grouped keys.  key_states [B,H,n,G,128]; outlier_indices uint8 [B,H,n,oc];
    rand_prj [sketch_dim,128].  Returns (key_quant uint8 [B,H,n,G,sketch_dim/8], key_outlier_quant uint8
    [B,H,n,G,outlier_sketch_dim/8], outlier_norms [B,H,n,G] in the key dtype)."""
    _need_cuda(key_states, outlier_indices, rand_prj)
    B, H, n, G, D = key_states.shape
    dt = _dtype_enum(key_states)
    pdt = _proj_dtype_enum(rand_prj, key_states)
    if outlier_indices.dtype != torch.uint8 or outlier_indices.shape[:3] != (B, H, n):
        raise ValueError("outlier_indices must be uint8 [B,H,n,outlier_count]")
    key_states, outlier_indices, rand_prj = key_states.contiguous(), outlier_indices.contiguous(), rand_prj.contiguous()
    s = rand_prj.shape[0]
    kq = torch.empty((B, H, n, G, s // 8), dtype=torch.uint8, device=key_states.device)
    koq = torch.empty((B, H, n, G, outlier_sketch_dim // 8), dtype=torch.uint8, device=key_states.device)
    norms = torch.empty((B, H, n, G), dtype=key_states.dtype, device=key_states.device)
    with torch.cuda.device(key_states.device):
        rc = lib().cq_qjl_quant(_ptr(key_states), _ptr(outlier_indices), _ptr(rand_prj), pdt, B * H * n, G, D, s,
                                outlier_sketch_dim, outlier_indices.shape[3], dt, _ptr(kq), _ptr(koq), _ptr(norms),
                                _stream())
    check(rc, "cq_qjl_quant")
    return kq, koq, norms


def qjl_gqa_score(key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices, query_sketch,
                  query_states, rand_prj):
    """Score estimate of one query per head against QJL-sketched keys (GQA: the keys stay at KV-head
    count).  query_states [B,Hq,1,128], query_sketch fp32 [B,Hq,1,sketch_dim], rand_prj [128,sketch_dim].
    Returns fp32 [B,Hq,n*G,1] as the reference's kernel does."""
    _need_cuda(key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices, query_sketch,
               query_states, rand_prj)
    B, Hkv, n, G, hb = key_quant.shape
    Hq, D = query_states.shape[1], query_states.shape[-1]
    dt = _dtype_enum(query_states)
    pdt = _proj_dtype_enum(rand_prj, query_states)
    if query_sketch.dtype != torch.float32:
        query_sketch = query_sketch.float()
    if key_norm.dtype != query_states.dtype or key_outlier_norm.dtype != query_states.dtype:
        raise TypeError("key norms must have the query dtype")
    if Hq % Hkv:
        raise ValueError("query heads must be a multiple of key heads")
    tensors = [t.contiguous() for t in (key_quant, key_outlier_quant, key_norm, key_outlier_norm, outlier_indices,
                                        query_sketch, query_states, rand_prj)]
    scores = torch.empty((B, Hq, n * G, 1), dtype=torch.float32, device=query_states.device)
    with torch.cuda.device(query_states.device):
        rc = lib().cq_qjl_gqa_score(*[_ptr(t) for t in tensors], pdt, B, Hkv, Hq // Hkv, n, G, D, hb * 8,
                                    key_outlier_quant.shape[-1] * 8, outlier_indices.shape[3], dt, _ptr(scores),
                                    _stream())
    check(rc, "cq_qjl_gqa_score")
    return scores
