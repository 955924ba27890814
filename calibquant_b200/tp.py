"""Tensor-parallel decode of the InternLM2 backbone over the GPUs of one node (one process per GPU).

The reference runs on one device; this module is the multi-GPU side of the decode path.  Rank r of G owns
the KV heads ``[r*Hkv/G, (r+1)*Hkv/G)`` with their query heads and the matching slices of every weight:

* ``wqkv``  rows of its KV heads (per KV head the projection emits n_rep q heads, k, v: contiguous rows),
* ``wo``    the columns that multiply its heads' outputs, so the product of its local attention output is a
            partial [B, hidden] sum -- the all-gather of head outputs followed by the full ``wo`` and the sum
            of the per-rank partial products are the same numbers, and the partial sums need no gather before
            the GEMM,
* ``w1/w3`` rows ``[r*F/G, (r+1)*F/G)`` stacked into one ``w13`` matrix, ``w2`` the matching columns
            (again a partial [B, hidden] sum),
* ``output`` rows of its vocabulary slice; the next token is the arg-max over the ranks' local maxima.

Two collectives per layer and step (after ``wo`` and after ``w2``), each a ``PeerComm.push`` of the partial rows
followed by the next layer-norm launch that sums the G partials it finds in its own buffer
(``cq_comm_push`` / ``cq_comm_reduce_add_rmsnorm``: plain peer stores over NVLink, no NCCL call on the decode
path).  The quantized KV cache is sharded with the heads, so attention needs no communication at all.
Prefill uses ``torch.distributed.all_reduce`` for the same sums (it is not the timed path).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, ops, sharding
from ._lib import check, lib


class PeerComm:
    """This rank's receive buffer plus the peers' buffers mapped through CUDA IPC."""

    def __init__(self, rank: int, world: int, slot_bytes: int, device, group=None, _local=None):
        self.rank, self.world, self.slot_bytes, self.device, self.group = rank, world, int(slot_bytes), device, group
        self._opened = []
        self.ptrs = (ctypes.c_void_p * world)()
        if _local is not None:                  # single-process group (tests, world == 1): pointers are shared
            self.buf = _local[rank]
            for q in range(world):
                self.ptrs[q] = _local[q]
            self._owned = False
            return
        self._owned = True
        nbytes = lib().cq_comm_buffer_bytes(world, self.slot_bytes)
        handle = (ctypes.c_ubyte * 64)()
        buf = ctypes.c_void_p()
        with torch.cuda.device(device):
            check(lib().cq_comm_alloc(nbytes, ctypes.byref(buf), handle), "cq_comm_alloc")
            self.buf = buf.value
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle), group=group)
            for q in range(world):
                if q == rank:
                    self.ptrs[q] = self.buf
                else:
                    peer = ctypes.c_void_p()
                    raw = (ctypes.c_ubyte * 64).from_buffer_copy(handles[q])
                    check(lib().cq_comm_open(raw, ctypes.byref(peer)), "cq_comm_open")
                    self.ptrs[q] = peer.value
                    self._opened.append(peer.value)
        dist.barrier(group=group)

    @classmethod
    def local_group(cls, world: int, slot_bytes: int, device):
        """``world`` communicators inside one process on one device (the buffers see each other directly).
        With them the ranks of a collective run one after the other on one stream -- all pushes, then all
        reduces -- which exercises slots, flags and sequence numbers without any concurrency."""
        nbytes = lib().cq_comm_buffer_bytes(world, slot_bytes)
        bufs, keep = [], []
        with torch.cuda.device(device):
            for _ in range(world):
                handle = (ctypes.c_ubyte * 64)()
                buf = ctypes.c_void_p()
                check(lib().cq_comm_alloc(nbytes, ctypes.byref(buf), handle), "cq_comm_alloc")
                bufs.append(buf.value)
        comms = [cls(r, world, slot_bytes, device, _local=bufs) for r in range(world)]
        comms[0]._free_all = bufs
        return comms

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def push(self, x: torch.Tensor):
        """First half of a collective: this rank's rows go to slot ``rank`` of every rank's buffer."""
        if not x.is_contiguous():
            x = x.contiguous()
        check(lib().cq_comm_push(ctypes.c_void_p(x.data_ptr()), x.numel() * x.element_size(), self.ptrs,
                                 self.rank, self.world, self.slot_bytes, self._stream()), "cq_comm_push")

    def reduce_add_rmsnorm(self, residual, weight, eps, out=None, normalize=True):
        """Second half: ``residual += sum of the pushed rows`` in place, then RMSNorm (as ``ops.add_rmsnorm``)."""
        hidden = residual.shape[-1]
        rows = residual.numel() // hidden
        if normalize and out is None:
            out = torch.empty_like(residual)
        check(lib().cq_comm_reduce_add_rmsnorm(ctypes.c_void_p(self.buf), self.world, self.slot_bytes,
                                               ctypes.c_void_p(residual.data_ptr()),
                                               ctypes.c_void_p(weight.data_ptr()) if normalize else None,
                                               ctypes.c_void_p(out.data_ptr()) if normalize else None,
                                               rows, hidden, float(eps), ops._dtype_enum(residual), self._stream()),
              "cq_comm_reduce_add_rmsnorm")
        return out if normalize else None

    def allreduce_add_rmsnorm(self, partial, residual, weight, eps, out=None, normalize=True):
        """A whole collective in one launch: ``residual += sum over the ranks of partial`` in place, then RMSNorm.
        Every rank calls it with its own ``partial`` [rows, hidden] (rows <= 64)."""
        hidden = residual.shape[-1]
        rows = residual.numel() // hidden
        if not partial.is_contiguous():
            partial = partial.contiguous()
        if normalize and out is None:
            out = torch.empty_like(residual)
        check(lib().cq_comm_allreduce_add_rmsnorm(ctypes.c_void_p(partial.data_ptr()), self.ptrs, self.rank, self.world,
                                                  self.slot_bytes, ctypes.c_void_p(residual.data_ptr()),
                                                  ctypes.c_void_p(weight.data_ptr()) if normalize else None,
                                                  ctypes.c_void_p(out.data_ptr()) if normalize else None,
                                                  rows, hidden, float(eps), ops._dtype_enum(residual), self._stream()),
              "cq_comm_allreduce_add_rmsnorm")
        return out if normalize else None

    def gather(self, like: torch.Tensor) -> torch.Tensor:
        """Second half: the pushed rows of all ranks, ``[world, *like.shape]``."""
        out = torch.empty((self.world, *like.shape), dtype=like.dtype, device=like.device)
        check(lib().cq_comm_gather(ctypes.c_void_p(self.buf), self.world, self.slot_bytes,
                                   ctypes.c_void_p(out.data_ptr()), like.numel() * like.element_size(),
                                   self._stream()), "cq_comm_gather")
        return out

    def status(self) -> int:
        """0, or CQ_ERR_TIMEOUT if a wait for a peer ran out since the buffer was made.  Synchronises."""
        return lib().cq_comm_status(ctypes.c_void_p(self.buf), self._stream())

    def close(self):
        for p in self._opened:
            lib().cq_comm_close(ctypes.c_void_p(p))
        self._opened = []
        if self._owned and self.buf:
            lib().cq_comm_free(ctypes.c_void_p(self.buf))
            self.buf = None
        for p in getattr(self, "_free_all", []):
            lib().cq_comm_free(ctypes.c_void_p(p))
        self._free_all = []


def _slice_linear(lin: torch.nn.Linear, rows=None, cols=None) -> torch.nn.Linear:
    w = lin.weight
    if rows is not None:
        w = w[rows[0]:rows[1]]
    if cols is not None:
        w = w[:, cols[0]:cols[1]]
    new = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, device=w.device, dtype=w.dtype)
    with torch.no_grad():
        new.weight.copy_(w)
    return new


def shard_layer_(layer, rank: int, world: int):
    """Keep this rank's slices of one decoder layer's weights (see the module docstring)."""
    attn, ff = layer.attention, layer.feed_forward
    n_rep, D = attn.num_key_value_groups, attn.head_dim
    r0, r1 = sharding.wqkv_rows(rank, world, attn.num_key_value_heads, n_rep, D)
    h0, h1 = sharding.kv_head_range(rank, world, attn.num_key_value_heads)
    attn.wqkv = _slice_linear(attn.wqkv, rows=(r0, r1))
    attn.wo = _slice_linear(attn.wo, cols=(h0 * n_rep * D, h1 * n_rep * D))
    attn._shard = (rank, world, None)
    attn._shard_rowparallel = True            # wo consumes the local heads: no gather of head outputs
    F = ff.w1.out_features
    if F % world:
        raise ValueError(f"world size {world} must divide the FFN width {F}")
    f0, f1 = rank * F // world, (rank + 1) * F // world
    w1, w3 = _slice_linear(ff.w1, rows=(f0, f1)), _slice_linear(ff.w3, rows=(f0, f1))
    w13 = torch.nn.Linear(w1.in_features, 2 * (f1 - f0), bias=False, device=w1.weight.device, dtype=w1.weight.dtype)
    with torch.no_grad():
        w13.weight[: f1 - f0].copy_(w1.weight)
        w13.weight[f1 - f0:].copy_(w3.weight)
    ff.w13 = w13
    ff.w1 = ff.w3 = None
    ff.w2 = _slice_linear(ff.w2, cols=(f0, f1))
    return layer


def shard_model_(lm, rank: int, world: int, comm: PeerComm | None, group=None):
    """Shard an ``InternLM2ForCausalLM`` in place for tensor-parallel decode.  ``comm`` carries the decode-step
    collectives; prefill sums go through ``torch.distributed`` on ``group``."""
    if world == 1:
        return lm
    for layer in lm.model.layers:
        shard_layer_(layer, rank, world)
    V = lm.output.out_features
    if V % world:
        raise ValueError(f"world size {world} must divide the vocabulary {V}")
    lm.output = _slice_linear(lm.output, rows=(rank * V // world, (rank + 1) * V // world))
    lm._tp = (rank, world, comm, group, V // world)
    return lm


def global_argmax_torch(local_logits: torch.Tensor, rank: int, world: int, vocab_per_rank: int, group=None):
    """Next token from vocabulary-sharded logits [B, V/G] with a ``torch.distributed`` all-gather (prefill)."""
    val, idx = local_logits.float().max(-1)
    mine = torch.stack([val, (idx + rank * vocab_per_rank).float()], -1).contiguous()
    allv = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allv, mine, group=group)
    allv = torch.stack(allv)                                   # [G, B, 2]
    best = allv[..., 0].argmax(0)
    return allv[best, torch.arange(mine.shape[0], device=mine.device), 1].long()


def global_argmax_peer(local_logits: torch.Tensor, comm: PeerComm, vocab_per_rank: int):
    """The same through the peer buffers (decode step; replayable from a CUDA graph)."""
    val, idx = local_logits.float().max(-1)
    mine = torch.stack([val, (idx + comm.rank * vocab_per_rank).float()], -1).contiguous()   # [B, 2] fp32
    if mine.numel() * 4 % 16:
        raise ValueError("batch must be even for the arg-max exchange")
    comm.push(mine)
    allv = comm.gather(mine)                                    # [G, B, 2]
    best = allv[..., 0].argmax(0)
    return allv[best, torch.arange(mine.shape[0], device=mine.device), 1].long()
