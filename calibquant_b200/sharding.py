"""Multi-GPU partitioning of the quantized-KV attention path (one process per GPU).

The reference has no multi-GPU code; attention is independent per (batch row, KV head), so two
partitionings are offered:

* **by KV head** (model decode): rank r owns the contiguous KV heads ``[r*Hkv/G, (r+1)*Hkv/G)`` and
  their query heads.  It needs only its rows of ``wqkv`` -- contiguous, because the projection
  emits per KV head ``(n_rep q heads, k, v)`` (``patch_internvl.py:219-234``) -- packs and holds only
  its heads' cache, and produces ``o_r [B, Hq/G, D]``.  One collective per layer and step: an
  all-gather of ``o_r`` into ``[B, Hq*D]`` (NCCL over NVLink on GPUs, gloo in CPU tests), after
  which ``wo`` runs replicated.
* **by batch** (attention-only stress): rank r owns rows ``[r*B/G, (r+1)*B/G)``; no communication.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def kv_head_range(rank: int, world: int, n_kv_heads: int):
    """Contiguous KV-head range of ``rank``; ``world`` must divide ``n_kv_heads``."""
    if n_kv_heads % world:
        raise ValueError(f"world size {world} must divide the {n_kv_heads} KV heads")
    per = n_kv_heads // world
    return rank * per, (rank + 1) * per


def batch_range(rank: int, world: int, batch: int):
    """Rows of ``rank`` when the batch is split as evenly as possible (first ranks take the extra)."""
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def wqkv_rows(rank: int, world: int, n_kv_heads: int, n_rep: int, head_dim: int):
    """Row range of the fused ``wqkv`` weight that produces the q/k/v of this rank's KV heads."""
    h0, h1 = kv_head_range(rank, world, n_kv_heads)
    per_head = (n_rep + 2) * head_dim
    return h0 * per_head, h1 * per_head


def shard_wqkv(weight: torch.Tensor, rank: int, world: int, n_kv_heads: int, n_rep: int, head_dim: int):
    r0, r1 = wqkv_rows(rank, world, n_kv_heads, n_rep, head_dim)
    return weight[r0:r1]


def all_gather_heads(o_local: torch.Tensor, group=None) -> torch.Tensor:
    """o_local [B, Hq/G, D] on every rank -> [B, Hq, D] with rank r's heads at ``[r*Hq/G, ...)``.

    The collective gathers rank-major ``[G, B, Hq/G, D]``; the head-major view is formed afterwards
    (a copy of B*Hq*D elements, 16-96 KB per layer at the benchmark shapes).
    """
    world = dist.get_world_size(group)
    if world == 1:
        return o_local
    o_local = o_local.contiguous()
    B, h, D = o_local.shape
    gathered = torch.empty((world * B, h, D), dtype=o_local.dtype, device=o_local.device)
    dist.all_gather_into_tensor(gathered, o_local, group=group)
    return gathered.view(world, B, h, D).permute(1, 0, 2, 3).reshape(B, world * h, D)


def all_gather_last_dim(x: torch.Tensor, group=None) -> torch.Tensor:
    """x [..., n] on every rank -> [..., world*n], rank r's slice at ``[r*n, (r+1)*n)``."""
    world = dist.get_world_size(group)
    if world == 1:
        return x
    lead, n = x.shape[:-1], x.shape[-1]
    flat = x.reshape(-1, n).contiguous()
    gathered = torch.empty((world * flat.shape[0], n), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(gathered, flat, group=group)
    return gathered.view(world, flat.shape[0], n).permute(1, 0, 2).reshape(*lead, world * n)


class HeadShardedAttention:
    """Decode attention over this rank's KV heads followed by the all-gather of head outputs.

    ``attend(q_local, state) -> o_local [B, Hq/G, 1, D]`` is the local attention; by default it is
    ``ops.decode_attention`` on the rank's packed cache (``state`` = dict with ``k_pack, v_pack, k_fp,
    v_fp, t_sys, bits``).  Tests on CPU inject another callable to exercise the plumbing.
    """

    def __init__(self, rank: int, world: int, n_q_heads: int, n_kv_heads: int, head_dim: int = 128,
                 group=None, attend=None):
        self.rank, self.world, self.group = rank, world, group
        self.n_q_heads, self.n_kv_heads, self.head_dim = n_q_heads, n_kv_heads, head_dim
        self.n_rep = n_q_heads // n_kv_heads
        self.h0, self.h1 = kv_head_range(rank, world, n_kv_heads)
        self.attend = attend or self._attend_cuda

    @staticmethod
    def _attend_cuda(q_local, state):
        from . import ops
        return ops.decode_attention(q_local, state["k_pack"], state["v_pack"], state["k_fp"], state["v_fp"],
                                    state["t_sys"], state["bits"], calibrate=state.get("calibrate"))

    def local_q(self, q_all: torch.Tensor) -> torch.Tensor:
        """q_all [B, Hq, 1, D] -> this rank's query heads."""
        return q_all[:, self.h0 * self.n_rep:self.h1 * self.n_rep]

    def __call__(self, q_local: torch.Tensor, state) -> torch.Tensor:
        """Returns the gathered output [B, Hq, D] (identical on every rank)."""
        o = self.attend(q_local, state)
        B = o.shape[0]
        return all_gather_heads(o.reshape(B, -1, self.head_dim), self.group)
