"""Drop-in for the reference module ``qjl/qjl_utils.py``: ``repeat_kv_quant``, the Johnson-
Lindenstrauss sign sketch ``QJLSketch`` and the streaming KV-cache key quantizer ``QJLKeyQuantizer``
(constructor and methods of ``qjl/qjl_utils.py:99-195``: ``build_sketch``, ``update_sketch``,
``attention_score``, the fp residual buffer that is flushed every ``buffer_size`` tokens).

``QJLKeyQuantizer(None, ...)`` (no sketch object) keeps the same interface but stores keys in the
per-channel group format of ``qjl/new_pack.py`` at ``qjl_dim`` bits.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from . import qjl_kernel


def repeat_kv_quant(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B,Hkv,S,X] -> [B,Hkv*n_rep,S,X] (``qjl/qjl_utils.py:6-11``).  The kernels of this package
    take the un-repeated tensors, so this exists only for callers that still expand explicitly."""
    batch, num_key_value_heads, slen, head_dim = hidden_states.shape
    if n_rep == 1:
        return hidden_states
    hidden_states = hidden_states[:, :, None, :, :].expand(batch, num_key_value_heads, n_rep, slen, head_dim)
    return hidden_states.reshape(batch, num_key_value_heads * n_rep, slen, head_dim)


class QJLSketch(torch.nn.Module):
    """Random projection of the QJL method (``qjl/qjl_utils.py:14-96``).  ``dim = (head_dim,
    sketch_dim)``; with ``rot=True`` every 128-column block of the Gaussian matrix is replaced by the
    Q factor of its QR decomposition times sqrt(head_dim).  ``proj_dir_score`` [head_dim, sketch_dim]
    sketches queries, its transpose ``proj_dir_quant`` quantizes keys."""

    def __init__(self, dim, dim_outlier, device=None, rng=None, rot=True, rht=False):
        super().__init__()
        self.device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
        assert len(dim) == 2, "dim should be a tuple of 2 elements"
        if rht:
            raise NotImplementedError("the randomized Hadamard variant needs scipy's hadamard; not built")
        self.dim = dim
        self.dim_outlier = dim_outlier
        self.proj_dir = self._init_proj_dir(rng).contiguous()
        self.proj_dir_score = self.init_rot_dir().contiguous() if rot else self.proj_dir.to(torch.float16)
        self.proj_dir_quant = self.proj_dir_score.transpose(0, 1).contiguous()

    def _init_proj_dir(self, rng):
        return torch.randn(self.dim, generator=rng, dtype=torch.float32, device=self.device)

    def init_rot_dir(self):
        rot_matrices = []
        num_chunks = (self.dim[1] + self.dim[0] - 1) // self.dim[0]
        for i in range(num_chunks):
            q, _ = torch.linalg.qr(self.proj_dir[:, i * self.dim[0]:(i + 1) * self.dim[0]], mode="reduced")
            rot_matrices.append(q)
        return torch.cat(rot_matrices, dim=-1) * math.sqrt(self.dim[0])

    def quantize(self, data, outlier_indices):
        """data [B,H,n,G,D], outlier_indices uint8 [B,H,n,oc] -> (key_quant, key_outlier_quant,
        key_outlier_norm)."""
        assert data.shape[-1] == self.dim[0], "embedding dimension should match projection dimension"
        assert data.shape[:3] == outlier_indices.shape[:3], "outlier indices shape should match input shape"
        return qjl_kernel.qjl_quant(data, outlier_indices, self.proj_dir_quant, self.dim_outlier)

    def calc_score(self, query, data_quant, outlier_quant, outlier_indices, norm_data, norm_outlier):
        """query [B,Hq,1,D] against sketched keys -> fp32 scores [B,Hq,n*G,1]."""
        assert query.shape[-1] == self.dim[0], "embedding dimension should match projection dimension"
        assert query.shape[:1] == data_quant.shape[:1] == outlier_indices.shape[:1], \
            "query shape should match outlier indices and data quant shapes"
        assert data_quant.shape[:4] == norm_data.shape[:4], "data quant and its norm should have same shape"
        assert outlier_quant.shape[:4] == norm_outlier.shape[:4], "outlier quant and its norm should have same shape"
        sketched_q = torch.matmul(query.to(self.proj_dir_score.dtype), self.proj_dir_score)
        return qjl_kernel.qjl_gqa_score(data_quant, outlier_quant, norm_data, norm_outlier, outlier_indices,
                                        sketched_q, query, self.proj_dir_score)


class QJLKeyQuantizer:
    """Streaming key cache: sketched blocks plus an fp residual of fewer than ``buffer_size`` keys
    (``qjl/qjl_utils.py:99-195``).  With ``qjl_sketch=None`` see ``_GroupFormatKeyQuantizer``."""

    def __new__(cls, qjl_sketch, *args, **kwargs):
        if qjl_sketch is None and cls is QJLKeyQuantizer:
            return object.__new__(_GroupFormatKeyQuantizer)
        return object.__new__(cls)

    def __init__(self, qjl_sketch, outliers_count: int, buffer_size: int, group_size: int, qjl_dim: int) -> None:
        self.qjl_sketch = qjl_sketch
        self.outliers_count = outliers_count
        self.buffer_size = buffer_size
        self.group_size = group_size
        self.qjl_dim = qjl_dim
        self.seq_len = None
        self.outlier_indices = None
        self.key_states_quant = None
        self.key_outliers_quant = None
        self.key_outliers_norm = None
        self.key_states_norm = None
        self.key_residual = None

    def _sketch_groups(self, groups: torch.Tensor):
        """groups [B,H,n,G,D] -> appends their sketches, outlier sets and norms."""
        norms = groups.norm(dim=-2)
        _, idx = norms.topk(self.outliers_count, dim=-1)
        idx = idx.to(torch.uint8).contiguous()
        kq, koq, onorm = self.qjl_sketch.quantize(groups.contiguous(), idx)
        knorm = torch.norm(groups, dim=-1)
        if self.key_states_quant is None:
            self.outlier_indices, self.key_states_quant, self.key_outliers_quant = idx, kq, koq
            self.key_outliers_norm, self.key_states_norm = onorm, knorm
        else:
            self.outlier_indices = torch.cat([self.outlier_indices, idx], dim=2)
            self.key_states_quant = torch.cat([self.key_states_quant, kq], dim=2)
            self.key_outliers_quant = torch.cat([self.key_outliers_quant, koq], dim=2)
            self.key_outliers_norm = torch.cat([self.key_outliers_norm, onorm], dim=2)
            self.key_states_norm = torch.cat([self.key_states_norm, knorm], dim=2)

    def build_sketch(self, key_states: torch.Tensor) -> None:
        """key_states [B,Hkv,T,D]: sketch the first T - T % buffer_size keys, keep the rest fp."""
        b, h, _, dim = key_states.shape
        self.seq_len = key_states.shape[-2]
        residual_size = self.seq_len % self.buffer_size
        if residual_size > 0:
            self.key_residual = key_states[:, :, self.seq_len - residual_size:, :]
        if residual_size == self.seq_len:
            return None
        num_groups = (self.seq_len - residual_size) // self.group_size
        self._sketch_groups(key_states[:, :, :self.seq_len - residual_size, :].reshape(
            (b, h, num_groups, self.group_size, dim)))

    def update_sketch(self, key_states: torch.Tensor) -> None:
        assert key_states.shape[-2] == 1, "appending more than one embedding in the stream!"
        self.seq_len += 1
        if self.key_residual is not None:
            self.key_residual = torch.cat([self.key_residual, key_states], dim=-2)
        else:
            self.key_residual = key_states
        if self.seq_len % self.buffer_size != 0:
            return None
        b, h, _, dim = self.key_residual.shape
        self._sketch_groups(self.key_residual.reshape((b, h, -1, self.group_size, dim)))
        self.key_residual = None

    def attention_score(self, query_states: torch.Tensor) -> torch.Tensor:
        """query_states [B,Hq,1,D] -> unscaled scores [B,Hq,1,T] (fp32) over sketched keys + residual."""
        b, h, _, dim = query_states.shape
        assert query_states.shape[-2] == 1, "appending more than one embedding in the stream!"
        parts = []
        if self.key_states_quant is not None:
            parts.append(self.qjl_sketch.calc_score(query_states, self.key_states_quant,
                                                    self.key_outliers_quant.contiguous(), self.outlier_indices,
                                                    self.key_states_norm, self.key_outliers_norm).transpose(-1, -2))
        if self.key_residual is not None:
            residual = repeat_kv_quant(self.key_residual, n_rep=h // self.key_residual.shape[1])
            parts.append(torch.matmul(query_states, residual.transpose(-1, -2)))
        return torch.cat(parts, dim=-1) if len(parts) > 1 else parts[0]


class _GroupFormatKeyQuantizer(QJLKeyQuantizer):
    """Same interface, keys kept in the per-channel group format of ``qjl/new_pack.py`` at
    ``qjl_dim`` bits (``qjl_sketch`` and ``outliers_count`` are ignored)."""

    def __init__(self, qjl_sketch, outliers_count: int, buffer_size: int, group_size: int, qjl_dim: int) -> None:
        self.qjl_sketch = qjl_sketch
        self.outliers_count = outliers_count
        self.buffer_size = buffer_size
        self.group_size = group_size
        self.bits = qjl_dim
        self.seq_len = None
        self.blocks = []            # list of (code, scale, mn) per flushed block, K per channel
        self.key_residual = None    # [B,Hkv,r,D], r < buffer_size

    def _quantize(self, keys: torch.Tensor):
        self.blocks.append(ops.pack_k_per_channel(keys, self.group_size, self.bits))

    def build_sketch(self, key_states: torch.Tensor) -> None:
        """key_states [B,Hkv,T,D]: quantize the first T - T % buffer_size keys, keep the rest fp."""
        self.seq_len = key_states.shape[-2]
        residual_size = self.seq_len % self.buffer_size
        if residual_size > 0:
            self.key_residual = key_states[:, :, self.seq_len - residual_size:, :].contiguous()
        if residual_size == self.seq_len:
            return None
        self._quantize(key_states[:, :, :self.seq_len - residual_size, :])

    def update_sketch(self, key_states: torch.Tensor) -> None:
        assert key_states.shape[-2] == 1, "appending more than one embedding in the stream!"
        self.seq_len += 1
        if self.key_residual is not None:
            self.key_residual = torch.cat([self.key_residual, key_states], dim=-2)
        else:
            self.key_residual = key_states
        if self.seq_len % self.buffer_size != 0:
            return None
        self._quantize(self.key_residual)
        self.key_residual = None

    def attention_score(self, query_states: torch.Tensor) -> torch.Tensor:
        """query_states [B,Hq,1,D] -> unscaled scores [B,Hq,1,T] over quantized blocks + residual."""
        assert query_states.shape[-2] == 1, "appending more than one embedding in the stream!"
        parts = [ops.qbmm(self.group_size, query_states, code, scale, mn, self.bits)
                 for code, scale, mn in self.blocks]
        if self.key_residual is not None:
            n_rep = query_states.shape[1] // self.key_residual.shape[1]
            residual = repeat_kv_quant(self.key_residual, n_rep)
            parts.append(torch.matmul(query_states, residual.transpose(-1, -2)))
        return torch.cat(parts, dim=-1) if len(parts) > 1 else parts[0]
