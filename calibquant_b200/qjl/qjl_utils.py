"""Drop-in for the parts of the reference module ``qjl/qjl_utils.py`` that the quantized-KV
attention path uses: ``repeat_kv_quant`` and the KV-cache key quantizer object.

``QJLKeyQuantizer`` keeps the reference's constructor and methods (``qjl/qjl_utils.py:99-195``:
``build_sketch``, ``update_sketch``, ``attention_score``, the fp residual buffer that is flushed
every ``buffer_size`` tokens), but stores keys in the per-channel group format of
``qjl/new_pack.py`` at ``qjl_dim`` bits instead of a Johnson-Lindenstrauss sign sketch: the
sketch arithmetic belongs to the reference's separate QJL baseline, not to this path.
"""

from __future__ import annotations

import torch

from .. import ops


def repeat_kv_quant(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B,Hkv,S,X] -> [B,Hkv*n_rep,S,X] (``qjl/qjl_utils.py:6-11``).  The kernels of this package
    take the un-repeated tensors, so this exists only for callers that still expand explicitly."""
    batch, num_key_value_heads, slen, head_dim = hidden_states.shape
    if n_rep == 1:
        return hidden_states
    hidden_states = hidden_states[:, :, None, :, :].expand(batch, num_key_value_heads, n_rep, slen, head_dim)
    return hidden_states.reshape(batch, num_key_value_heads * n_rep, slen, head_dim)


class QJLKeyQuantizer:
    """Streaming key cache: quantized blocks plus an fp residual of fewer than ``buffer_size`` keys.

    ``qjl_sketch`` and ``outliers_count`` are accepted for signature compatibility and ignored.
    ``qjl_dim`` is the number of bits per key element (the reference passes ``k_bits`` there).
    """

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
