"""Drop-in for the reference module ``patch_internvl.py``: the model patch and the two patched
InternLM2 attention forwards, running on the calibquant_b200 CUDA kernels.

Kept from the reference (names, arguments, return values):
``patch_model(model, quant_method, **kwargs)`` (``patch_internvl.py:645-660``),
``ATTN_FORWARD_FUNCTIONS`` with keys ``"calibquant"`` and ``"qjl"`` (``:639-642``),
``custom_generate`` (``:35-93``), ``repeat_kv`` (``:97-106``), ``rotate_half`` /
``apply_rotary_pos_emb`` (``:110-138``), the module globals ``BITS_KV, SCALE_K, SCALE_V, LOW_BITS,
SPROMPT_LEN, CHUNK_SIZE`` (``:20-31``) and the ``IMAGE_TOKEN_NUM`` environment side channel
(``:78, :189``).

What changes underneath:
* the visual span of the KV cache is held in the group format (K per channel, V per token,
  32-element groups, ``BITS_KV`` bits) written by one pack kernel each;
* a decode step is ONE call (``ops.decode_attention``) covering scores with post-scaling, logit
  calibration, softmax, packed attn.V and the fp16 system/text segments -- no ``repeat_kv`` copies,
  no transposes, no per-step ``torch.cat`` of the text cache (it lives in a pre-allocated buffer);
* prefill attention is ``ops.prefill_attention`` (causal over the whole sequence, no chunk loop).
"""

from __future__ import annotations

import math
import os
import warnings
from typing import Optional, Tuple

import torch

from . import ops
from .qjl.matmul import cuda_quantized_bmm_dynamic
from .qjl.new_pack import triton_quantize_and_pack_along_last_dim
from .qjl.qjl_utils import QJLKeyQuantizer, repeat_kv_quant

# global hyperparameters for quantization (same names and defaults as the reference)
BITS_KV = 1
# layout of the quantized visual span: "group" (32-element groups, the layout of the reference's qjl kernels)
# or "uint8" (the reference's calibquant forward: one scale per channel over the whole span, clip factors
# SCALE_K / SCALE_V, bytes packed most-significant field first); chosen by patch_model(..., kv_format=...)
KV_FORMAT = "group"

if BITS_KV == 1:
    SCALE_V = 0.3
    SCALE_K = 0.5
else:
    SCALE_V = 1
    SCALE_K = 1

LOW_BITS = True
SPROMPT_LEN = 41
CHUNK_SIZE = 1024      # kept for compatibility; the prefill kernel needs no chunking
GROUP_SIZE = 32
TEXT_CAPACITY_STEP = 256   # growth step of the pre-allocated system+text cache


@torch.no_grad()
def custom_generate(self, pixel_values=None, input_ids=None, attention_mask=None, visual_features=None,
                    generation_config=None, output_hidden_states=None, **generate_kwargs):
    """``InternVLChatModel.generate`` replacement (``patch_internvl.py:35-93``): embeds the prompt,
    scatters the ViT features over the image-context tokens, publishes ``IMAGE_TOKEN_NUM`` and
    calls the language model's ``generate`` with ``inputs_embeds``."""
    assert self.img_context_token_id is not None
    if pixel_values is not None:
        if visual_features is not None:
            vit_embeds = visual_features
        else:
            chunks = [self.extract_feature(pixel_values[i:i + 10]) for i in range(0, pixel_values.size(0), 10)]
            vit_embeds = torch.cat(chunks, dim=0)
        input_embeds = self.language_model.get_input_embeddings()(input_ids)
        B, N, C = input_embeds.shape
        input_embeds = input_embeds.reshape(B * N, C)
        selected = input_ids.reshape(B * N) == self.img_context_token_id
        assert selected.sum() != 0
        input_embeds[selected] = vit_embeds.reshape(-1, C).to(input_embeds.device)
        os.environ["IMAGE_TOKEN_NUM"] = str(int(vit_embeds.shape[0] * vit_embeds.shape[1] / B))
        input_embeds = input_embeds.reshape(B, N, C)
    else:
        input_embeds = self.language_model.get_input_embeddings()(input_ids)
    return self.language_model.generate(inputs_embeds=input_embeds, attention_mask=attention_mask,
                                        generation_config=generation_config,
                                        output_hidden_states=output_hidden_states, use_cache=True,
                                        **generate_kwargs)


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B,Hkv,S,D] -> [B,Hkv*n_rep,S,D]; kept for callers, the kernels never need it."""
    batch, num_key_value_heads, slen, head_dim = hidden_states.shape
    if n_rep == 1:
        return hidden_states
    hidden_states = hidden_states[:, :, None, :, :].expand(batch, num_key_value_heads, n_rep, slen, head_dim)
    return hidden_states.reshape(batch, num_key_value_heads * n_rep, slen, head_dim)


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids, unsqueeze_dim=1):
    """Non-interleaved RoPE on q [B,Hq,q,D] and k [B,Hkv,q,D]; cos/sin are [seq, D] tables."""
    cos = cos[position_ids].unsqueeze(unsqueeze_dim)
    sin = sin[position_ids].unsqueeze(unsqueeze_dim)
    # same two rounded steps as the reference: copy.mul_(cos) then addcmul_(rotate_half(x), sin)
    return torch.addcmul(q * cos, rotate_half(q), sin), torch.addcmul(k * cos, rotate_half(k), sin)


class _dummy_class_for_accessing_shape:
    def __init__(self, kv_seq_len):
        self.shape = (-1, -1, kv_seq_len, -1)


class _TextCache:
    """System + text K/V of one layer in pre-allocated [B,Hkv,capacity,D] buffers.  ``views()``
    returns ``[B,Hkv,length,D]`` slices (token rows contiguous), so appending a token is one small
    copy instead of the reference's ``torch.cat`` of the whole cache (``patch_internvl.py:265-266``)."""

    def __init__(self, k, v):
        B, H, T, D = k.shape
        cap = T + TEXT_CAPACITY_STEP
        self.k = torch.empty((B, H, cap, D), dtype=k.dtype, device=k.device)
        self.v = torch.empty_like(self.k)
        self.k[:, :, :T] = k
        self.v[:, :, :T] = v
        self.length = T

    @classmethod
    def empty(cls, batch, heads, length, head_dim, dtype, device):
        """Buffers for ``length`` tokens that the caller fills (the fused prefill kernel writes them)."""
        self = cls.__new__(cls)
        self.k = torch.empty((batch, heads, length + TEXT_CAPACITY_STEP, head_dim), dtype=dtype, device=device)
        self.v = torch.empty_like(self.k)
        self.length = length
        return self

    def append(self, k, v):
        n = k.shape[2]
        if self.length + n > self.k.shape[2]:
            grow = max(TEXT_CAPACITY_STEP, n)
            pad = torch.empty((*self.k.shape[:2], grow, self.k.shape[3]), dtype=self.k.dtype, device=self.k.device)
            self.k = torch.cat([self.k, pad], dim=2)
            self.v = torch.cat([self.v, pad.clone()], dim=2)
        self.k[:, :, self.length:self.length + n] = k
        self.v[:, :, self.length:self.length + n] = v
        self.length += n

    def views(self):
        return self.k[:, :, :self.length], self.v[:, :, :self.length]

    # ---- static mode: the token count lives on the device, so that one captured CUDA graph can
    # ---- append a token and attend over the live part at every decode step
    def enable_static(self, capacity, len_dev=None):
        """``len_dev``: int32 device scalar holding the live token count.  Layers of one model hold
        equally many tokens, so their caches may share one counter; whoever owns it adds one per
        decode step *before* the layers run (the count then includes the token being appended)."""
        if capacity > self.k.shape[2]:
            pad = torch.empty((*self.k.shape[:2], capacity - self.k.shape[2], self.k.shape[3]),
                              dtype=self.k.dtype, device=self.k.device)
            self.k = torch.cat([self.k, pad], dim=2)
            self.v = torch.cat([self.v, pad.clone()], dim=2)
        self.len_dev = len_dev if len_dev is not None else \
            torch.tensor([self.length], dtype=torch.int32, device=self.k.device)


def _split_qkv(self, hidden_states):
    """``wqkv`` output -> q [B,q,Hq,D], k [B,q,Hkv,D], v [B,q,Hkv,D] as strided views (no copies):
    per KV head the projection emits n_rep query heads, then k, then v (``patch_internvl.py:219-234``)."""
    bsz, q_len, _ = hidden_states.size()
    qkv = self.wqkv(hidden_states).view(bsz, q_len, -1, 2 + self.num_key_value_groups, self.head_dim)
    q = qkv[..., : self.num_key_value_groups, :].reshape(bsz, q_len, -1, self.head_dim)
    return q, qkv[..., -2, :], qkv[..., -1, :]


def _shard_world(self):
    shard = getattr(self, "_shard", None)
    return shard[1] if shard else 1


def _gather_heads(self, x):
    """x [B,q,Hq_local*D] -> [B,q,Hq*D].  Identity unless ``shard_attention_`` split this layer by KV
    head across ranks; then the single collective of the layer: an all-gather of the head outputs."""
    shard = getattr(self, "_shard", None)
    if not shard or getattr(self, "_shard_rowparallel", False):
        return x          # not sharded, or `wo` holds only the columns of the local heads (calibquant_b200.tp)
    from . import sharding
    return sharding.all_gather_last_dim(x, shard[2])


def shard_attention_(attn, rank: int, world: int, group=None):
    """Keep only this rank's KV heads in ``attn.wqkv`` (their rows are contiguous, see
    ``sharding.wqkv_rows``); the patched forward then packs, caches and attends over the local heads
    and all-gathers the head outputs before the (replicated) ``wo``."""
    from . import sharding
    if world == 1:
        return attn
    r0, r1 = sharding.wqkv_rows(rank, world, attn.num_key_value_heads, attn.num_key_value_groups, attn.head_dim)
    local = torch.nn.Linear(attn.wqkv.in_features, r1 - r0, bias=False, device=attn.wqkv.weight.device,
                            dtype=attn.wqkv.weight.dtype)
    with torch.no_grad():
        local.weight.copy_(attn.wqkv.weight[r0:r1])
    attn.wqkv = local
    attn._shard = (rank, world, group)
    return attn


def _image_token_num():
    return int(os.environ.get("IMAGE_TOKEN_NUM"))


def _pop_padding_mask(kwargs, attention_mask):
    if "padding_mask" in kwargs:
        warnings.warn("Passing `padding_mask` is deprecated and will be removed in v4.37. "
                      "Please make sure use `attention_mask` instead.`")
        attention_mask = kwargs.pop("padding_mask")
    return attention_mask


def forward_internlm2_calibquant(self, hidden_states: torch.Tensor,
                                 attention_mask: Optional[torch.LongTensor] = None,
                                 position_ids: Optional[torch.LongTensor] = None,
                                 past_key_value: Optional[Tuple[torch.Tensor]] = None,
                                 output_attentions: bool = False, use_cache: bool = False, **kwargs):
    """Patched ``InternLM2FlashAttention2.forward`` (``patch_internvl.py:141-484``).

    Prefill (q_len > 1): RoPE, quantize the visual span ``[SPROMPT_LEN, SPROMPT_LEN+IMAGE_TOKEN_NUM)``
    of K (per channel) and V (per token) at ``BITS_KV`` bits, keep system+text K/V in fp, run causal
    attention over the unquantized K/V.  Decode (q_len == 1): one fused attention call over
    [system | quantized visual | text] with logit calibration when ``BITS_KV <= 2``.
    Returns ``(attn_output, None, past_key_value)``; ``past_key_value`` is the legacy
    ``(K_fp, V_fp)`` tuple of system+text tokens and the quantized state lives on the module, as in
    the reference.
    """
    self.sprompt_len = SPROMPT_LEN
    self.image_token_num = _image_token_num()
    self.normalize = BITS_KV <= 2
    attention_mask = _pop_padding_mask(kwargs, attention_mask)
    bsz, q_len, _ = hidden_states.size()

    if q_len == 1 and getattr(self, "_static_decode", False):
        # graph-replayable step: everything that changes between steps is read from device memory.
        # One launch splits the projection, rotates q and k and appends k, v at the device-side
        # token count (already advanced by the owner of the counter), one call attends over the
        # live part of the cache.
        tc = self._text_cache
        cos, sin = self.rotary_emb(hidden_states, seq_len=self._static_rope_len)
        n_rep = self.num_key_value_groups
        q = ops.rope_split_append(self.wqkv(hidden_states), cos, sin, position_ids,
                                  self.wqkv.out_features // ((n_rep + 2) * self.head_dim), n_rep,
                                  tc.k, tc.v, t_fp_dev=tc.len_dev)
        if getattr(self, "_u8_state", None) is not None:
            from . import calibquant as _cq
            attn = _cq.decode_attention(q, self._u8_state, tc.k, tc.v, BITS_KV, self.sprompt_len,
                                        normalize=self.normalize, t_fp_dev=tc.len_dev).to(q.dtype)
        else:
            attn = ops.decode_attention(q, self.k_pack, self.v_pack, tc.k, tc.v, self.sprompt_len if LOW_BITS else 0,
                                        BITS_KV, group_size=GROUP_SIZE, calibrate=self.normalize and LOW_BITS,
                                        t_fp_dev=tc.len_dev)
        attn = _gather_heads(self, attn.transpose(1, 2).reshape(bsz, q_len, -1))
        return self.wo(attn.reshape(bsz, q_len, -1)), None, past_key_value

    if q_len > 1:
        # prefill: one launch splits the projection, rotates q and k and writes the system + text rows
        # of the fp cache; the pack kernels then read the visual span of the rotated keys and (in
        # place, through strides) of the values; the dense attention reads the same buffers.
        if past_key_value is not None:
            raise NotImplementedError("chunked prefill on top of an existing cache is not supported")
        n_rep = self.num_key_value_groups
        n_kv = self.wqkv.out_features // ((n_rep + 2) * self.head_dim)
        s0, n_vis = (self.sprompt_len, self.image_token_num) if LOW_BITS else (0, 0)
        if n_vis % GROUP_SIZE:
            raise ValueError(f"IMAGE_TOKEN_NUM must be a multiple of {GROUP_SIZE}, got {n_vis}")
        if s0 + n_vis > q_len:
            raise ValueError(f"the visual span [{s0}, {s0 + n_vis}) does not fit a prompt of {q_len} tokens")
        cos, sin = self.rotary_emb(hidden_states, seq_len=q_len)
        tc = _TextCache.empty(bsz, n_kv, q_len - n_vis, self.head_dim, hidden_states.dtype, hidden_states.device)
        q, k, v = ops.prefill_rope_split(self.wqkv(hidden_states), cos, sin, position_ids, n_kv, n_rep,
                                         tc.k, tc.v, s0, n_vis)
        self.k_pack = self.v_pack = self._u8_state = None
        if LOW_BITS and KV_FORMAT == "uint8":
            # patch_internvl.py:288-339: whole-span per-channel min-max with the clip factors, codes as bytes
            from . import calibquant as _cq
            enc_k, sk, zk = _cq.quant_encode(k[:, s0:s0 + n_vis], BITS_KV, scale=SCALE_K)
            enc_v, sv, zv = _cq.quant_encode(v[:, s0:s0 + n_vis], BITS_KV, scale=SCALE_V)
            self._u8_state = {"enc_k": enc_k, "enc_v": enc_v, "scale_key": sk, "zero_point_key": zk,
                              "scale_value": sv, "zero_point_value": zv}
        elif LOW_BITS:
            self.k_pack = ops.pack_k_per_channel(k.transpose(1, 2)[:, :, s0:s0 + n_vis], GROUP_SIZE, BITS_KV)
            self.v_pack = ops.pack_v_per_token(v.transpose(1, 2)[:, :, s0:s0 + n_vis], GROUP_SIZE, BITS_KV)
        self._text_cache = tc
        past_key_value = tc.views() if use_cache else None
        attn = ops.prefill_attention(q, k, v)
        attn = _gather_heads(self, attn.reshape(bsz, q_len, -1))
        attn_output = self.wo(attn.reshape(bsz, q_len, -1))
        return attn_output, None, past_key_value

    q, k, v = _split_qkv(self, hidden_states)
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)          # [B,H,q,D] views
    kv_seq_len = q_len
    if past_key_value is not None:
        kv_seq_len += past_key_value[0].shape[-2] + (self.image_token_num if LOW_BITS else 0)
    cos, sin = self.rotary_emb(v, seq_len=kv_seq_len)
    q, k = apply_rotary_pos_emb(q, k, cos, sin, position_ids)

    # ---- decode step -------------------------------------------------------------------------
    self._text_cache.append(k, v)
    k_fp, v_fp = self._text_cache.views()
    past_key_value = (k_fp, v_fp) if use_cache else None
    if attention_mask is not None and attention_mask.size() != (bsz, 1, q_len, kv_seq_len):
        raise ValueError(f"Attention mask should be of size {(bsz, 1, q_len, kv_seq_len)}, "
                         f"but is {attention_mask.size()}")
    t_sys = self.sprompt_len if LOW_BITS else 0
    if getattr(self, "_u8_state", None) is not None:
        from . import calibquant as _cq
        attn = _cq.decode_attention(q, self._u8_state, k_fp, v_fp, BITS_KV, t_sys, normalize=self.normalize,
                                    mask=attention_mask).to(q.dtype)             # bfloat16 out, as the reference
    else:
        attn = ops.decode_attention(q, self.k_pack, self.v_pack, k_fp, v_fp, t_sys, BITS_KV,
                                    group_size=GROUP_SIZE, calibrate=self.normalize and LOW_BITS,
                                    mask=attention_mask)                         # [B,Hq,1,D]
    local_heads = self.num_heads // _shard_world(self)
    if attn.size() != (bsz, local_heads, q_len, self.head_dim):
        raise ValueError(f"`attn_output` should be of size {(bsz, local_heads, q_len, self.head_dim)}, "
                         f"but is {attn.size()}")
    attn = _gather_heads(self, attn.transpose(1, 2).reshape(bsz, q_len, -1))
    attn_output = self.wo(attn.reshape(bsz, q_len, -1))
    return attn_output, None, past_key_value


def forward_internlm2_qjl(self, hidden_states: torch.Tensor,
                          attention_mask: Optional[torch.LongTensor] = None,
                          position_ids: Optional[torch.LongTensor] = None,
                          past_key_value: Optional[Tuple[torch.Tensor]] = None,
                          output_attentions: bool = False, use_cache: bool = False, **kwargs):
    """Patched forward with the reference's ``qjl`` structure (``patch_internvl.py:492-636``): the
    state travels in the 9-tuple ``(shape, kv_quant, K_sys, K_txt, V_code, V_scale, V_mn, V_sys,
    V_txt)``; values use ``triton_quantize_and_pack_along_last_dim`` + ``cuda_quantized_bmm_dynamic``
    and keys a ``QJLKeyQuantizer`` (the JL sign sketch ``config.qjl``, or per-channel group
    quantization when that is None).  No logit calibration, as in the reference's qjl forward.
    """
    self.sprompt_len = SPROMPT_LEN
    self.image_token_num = _image_token_num()
    attention_mask = _pop_padding_mask(kwargs, attention_mask)
    bsz, q_len, _ = hidden_states.size()
    cfg = self.config
    q, k, v = _split_qkv(self, hidden_states)
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    kv_seq_len = q_len + (past_key_value[0].shape[-2] if past_key_value is not None else 0)
    cos, sin = self.rotary_emb(v, seq_len=kv_seq_len)
    q, k = apply_rotary_pos_emb(q, k, cos, sin, position_ids)
    n_rep = self.num_key_value_groups

    if past_key_value is not None:
        (_, kv_quant, k_sys, k_txt, v_code, v_scale, v_mn, v_sys, v_txt) = past_key_value
        k_txt = torch.cat([k_txt, k], dim=2)
        v_txt = torch.cat([v_txt, v], dim=2)
        att_sys = q @ repeat_kv(k_sys, n_rep).transpose(2, 3)
        att_txt = q @ repeat_kv(k_txt, n_rep).transpose(2, 3)
        att = torch.cat((att_sys, kv_quant.attention_score(q), att_txt), dim=-1) / self.head_dim ** 0.5
        if attention_mask is not None:
            if attention_mask.size() != (bsz, 1, q_len, kv_seq_len):
                raise ValueError(f"Attention mask should be of size {(bsz, 1, q_len, kv_seq_len)}, "
                                 f"but is {attention_mask.size()}")
            att = torch.max(att + attention_mask, torch.tensor(torch.finfo(att.dtype).min, device=att.device))
        att = torch.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype)
        s0, s1 = self.sprompt_len, self.sprompt_len + self.image_token_num
        out = cuda_quantized_bmm_dynamic(cfg.group_size, att[:, :, :, s0:s1].contiguous(),
                                         v_code, v_scale, v_mn, cfg.v_bits)
        out = out + (att[..., s1:] @ repeat_kv(v_txt, n_rep) + att[..., :s0] @ repeat_kv(v_sys, n_rep))
        attn_output = out.transpose(1, 2)
    else:
        attn_output = ops.prefill_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        sizes = [self.sprompt_len, self.image_token_num, q_len - self.sprompt_len - self.image_token_num]
        k_sys, k_vis, k_txt = k.split(sizes, dim=-2)
        v_sys, v_vis, v_txt = v.split(sizes, dim=-2)
        sketch = getattr(cfg, "qjl", None)
        if sketch is not None and sketch.proj_dir_score.device != k.device:   # the model moved after patching
            for name in ("proj_dir", "proj_dir_score", "proj_dir_quant"):
                setattr(sketch, name, getattr(sketch, name).to(k.device))
            sketch.device = k.device
        kv_quant = QJLKeyQuantizer(sketch, cfg.outlier_count_general, cfg.buffer_size, cfg.group_size, cfg.k_bits)
        kv_quant.build_sketch(k_vis)
        if v.shape[-2] <= cfg.buffer_size:
            raise NotImplementedError("value_states.shape[-2] <= self.config.buffer_size")
        v_code, v_scale, v_mn = triton_quantize_and_pack_along_last_dim(v_vis.contiguous(), cfg.group_size,
                                                                        cfg.v_bits)
        k_sys, k_txt, v_sys, v_txt = (t.contiguous() for t in (k_sys, k_txt, v_sys, v_txt))
    past_key_value = (_dummy_class_for_accessing_shape(kv_seq_len), kv_quant, k_sys, k_txt,
                      v_code, v_scale, v_mn, v_sys, v_txt) if use_cache else None
    attn_output = self.wo(attn_output.reshape(bsz, q_len, self.hidden_size))
    return attn_output, None, past_key_value


ATTN_FORWARD_FUNCTIONS = {
    "calibquant": forward_internlm2_calibquant,
    "qjl": forward_internlm2_qjl,
}


def patch_model(model, quant_method="calibquant", **kwargs):
    """Swap the chat model's ``generate`` and the attention class's ``forward`` in place, exactly
    as ``patch_internvl.py:645-660``; the ``qjl`` settings land on ``model.config.llm_config``.
    ``kv_format="uint8"`` (with ``"calibquant"``) keeps the visual span in the reference's own byte format
    and decodes with ``calibquant.decode_attention``; the default ``"group"`` is the 32-element group format."""
    print("Patching InternVLChatModel.generate function ...")
    if hasattr(model, "extract_feature"):
        model.__class__.generate = custom_generate
    print(f"Patching InternLM2FlashAttention2.forward function ... {quant_method}")
    model.language_model.model.layers[0].attention.__class__.forward = ATTN_FORWARD_FUNCTIONS[quant_method]
    if quant_method == "calibquant":
        global KV_FORMAT
        kv_format = kwargs.get("kv_format", "group")
        if kv_format not in ("group", "uint8"):
            raise ValueError(f"kv_format must be 'group' or 'uint8', got {kv_format!r}")
        KV_FORMAT = kv_format
    if quant_method == "qjl":
        cfg = model.config.llm_config
        cfg.k_bits = kwargs.get("k_bits", 2)
        cfg.v_bits = kwargs.get("v_bits", 2)
        cfg.group_size = kwargs.get("group_size", 32)
        cfg.buffer_size = kwargs.get("buffer_size", 128)
        cfg.outlier_count_general = kwargs.get("outlier_count_general", 32)
        # key_format="qjl" (default, as the reference): Johnson-Lindenstrauss sign sketch of the keys;
        # key_format="group": the same forward with keys in the per-channel group format
        if kwargs.get("key_format", "qjl") == "qjl":
            from .qjl.qjl_utils import QJLSketch
            dev = next(model.parameters()).device
            generator = torch.Generator(device=dev).manual_seed(kwargs.get("seed", 1234))
            cfg.qjl = QJLSketch(dim=(128, cfg.k_bits * 128), dim_outlier=256, device=dev, rot=True, rng=generator)
        else:
            cfg.qjl = None
    return model
