"""HF-free InternLM2 backbone (the language model of InternVL2.5) for running the patched
attention forward without downloading anything.

Only what the quantized-KV attention path touches is modelled faithfully: the fused ``wqkv``
projection with its per-KV-head ``(n_rep q heads, k, v)`` output layout, rotary embeddings with
``rotary_emb(x, seq_len) -> (cos, sin)``, the attribute names the patched forward reads
(``num_heads, num_key_value_groups, head_dim, hidden_size, wo, is_causal, config``) and the
decoder-layer call signature.  Everything around it (RMSNorm, SwiGLU, embeddings, greedy loop) is
plain PyTorch: the reference leaves those to the third-party model code as well.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
from torch import nn


@dataclass
class InternLM2Config:
    hidden_size: int = 4096
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    vocab_size: int = 92544
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-5
    max_position_embeddings: int = 32768

    @property
    def head_dim(self):
        return self.hidden_size // self.num_attention_heads


INTERNLM2_5_7B = InternLM2Config()
INTERNLM2_20B = InternLM2Config(hidden_size=6144, num_attention_heads=48, num_key_value_heads=8,
                                intermediate_size=16384, num_hidden_layers=48)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * v.to(x.dtype)


class RotaryEmbedding(nn.Module):
    """cos/sin tables [seq_len, head_dim] in the dtype of ``x`` (non-interleaved halves)."""

    def __init__(self, dim, base):
        super().__init__()
        self.dim, self.base = dim, base
        self._cache = {}

    def forward(self, x, seq_len):
        key = (x.device, x.dtype)
        cached = self._cache.get(key)
        if cached is None or cached[0].shape[0] < seq_len:
            n = max(seq_len, 4096)
            inv = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, device=x.device, dtype=torch.float32) / self.dim))
            t = torch.arange(n, device=x.device, dtype=torch.float32)
            emb = torch.cat([torch.outer(t, inv)] * 2, dim=-1)
            cached = (emb.cos().to(x.dtype), emb.sin().to(x.dtype))
            self._cache[key] = cached
        return cached[0][:seq_len], cached[1][:seq_len]


class InternLM2Attention(nn.Module):
    def __init__(self, config: InternLM2Config):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = config.head_dim
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.is_causal = True
        self.wqkv = nn.Linear(self.hidden_size, (self.num_heads + 2 * self.num_key_value_heads) * self.head_dim,
                              bias=False)
        self.wo = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=False)
        self.rotary_emb = RotaryEmbedding(self.head_dim, config.rope_theta)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, **kwargs):
        raise RuntimeError("InternLM2Attention.forward is provided by calibquant_b200.patch_internvl.patch_model")


class InternLM2MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.w1 = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.w3 = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.w2 = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        if self.w1 is None:      # tensor-parallel shard: w1 / w3 slices stacked in `w13` (calibquant_b200.tp)
            gu = self.w13(x)
            n = gu.shape[-1] // 2
            return self.w2(nn.functional.silu(gu[..., :n]) * gu[..., n:])
        return self.w2(nn.functional.silu(self.w1(x)) * self.w3(x))


class InternLM2DecoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = InternLM2Attention(config)
        self.feed_forward = InternLM2MLP(config)
        self.attention_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.ffn_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                use_cache=True):
        h, _, present = self.attention(self.attention_norm(hidden_states), attention_mask=attention_mask,
                                       position_ids=position_ids, past_key_value=past_key_value,
                                       output_attentions=False, use_cache=use_cache)
        tp = getattr(self.attention, "_shard_rowparallel", False)     # partial sums: add up over the ranks
        if tp:
            torch.distributed.all_reduce(h, group=self.attention._shard[2])
        hidden_states = hidden_states + h
        f = self.feed_forward(self.ffn_norm(hidden_states))
        if tp:
            torch.distributed.all_reduce(f, group=self.attention._shard[2])
        hidden_states = hidden_states + f
        return hidden_states, present


class InternLM2Model(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.tok_embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([InternLM2DecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)


class InternLM2ForCausalLM(nn.Module):
    """``language_model`` of the chat model: ``.model.layers[i].attention`` as in HF."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = InternLM2Model(config)
        self.output = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

    def get_input_embeddings(self):
        return self.model.tok_embeddings

    @torch.no_grad()
    def forward_step(self, inputs_embeds, position_ids, past_key_values):
        h = inputs_embeds
        presents = []
        for i, layer in enumerate(self.model.layers):
            h, present = layer(h, position_ids=position_ids,
                               past_key_value=None if past_key_values is None else past_key_values[i])
            presents.append(present)
        h = self.model.norm(h[:, -1:])
        return self.output(h), presents

    def next_token(self, logits):
        """Greedy token from the last position's logits (vocabulary-sharded under tensor parallelism)."""
        tp = getattr(self, "_tp", None)
        if tp is None:
            return logits[:, -1].argmax(-1)
        from . import tp as _tp
        rank, world, _, group, v_per = tp
        return _tp.global_argmax_torch(logits[:, -1], rank, world, v_per, group)

    @torch.no_grad()
    def decode_token_fused(self, inputs_embeds, position_ids, past_key_values):
        """One fused decode step; returns the next token [B].  Under tensor parallelism every sum over the
        ranks rides on the step's own launches: the partial rows are pushed into the peers' buffers and the
        next layer norm adds them up (``calibquant_b200.tp``)."""
        tp = getattr(self, "_tp", None)
        if tp is None:
            return self.forward_step_fused(inputs_embeds, position_ids, past_key_values)[:, -1].argmax(-1)
        from . import tp as _tp
        x = self.decode_hidden_fused_tp(inputs_embeds, position_ids, past_key_values)
        return _tp.global_argmax_peer(self.output(x[:, -1]), tp[2], tp[4])

    @torch.no_grad()
    def decode_hidden_fused_tp(self, inputs_embeds, position_ids, past_key_values):
        """The tensor-parallel decode step up to the final norm: [B, 1, hidden], identical on every rank."""
        from . import ops
        rank, world, comm, _, v_per = self._tp
        eps = self.config.rms_norm_eps
        h = inputs_embeds.contiguous().clone()
        fused = h.shape[0] * h.shape[1] <= 64 and hasattr(comm, "allreduce_add_rmsnorm")   # one launch per collective

        def reduce(partial, weight):
            if fused:
                return comm.allreduce_add_rmsnorm(partial, h, weight, eps)
            comm.push(partial)
            return comm.reduce_add_rmsnorm(h, weight, eps)

        pending = None
        for i, layer in enumerate(self.model.layers):
            x = ops.add_rmsnorm(h, None, layer.attention_norm.weight, eps) if pending is None else \
                reduce(pending, layer.attention_norm.weight)
            a, _, _ = layer.attention(x, position_ids=position_ids, past_key_value=past_key_values[i],
                                      output_attentions=False, use_cache=True)
            x = reduce(a, layer.ffn_norm.weight)
            ff = layer.feed_forward
            pending = ff.w2(ops.swiglu_packed(ff.w13(x)))
        return reduce(pending, self.model.norm.weight)

    @torch.no_grad()
    def decode_hidden_fused(self, inputs_embeds, position_ids, past_key_values):
        """Decode step (one token per row) up to the final norm, with the elementwise blocks of every layer
        fused: residual add + RMSNorm in one launch, SwiGLU gate in one launch.  Same arithmetic and rounding
        points as ``forward_step``; the attention modules are called as usual.  Returns [B, 1, hidden]."""
        if getattr(self, "_tp", None) is not None:
            return self.decode_hidden_fused_tp(inputs_embeds, position_ids, past_key_values)
        from . import ops
        eps = self.config.rms_norm_eps
        h = inputs_embeds.contiguous().clone()      # running residual stream, updated in place
        delta = None
        for i, layer in enumerate(self.model.layers):
            x = ops.add_rmsnorm(h, delta, layer.attention_norm.weight, eps)
            a, _, _ = layer.attention(x, position_ids=position_ids, past_key_value=past_key_values[i],
                                      output_attentions=False, use_cache=True)
            x = ops.add_rmsnorm(h, a.contiguous(), layer.ffn_norm.weight, eps)
            ff = layer.feed_forward
            delta = ff.w2(ops.swiglu(ff.w1(x), ff.w3(x)))
        return ops.add_rmsnorm(h, delta, self.model.norm.weight, eps)

    @torch.no_grad()
    def forward_step_fused(self, inputs_embeds, position_ids, past_key_values):
        """Logits [B, 1, vocab] of one fused decode step (see ``decode_hidden_fused``)."""
        return self.output(self.decode_hidden_fused(inputs_embeds, position_ids, past_key_values)[:, -1:])

    @torch.no_grad()
    def generate(self, inputs_embeds, max_new_tokens, **_):
        """Greedy decoding from embeddings: one prefill pass, then one token per step."""
        B, T, _ = inputs_embeds.shape
        pos = torch.arange(T, device=inputs_embeds.device).unsqueeze(0).expand(B, T)
        logits, past = self.forward_step(inputs_embeds, pos, None)
        tokens = []
        for step in range(max_new_tokens):
            nxt = self.next_token(logits)
            tokens.append(nxt)
            if step == max_new_tokens - 1:
                break
            emb = self.model.tok_embeddings(nxt).unsqueeze(1)
            pos = torch.full((B, 1), T + step, device=emb.device, dtype=torch.long)
            logits, past = self.forward_step(emb, pos, past)
        return torch.stack(tokens, dim=1)


class GraphedDecoder:
    """Greedy decoding with the whole step (embedding, all layers, logits, argmax, cache append,
    position and length counters) captured once in a CUDA graph and replayed per token.  Everything
    that changes from step to step lives on the device: the token, the position, and each layer's
    text-cache length, which the attention kernels read through ``t_fp_dev``."""

    def __init__(self, lm: "InternLM2ForCausalLM", past, first_token, start_pos: int, max_new_tokens: int,
                 fused: bool = True):
        self.lm, self.past, self.fused = lm, past, fused
        B = first_token.shape[0]
        dev = first_token.device
        self.caches = [layer.attention._text_cache for layer in lm.model.layers]
        self.len_dev = torch.tensor([self.caches[0].length], dtype=torch.int32, device=dev)
        for layer, tc in zip(lm.model.layers, self.caches):
            assert tc.length == self.caches[0].length
            tc.enable_static(tc.length + max_new_tokens + 2, self.len_dev)
            layer.attention._static_decode = True
            layer.attention._static_rope_len = start_pos + max_new_tokens + 2
        self.tok = first_token.clone()
        self.pos = torch.full((B, 1), start_pos, device=dev, dtype=torch.long)
        self.out = torch.zeros((max_new_tokens + 2, B), device=dev, dtype=torch.long)
        self.step_idx = torch.zeros(1, device=dev, dtype=torch.long)
        state0 = (self.tok.clone(), self.caches[0].length)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                       # warm-up outside capture, then roll back
            for _ in range(2):
                self._step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._reset(state0, start_pos)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):     # the warm-up's stream: its scratch buffers are reused
            self._step()
        self._reset(state0, start_pos)

    def _reset(self, state0, start_pos):
        self.tok.copy_(state0[0])
        self.pos.fill_(start_pos)
        self.step_idx.zero_()
        self.len_dev.fill_(state0[1])

    @torch.no_grad()
    def _step(self):
        emb = self.lm.model.tok_embeddings(self.tok).unsqueeze(1)
        self.len_dev += 1                 # the caches now count the token this step appends
        if self.fused:
            nxt = self.lm.decode_token_fused(emb, self.pos, self.past)
        else:
            nxt = self.lm.next_token(self.lm.forward_step(emb, self.pos, self.past)[0])
        self.tok.copy_(nxt)
        self.out.index_copy_(0, self.step_idx, self.tok.unsqueeze(0))
        self.pos += 1
        self.step_idx += 1

    def run(self, n_steps: int):
        """Replay ``n_steps`` decode steps; returns the generated tokens [B, n_steps]."""
        done = getattr(self, "_steps_done", 0)
        if done + n_steps > self.out.shape[0]:
            raise ValueError(f"the decoder holds room for {self.out.shape[0]} steps, {done} are done, "
                             f"{n_steps} more requested")
        for _ in range(n_steps):
            self.graph.replay()
        self._steps_done = done + n_steps
        return self.out[done:done + n_steps].t()

    def close(self):
        for layer, tc in zip(self.lm.model.layers, self.caches):
            layer.attention._static_decode = False
            tc.length = int(self.len_dev.item())


class ChatModelShell(nn.Module):
    """Minimal stand-in for InternVLChatModel: holds ``language_model`` and ``config.llm_config``
    so that ``patch_model`` can be applied exactly as to the real model."""

    def __init__(self, config: InternLM2Config):
        super().__init__()
        self.language_model = InternLM2ForCausalLM(config)
        self.config = type("Cfg", (), {})()
        self.config.llm_config = self.language_model.model.layers[0].attention.config
        self.img_context_token_id = None

    def generate(self, inputs_embeds, image_token_num, max_new_tokens):
        os.environ["IMAGE_TOKEN_NUM"] = str(int(image_token_num))
        return self.language_model.generate(inputs_embeds, max_new_tokens)


def init_weights_(module: nn.Module, seed: int, std: float = 0.02):
    """Seeded N(0, std) init of every matrix (norm weights stay 1), as the synthetic benchmarks use."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            if p.dim() >= 2:
                p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * std).to(p.dtype))
