"""Patched attention forward (prefill + decode steps) on the GPU vs the CPU oracle of the same
layer, and the model-patching entry points.

Tolerance: rel-L2 <= 2e-2 on the layer output.  On top of the attention tolerance (1e-2) the two
sides run their projections through different fp16 GEMMs, so a few K/V elements that sit exactly on
a quantization threshold can take the neighbouring code."""

import os

import pytest
import torch

from oracle.forward import AttentionOracle
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _layer(hq, hkv, seed, dtype=torch.float16):
    from calibquant_b200.internlm2 import ChatModelShell, InternLM2Config, init_weights_
    cfg = InternLM2Config(hidden_size=hq * 128, num_attention_heads=hq, num_key_value_heads=hkv,
                          intermediate_size=256, num_hidden_layers=1, vocab_size=64)
    shell = ChatModelShell(cfg).to(dtype)
    init_weights_(shell, seed, std=0.05)
    return shell


@pytest.mark.parametrize("kv_format", ["group", "uint8"])
@pytest.mark.parametrize("bits", [1, 2, 4])
def test_calibquant_forward_matches_oracle(bits, kv_format):
    from calibquant_b200 import patch_internvl as pi
    shell = _layer(8, 2, seed=bits)
    pi.patch_model(shell, "calibquant", kv_format=kv_format)
    assert pi.KV_FORMAT == kv_format
    pi.BITS_KV = bits
    pi.SCALE_K, pi.SCALE_V = (0.5, 0.3) if bits == 1 else (1, 1)      # as the reference derives them from BITS_KV
    try:
        attn_cpu = shell.language_model.model.layers[0].attention
        oracle = AttentionOracle(attn_cpu.wqkv.weight.detach().clone(), attn_cpu.wo.weight.detach().clone(),
                                 8, 2, bits=bits, kv_format=kv_format)
        shell.cuda()
        attn = shell.language_model.model.layers[0].attention
        t_vis, t_txt, B = 256, 13, 2
        T = 41 + t_vis + t_txt
        g = torch.Generator().manual_seed(17)
        h = (torch.randn(B, T, 1024, generator=g) * 0.5).half()
        os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
        pos = torch.arange(T).unsqueeze(0).expand(B, T)
        out, w, past = attn(h.cuda(), position_ids=pos.cuda(), use_cache=True)
        ref = oracle.prefill(h, t_vis)
        assert w is None and past[0].shape == (B, 2, 41 + t_txt, 128)
        assert rel_l2(out, ref) <= TOL, rel_l2(out, ref)
        for step in range(3):
            hd = (torch.randn(B, 1, 1024, generator=g) * 0.5).half()
            pos = torch.full((B, 1), T + step, dtype=torch.long)
            out, _, past = attn(hd.cuda(), position_ids=pos.cuda(), past_key_value=past, use_cache=True)
            ref = oracle.decode(hd)
            assert past[0].shape[2] == 41 + t_txt + step + 1
            assert rel_l2(out, ref) <= TOL, (step, rel_l2(out, ref))
    finally:
        pi.BITS_KV = 1
        pi.SCALE_K, pi.SCALE_V = 0.5, 0.3
        pi.KV_FORMAT = "group"


def test_qjl_forward_structure_and_scores():
    """The qjl-keyed forward keeps the reference's 9-tuple state and, with no calibration, must
    agree with the oracle of the same arithmetic (2-bit keys and values, group 32)."""
    from calibquant_b200 import patch_internvl as pi
    shell = _layer(8, 2, seed=5)
    pi.patch_model(shell, "qjl", k_bits=2, v_bits=2, buffer_size=128, key_format="group")
    attn_cpu = shell.language_model.model.layers[0].attention
    oracle = AttentionOracle(attn_cpu.wqkv.weight.detach().clone(), attn_cpu.wo.weight.detach().clone(),
                             8, 2, bits=2, calibrate=False)
    shell.cuda()
    attn = shell.language_model.model.layers[0].attention
    t_vis, t_txt, B = 256, 9, 1
    T = 41 + t_vis + t_txt
    g = torch.Generator().manual_seed(3)
    h = (torch.randn(B, T, 1024, generator=g) * 0.5).half()
    os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
    pos = torch.arange(T).unsqueeze(0).expand(B, T)
    out, _, past = attn(h.cuda(), position_ids=pos.cuda(), use_cache=True)
    assert len(past) == 9 and past[0].shape[2] == T
    assert rel_l2(out, oracle.prefill(h, t_vis)) <= TOL
    hd = (torch.randn(B, 1, 1024, generator=g) * 0.5).half()
    out, _, past = attn(hd.cuda(), position_ids=torch.full((B, 1), T).cuda(), past_key_value=past, use_cache=True)
    assert past[0].shape[2] == T + 1 and past[3].shape[2] == t_txt + 1
    assert rel_l2(out, oracle.decode(hd)) <= TOL
    pi.patch_model(shell, "calibquant")


def test_key_quantizer_object_streaming():
    """build_sketch / update_sketch / attention_score: residual buffer flushes every buffer_size keys."""
    from calibquant_b200.qjl.qjl_utils import QJLKeyQuantizer
    from oracle import group_format as gf
    g = torch.Generator().manual_seed(1)
    k = torch.randn(1, 2, 300, 128, generator=g).half()
    q = torch.randn(1, 8, 1, 128, generator=g).half()
    kq = QJLKeyQuantizer(None, 32, 128, 32, 2)
    kq.build_sketch(k.cuda())
    assert kq.seq_len == 300 and kq.key_residual.shape[2] == 300 % 128 and len(kq.blocks) == 1
    s = kq.attention_score(q.cuda())
    assert s.shape == (1, 8, 1, 300)
    pack = gf.quantize_and_pack_last_dim(k[:, :, :256].transpose(2, 3).contiguous(), 32, 2)
    ref_q = gf.qbmm(32, q, *[gf.repeat_kv(t, 4) for t in pack], 2)
    ref_r = torch.matmul(q, gf.repeat_kv(k[:, :, 256:], 4).transpose(2, 3))
    assert rel_l2(s.cpu(), torch.cat([ref_q, ref_r], -1)) <= 2e-3
    for i in range(128 - 44):
        kq.update_sketch(torch.randn(1, 2, 1, 128, generator=g).half().cuda())
    assert kq.key_residual is None and len(kq.blocks) == 2 and kq.seq_len == 384
    assert kq.attention_score(q.cuda()).shape == (1, 8, 1, 384)


def test_tiny_model_generates_and_is_deterministic():
    """Two-layer backbone through ChatModelShell.generate: prefill + greedy steps run end to end."""
    from calibquant_b200 import patch_internvl as pi
    from calibquant_b200.internlm2 import ChatModelShell, InternLM2Config, init_weights_
    cfg = InternLM2Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=1,
                          intermediate_size=1024, num_hidden_layers=2, vocab_size=128)
    shell = ChatModelShell(cfg).half()
    init_weights_(shell, 7, std=0.05)
    pi.patch_model(shell, "calibquant")
    shell.cuda()
    g = torch.Generator().manual_seed(2)
    emb = (torch.randn(2, 41 + 64 + 10, 512, generator=g) * 0.3).half().cuda()
    a = shell.generate(emb, image_token_num=64, max_new_tokens=5)
    b = shell.generate(emb, image_token_num=64, max_new_tokens=5)
    assert a.shape == (2, 5) and torch.equal(a, b)


@pytest.mark.parametrize("kv_format", ["group", "uint8"])
def test_graph_replayed_decode_matches_eager(kv_format):
    """The decode step captured in a CUDA graph (device-side token, position and cache-length
    counters) must generate exactly the tokens of the eager loop, in both formats of the visual span."""
    from calibquant_b200 import patch_internvl as pi
    from calibquant_b200.internlm2 import ChatModelShell, GraphedDecoder, InternLM2Config, init_weights_
    cfg = InternLM2Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=1,
                          intermediate_size=1024, num_hidden_layers=2, vocab_size=128)
    shell = ChatModelShell(cfg).half()
    init_weights_(shell, 7, std=0.05)
    pi.patch_model(shell, "calibquant", kv_format=kv_format)
    shell.cuda()
    lm = shell.language_model
    g = torch.Generator().manual_seed(2)
    T, t_vis, n_new = 41 + 256 + 10, 256, 6
    emb = (torch.randn(2, T, 512, generator=g) * 0.3).half().cuda()
    eager = shell.generate(emb, image_token_num=t_vis, max_new_tokens=n_new)
    os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
    pos = torch.arange(T, device="cuda").unsqueeze(0).expand(2, T)
    with torch.no_grad():
        logits, past = lm.forward_step(emb, pos, None)
    first = logits[:, -1].argmax(-1)
    dec = GraphedDecoder(lm, past, first, T, n_new)
    toks = dec.run(n_new - 1)
    dec.close()
    pi.KV_FORMAT = "group"
    assert torch.equal(first, eager[:, 0])
    assert torch.equal(toks, eager[:, 1:])
