"""Head-sharded and batch-sharded partitioning, exercised with two gloo ranks on CPU.

The local attention is the CPU oracle here (the CUDA kernels are covered by the gpu tests); what
is under test is the host logic: which heads / weight rows / batch rows a rank owns and that the
all-gather of head outputs reproduces the unsharded result exactly."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from calibquant_b200 import sharding
from oracle import generator
from oracle import group_format as gf


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_attend(q_local, state):
    return gf.decode_attention(q_local, state["k_pack"], state["v_pack"], state["k_sys"], state["k_txt"],
                               state["v_sys"], state["v_txt"], state["bits"])


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, Hkv, t_vis, bits = 2, 8, 4, 64, 1
        k, v, q = generator.make_kvq(B, Hq, Hkv, 41 + t_vis + 7, seed=3)
        k_sys, k_vis, k_txt = generator.split_spans(k, t_vis)
        v_sys, v_vis, v_txt = generator.split_spans(v, t_vis)
        sh = sharding.HeadShardedAttention(rank, world, Hq, Hkv, attend=_oracle_attend)
        hs = slice(sh.h0, sh.h1)
        state = {
            "k_pack": gf.quantize_and_pack_last_dim(k_vis[:, hs].transpose(2, 3).contiguous(), 32, bits),
            "v_pack": gf.quantize_and_pack_last_dim(v_vis[:, hs].contiguous(), 32, bits),
            "k_sys": k_sys[:, hs], "k_txt": k_txt[:, hs], "v_sys": v_sys[:, hs], "v_txt": v_txt[:, hs],
            "bits": bits,
        }
        o = sh(sh.local_q(q), state)                                    # [B, Hq, D] on every rank
        full = gf.decode_attention_from_fp(q, k, v, t_vis, bits, 41)[0].reshape(B, Hq, 128)
        assert torch.equal(o, full), "gathered head outputs differ from the unsharded result"
        # every rank must hold the same gathered tensor
        ref = o.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, o)
        # weight rows: the rank's slice of wqkv yields exactly its heads' q/k/v
        n_rep, D, hidden = Hq // Hkv, 128, 256
        g = torch.Generator().manual_seed(0)
        w = torch.randn((Hq + 2 * Hkv) * D, hidden, generator=g)
        x = torch.randn(3, hidden, generator=g)
        full_out = (x @ w.t()).view(3, Hkv, n_rep + 2, D)
        mine = (x @ sharding.shard_wqkv(w, rank, world, Hkv, n_rep, D).t()).view(3, -1, n_rep + 2, D)
        assert torch.equal(mine, full_out[:, sh.h0:sh.h1])
        # batch split covers every row once
        lo, hi = sharding.batch_range(rank, world, 5)
        rows = torch.zeros(5)
        rows[lo:hi] = 1
        dist.all_reduce(rows)
        assert torch.equal(rows, torch.ones(5))
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _tp_worker(rank, world, port, out_dir):
    """Tensor-parallel slices of one decoder layer: partial products summed over the ranks (gloo) reproduce the
    unsharded layer's linear algebra; the vocabulary-sharded arg-max picks the same token."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from calibquant_b200 import tp
        from calibquant_b200.internlm2 import InternLM2Config, InternLM2DecoderLayer, init_weights_
        cfg = InternLM2Config(hidden_size=256, num_attention_heads=8, num_key_value_heads=4, intermediate_size=384,
                              num_hidden_layers=1, vocab_size=64)
        full = InternLM2DecoderLayer(cfg).double()
        init_weights_(full, 3, std=0.1)
        mine = InternLM2DecoderLayer(cfg).double()
        mine.load_state_dict(full.state_dict())
        tp.shard_layer_(mine, rank, world)
        g = torch.Generator().manual_seed(9)
        x = torch.randn(5, 1, 256, generator=g, dtype=torch.float64)
        # feed-forward block: stacked w1/w3 slice + w2 column slice give a partial sum
        part = mine.feed_forward(x)
        dist.all_reduce(part)
        assert torch.allclose(part, full.feed_forward(x), atol=1e-12)
        # wqkv rows -> this rank's heads; wo columns of those heads -> a partial sum of the full wo product
        n_rep, D = 2, 32
        h0, h1 = sharding.kv_head_range(rank, world, 4)
        qkv_full = full.attention.wqkv(x).view(5, 1, 4, n_rep + 2, D)
        qkv_mine = mine.attention.wqkv(x).view(5, 1, -1, n_rep + 2, D)
        assert torch.equal(qkv_mine, qkv_full[:, :, h0:h1])
        o = torch.randn(5, 1, 8 * D, generator=g, dtype=torch.float64)      # stand-in for all heads' outputs
        part = mine.attention.wo(o[..., h0 * n_rep * D:h1 * n_rep * D])
        dist.all_reduce(part)
        assert torch.allclose(part, full.attention.wo(o), atol=1e-12)
        # vocabulary-sharded arg-max
        logits = torch.randn(5, 64, generator=g)
        v = 64 // world
        tok = tp.global_argmax_torch(logits[:, rank * v:(rank + 1) * v], rank, world, v)
        assert torch.equal(tok, logits.argmax(-1))
        open(os.path.join(out_dir, f"tp{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _count_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import bench
        # each rank sizes its timed region from its own probe (7 and 8 replays here); all must time the larger
        # count, or the slowest rank's total would be divided by another rank's count
        n = bench.agree_max(7 + rank, world, torch.device("cpu"))
        assert n == 8
        total_ms = torch.tensor([8 * 7.15], dtype=torch.float64)        # this rank's time for n replays of 100 steps
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
        assert abs(total_ms.item() / (100 * n) - 0.0715) < 1e-12
        assert bench.agree_max(5, 1, torch.device("cpu")) == 5          # single rank: no collective
        open(os.path.join(out_dir, f"n{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_time_the_same_number_of_replays(tmp_path):
    world = 2
    mp.spawn(_count_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"n{r}").exists() for r in range(world))


def test_two_rank_tensor_parallel_slices(tmp_path):
    world = 2
    mp.spawn(_tp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"tp{r}").exists() for r in range(world))


def test_two_rank_head_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_ranges():
    assert sharding.kv_head_range(3, 8, 8) == (3, 4)
    assert sharding.kv_head_range(1, 2, 8) == (4, 8)
    with pytest.raises(ValueError):
        sharding.kv_head_range(0, 3, 8)
    assert sharding.wqkv_rows(1, 8, 8, 4, 128) == (768, 1536)
    assert [sharding.batch_range(r, 4, 10) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.batch_range(0, 1, 16) == (0, 16)
