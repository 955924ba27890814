"""Worker for tests/test_gpu_multi.py (launched with torch.distributed.run, one rank per GPU):
the KV-head-sharded attention layer must reproduce the unsharded layer on every rank."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    import datetime
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    from calibquant_b200 import patch_internvl as pi
    from calibquant_b200.internlm2 import ChatModelShell, InternLM2Config, init_weights_
    cfg = InternLM2Config(hidden_size=1024, num_attention_heads=8, num_key_value_heads=4,
                          intermediate_size=512, num_hidden_layers=1, vocab_size=64)
    outs = []
    for sharded in (False, True):
        shell = ChatModelShell(cfg).half()
        init_weights_(shell, 11, std=0.05)                 # same seed on every rank
        pi.patch_model(shell, "calibquant")
        shell.cuda()
        attn = shell.language_model.model.layers[0].attention
        if sharded:
            pi.shard_attention_(attn, rank, world)
        g = torch.Generator().manual_seed(5)
        T, t_vis = 41 + 256 + 9, 256
        h = (torch.randn(2, T, 1024, generator=g) * 0.5).half().cuda()
        os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
        pos = torch.arange(T, device="cuda").unsqueeze(0).expand(2, T)
        o_pre, _, past = attn(h, position_ids=pos, use_cache=True)
        hd = (torch.randn(2, 1, 1024, generator=g) * 0.5).half().cuda()
        o_dec, _, past = attn(hd, position_ids=torch.full((2, 1), T, device="cuda"), past_key_value=past,
                              use_cache=True)
        outs.append((o_pre.float(), o_dec.float()))
    for a, b in zip(outs[0], outs[1]):
        err = float((a - b).norm() / a.norm())
        assert err <= 2e-3, f"rank {rank}: sharded layer deviates from the unsharded one: {err}"
    ref = outs[1][1].clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(ref, outs[1][1]), "ranks disagree on the gathered output"
    dist.barrier()
    tensor_parallel_decode(rank, world)
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK")
    dist.destroy_process_group()


class _NcclComm:
    """Stand-in for ``tp.PeerComm`` that sums through ``torch.distributed``: the same tensor-parallel step with a
    library collective, to tell an error of the peer-memory kernels from one of the sharding arithmetic."""

    def __init__(self, rank, world):
        self.rank, self.world, self.pending = rank, world, None

    def push(self, x):
        self.pending = x.float().clone()
        dist.all_reduce(self.pending)

    def reduce_add_rmsnorm(self, residual, weight, eps, out=None, normalize=True):
        from calibquant_b200 import ops
        residual.copy_((residual.float() + self.pending.view_as(residual)).to(residual.dtype))
        return ops.add_rmsnorm(residual, None, weight, eps) if normalize else None

    def status(self):
        return 0

    def close(self):
        pass


def tensor_parallel_decode(rank, world):
    """The tensor-parallel decode step (weights sliced by KV head, partial sums exchanged through the peers'
    buffers): its hidden state must equal, to the last bit, the same step with the sums done by NCCL, and agree
    with the unsharded model as far as a model with a 4-bit cache and random weights allows (at 1 bit the codes
    of the cache flip with the rounding of the partial sums, and layers after the first differ by tens of
    percent between any two summation orders); then greedy tokens from the replayed CUDA graph, which every
    rank must agree on."""
    from calibquant_b200 import patch_internvl as pi, tp
    from calibquant_b200.internlm2 import ChatModelShell, GraphedDecoder, InternLM2Config, init_weights_
    cfg = InternLM2Config(hidden_size=1024, num_attention_heads=8, num_key_value_heads=4,
                          intermediate_size=1536, num_hidden_layers=3, vocab_size=128)
    B, t_vis, n_new = 4, 256, 6
    T = 41 + t_vis + 9
    g = torch.Generator().manual_seed(21)
    emb = (torch.randn(B, T, cfg.hidden_size, generator=g) * 0.5).to(torch.bfloat16).cuda()
    os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
    pos = torch.arange(T, device="cuda").unsqueeze(0).expand(B, T)
    bits_before = pi.BITS_KV
    pi.BITS_KV = 4
    hid, toks = {}, None
    try:
        for mode in ("plain", "nccl", "peer"):
            shell = ChatModelShell(cfg).to(torch.bfloat16)
            init_weights_(shell, 13, std=0.05)
            pi.patch_model(shell, "calibquant")
            shell.cuda()
            lm = shell.language_model
            comm = None
            if mode != "plain":
                comm = _NcclComm(rank, world) if mode == "nccl" else \
                    tp.PeerComm(rank, world, B * cfg.hidden_size * 2, torch.device("cuda", torch.cuda.current_device()))
                tp.shard_model_(lm, rank, world, comm)
            with torch.no_grad():
                logits, past = lm.forward_step(emb, pos, None)
                first = lm.next_token(logits)
                e1 = lm.model.tok_embeddings(first).unsqueeze(1)
                p1 = torch.full((B, 1), T, device="cuda", dtype=torch.long)
                hid[mode] = lm.decode_hidden_fused(e1, p1, past).float().clone()      # one eager decode step
                if mode == "peer":
                    second = tp.global_argmax_peer(lm.output(hid[mode].to(torch.bfloat16)[:, -1]), comm, cfg.vocab_size // world)
                    dec = GraphedDecoder(lm, past, second, T + 1, n_new)
                    toks = dec.run(n_new).contiguous().clone()
                    dec.close()
                    assert comm.status() == 0, f"rank {rank}: a wait for a peer timed out"
            if comm is not None:
                dist.barrier()
                comm.close()
    finally:
        pi.BITS_KV = bits_before
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert torch.equal(hid["peer"], hid["nccl"]), f"rank {rank}: peer-memory sums differ from NCCL sums: {rel(hid['peer'], hid['nccl'])}"
    assert rel(hid["peer"], hid["plain"]) <= 0.1, f"rank {rank}: tensor-parallel step vs unsharded: {rel(hid['peer'], hid['plain'])}"
    ref = toks.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(ref, toks), "ranks disagree on the generated tokens"
    if rank == 0:
        print(f"tensor-parallel decode: peer == nccl sums, vs unsharded {rel(hid['peer'], hid['plain']):.4f}")


if __name__ == "__main__":
    main()
