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
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
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
    if rank == 0:
        print("MULTI_GPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
