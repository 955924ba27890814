"""Generate the golden fixtures in this folder by EXECUTING THE REFERENCE on CPU.

Run once, in a container that has the reference checkout (it is not needed to run
the tests, only to regenerate the fixtures):

    REFERENCE_ROOT=/path/to/calibquant python tests/golden/make_golden.py

What runs:
* ``qjl.new_pack.triton_quantize_and_pack_along_last_dim`` -- its two Triton kernels
  execute under the Triton interpreter (``TRITON_INTERPRET=1``) on CPU tensors;
* ``calibquant.quant`` -- plain eager torch;
* ``calibquant.encode`` -- eager (``TORCHDYNAMO_DISABLE=1``; same arithmetic as the
  compiled form);
* ``calibquant.fused_kernel`` / ``fused_kernel_wv`` -- Triton interpreter, with the
  output device switched to CPU, the autotuner cut to its first configuration and
  the SM-count heuristic replaced by a constant (all three only select *where/how*
  the kernel runs, not what it computes).

Inputs come from ``oracle.generator`` (seeded); each fixture stores inputs and the
reference's outputs, so the tests need neither the reference nor a GPU.
"""

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ["TORCHDYNAMO_DISABLE"] = "1"

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set REFERENCE_ROOT to the reference checkout (see the docstring)")
sys.path.insert(0, REF)

import torch  # noqa: E402

from oracle import generator  # noqa: E402

import calibquant as ref_cq  # noqa: E402
from qjl.new_pack import triton_quantize_and_pack_along_last_dim as ref_pack  # noqa: E402

ref_cq.DEVICE = "cpu"
for kern in (ref_cq.tiled_encoded_group_vecmat_transp_kernel,
             ref_cq.tiled_encoded_group_vecmat_kernel):
    kern.configs = kern.configs[:1]
ref_cq.tiled_encoded_group_vecmat_kernel.fn.values["NUM_SM"] = lambda args: 8


def pack_cases():
    out = {}
    for dtype, dname in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        k, v, _ = generator.make_kvq(2, 8, 2, 96, seed=7, dtype=dtype)
        for bit in (1, 2, 4):
            v_in = v.contiguous()                               # [B,Hkv,T,D]  per token
            k_in = k.transpose(2, 3).contiguous()               # [B,Hkv,D,T]  per channel
            for name, x in (("v", v_in), ("k", k_in)):
                code, scale, mn = ref_pack(x.clone(), 32, bit)
                out[f"{name}_{dname}_b{bit}"] = {
                    "data": x, "code": code.clone(), "scale": scale.clone(), "mn": mn.clone()}
    torch.save(out, os.path.join(HERE, "new_pack.pt"))
    print("new_pack.pt:", len(out), "cases")


def calibquant_cases():
    out = {}
    for bit in (1, 2, 4):
        dpe = 8 // bit
        clip_k, clip_v = (0.5, 0.3) if bit == 1 else (1, 1)
        k, v, q = generator.make_kvq(1, 8, 2, 80, seed=11 + bit, dtype=torch.float16)
        k_btHd = k.transpose(1, 2).contiguous()                 # [B,T,Hkv,D]
        v_btHd = v.transpose(1, 2).contiguous()
        kq, sk, zk = ref_cq.quant(k_btHd, bits=bit, per_channel=True, scale=clip_k, post_scale=True)
        vq, sv, zv = ref_cq.quant(v_btHd, bits=bit, per_channel=True, scale=clip_v, post_scale=True)
        enc_k = ref_cq.encode(kq.transpose(1, 2).to(torch.int64), bits=bit, datum_per_elem=dpe)
        enc_v = ref_cq.encode(vq.transpose(1, 2).to(torch.int64), bits=bit, datum_per_elem=dpe)
        lut = torch.arange(2 ** bit, dtype=torch.float16)
        n_rep = 4
        rep = lambda t: t[:, :, None].expand(t.shape[0], t.shape[1], n_rep, *t.shape[2:]) \
            .reshape(t.shape[0], t.shape[1] * n_rep, *t.shape[2:]).contiguous()
        w_k = (q * rep(sk.transpose(1, 2))).contiguous()        # [B,Hq,1,D]
        s = ref_cq.fused_kernel(lut, w_k, rep(enc_k), BITS=bit, DATUM_PER_ELM=dpe)
        g = torch.Generator().manual_seed(5)
        w_v = torch.softmax(torch.randn(1, 8, 1, 80, generator=g) * 3, dim=-1).half().contiguous()
        o = ref_cq.fused_kernel_wv(lut, w_v, rep(enc_v), BITS=bit, DATUM_PER_ELM=dpe)
        out[f"b{bit}"] = {
            "k": k_btHd, "v": v_btHd, "q": q, "clip_k": clip_k, "clip_v": clip_v,
            "kq": kq, "sk": sk, "zk": zk, "vq": vq, "sv": sv, "zv": zv,
            "enc_k": enc_k, "enc_v": enc_v, "w_k": w_k, "scores": s.clone(),
            "w_v": w_v, "out_v": o.clone()}
    torch.save(out, os.path.join(HERE, "calibquant.pt"))
    print("calibquant.pt:", len(out), "cases")


if __name__ == "__main__":
    pack_cases()
    calibquant_cases()
