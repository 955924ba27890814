#!/usr/bin/env python
"""Headline benchmark: 1-bit decode attention over a group-format quantized KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--bits 1] [--context 32768] [--batch 8]

A *step* is one decode-attention pass (all batch rows, all 32 query / 8 KV heads) over one
resident quantized cache.  The workload is the reference configuration "quantize+pack sweep"
at its largest point: batch 8, 8 KV heads, head_dim 128, context 32768, whole context
quantized, fp16.  Several caches are kept resident and visited round-robin so that every step
reads its cache from HBM, not from L2 (each cache alone exceeds the 126 MB L2).

value   = algorithmic bytes per step / device time per step  (GB/s, inputs resident in HBM)
e2e     = same metric through the public Python API (the host-buffer entry point of the C ABI) with
          the step's query coming from pinned host memory and the output going back to pinned host
          memory inside the timed region, one blocking call per step
roofline= achieved GB/s of the decode call against the measured HBM copy peak
cpu_baseline = the CPU oracle (a PyTorch port of the reference arithmetic) on a bounded
          sample of the same workload, on this host's cores

N > 1 (torchrun): batch-sharded replicas, no collective on the data path; every rank holds
its own batch of 8 rows (weak scaling); value aggregates all ranks over the max rank time.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D = 32, 8, 128
GROUP = 32
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/: (kernel, bits, context, batch) -> (bytes, the kernel instantiation that was captured, summary file).
# The figure is reported only while the library still builds that instantiation for the workload.
NCU_TRAFFIC = {
    ("attn_v", 1, 32768, 8): (87126272, "k2_attn_v<__half,1,512>", "profiles/decode_attn_1bit_b8_ctx32768.md"),
    ("scores", 1, 32768, 8): (70148352, "k1_scores<__half,1,true>", "profiles/decode_attn_1bit_b8_ctx32768.md"),
}
KERNEL_NAMES = {"scores": "k1_scores", "attn_v": "k2_attn_v"}
MIN_TIMED_MS = 50.0      # the device-timed region lasts at least this long, whatever --steps says


def workload_name(batch, t_vis, t_fp, bits):
    return (f"decode attention, batch {batch} per GPU, {HQ}q/{HKV}kv heads, head_dim {D}, "
            f"context {t_vis} quantized at {bits} bit (group 32) + {t_fp} fp16 tokens")


def algorithmic_bytes(batch, t_vis, t_fp, bits):
    """Bytes one step must move: K and V codes + scale + min once per KV head (GQA reuse),
    fp16 K/V of full-precision tokens, q in and o out."""
    per_vis_tok = 2 * (D * bits // 8 + (D // GROUP) * 4)        # 64 / 96 / 160 B
    kv = batch * HKV * (t_vis * per_vis_tok + t_fp * D * 2 * 2)
    qo = batch * HQ * D * 2 * 2
    return kv + qo


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def agree_max(n, world, device):
    """The same iteration count on every rank: the largest any rank asked for.  Each rank sizes its timed
    region from a probe of its own; the job's time is the slowest rank's total, and it is divided by this count."""
    if world == 1:
        return int(n)
    t = torch.tensor([int(n)], device=device, dtype=torch.int64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return int(t.item())


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, device_index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                uuid = torch.cuda.get_device_properties(device_index).uuid
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _reason_names(self, bits):
        nv = self.nv
        table = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        return {n for n, b in table.items() if bits & b}

    def _sample(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        try:
            bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            self.reasons |= self._reason_names(bits)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            try:
                self._sample()
            except Exception:
                break
            self._stop.wait(0.002)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if not self.nv:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable"}
        self._stop.set()
        self._thread.join()
        if not self.samples:
            self._sample()
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def time_pack(batch, t_vis, bits, device, reps=5):
    """Quantize+pack throughput (K per channel with the transpose fused, V per token) on fp16 tensors
    of the workload's shape; two source tensors alternate so that each pass streams from HBM."""
    from calibquant_b200 import ops
    g = torch.Generator(device=device).manual_seed(7)
    src = [torch.randn(batch, HKV, t_vis, D, generator=g, device=device).half() for _ in range(2)]
    n = batch * HKV * t_vis * D
    nbytes = n * (2 + bits / 8 + 4 / GROUP)
    out = {}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, fn in (("k_per_channel", ops.pack_k_per_channel), ("v_per_token", ops.pack_last_dim)):
        for i in range(2):
            fn(src[i % 2], GROUP, bits)
        torch.cuda.synchronize()
        ev0.record()
        for i in range(reps):
            fn(src[i % 2], GROUP, bits)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / reps
        out[name] = {"ms": round(ms, 4), "GBps": round(nbytes / ms / 1e6, 1)}
    out["bytes_per_element"] = 2 + bits / 8 + 4 / GROUP
    return out


def build_caches(batch, t_vis, t_fp, bits, n_caches, device, seed):
    """Synthetic caches with the reference generator's value distribution (K ~ N(0,1) times a
    per-channel lognormal factor, V ~ N(0,1)), generated and packed on the device."""
    from calibquant_b200 import ops
    g = torch.Generator(device=device).manual_seed(seed)
    caches = []
    for _ in range(n_caches):
        f = torch.exp(torch.randn(D, generator=g, device=device))
        k = (torch.randn(batch, HKV, t_vis, D, generator=g, device=device) * f).half()
        kp = ops.pack_k_per_channel(k, GROUP, bits)
        del k
        v = torch.randn(batch, HKV, t_vis, D, generator=g, device=device).half()
        vp = ops.pack_last_dim(v, GROUP, bits)
        del v
        if t_fp:
            kf = torch.randn(batch, HKV, t_fp, D, generator=g, device=device).half()
            vf = torch.randn(batch, HKV, t_fp, D, generator=g, device=device).half()
        else:
            kf = vf = None
        caches.append((kp, vp, kf, vf))
    return caches


def oracle_row(t_vis, t_fp, bits, seed=5):
    """One batch row of the workload rebuilt on the CPU from its own seed, with its oracle output."""
    from oracle import generator
    from oracle import group_format as gf
    sys_len = min(41, t_fp)
    k, v, q = generator.make_kvq(1, HQ, HKV, t_vis + t_fp, seed=generator.row_seed(seed, 0))
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
    kp = gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), GROUP, bits)
    vp = gf.quantize_and_pack_last_dim(v_vis.contiguous(), GROUP, bits)
    o = gf.decode_attention(q, kp, vp, k_sys, k_txt, v_sys, v_txt, bits)
    return q, kp, vp, torch.cat([k_sys, k_txt], 2), torch.cat([v_sys, v_txt], 2), o


def run_ours(args, rank, world, device):
    from calibquant_b200 import ops
    t_vis, t_fp, bits, batch = args.context, args.fp_tokens, args.bits, args.batch
    step_bytes = algorithmic_bytes(batch, t_vis, t_fp, bits)
    n_caches = max(3, -(-3 * L2_BYTES // step_bytes))
    n_caches = min(n_caches, 64)
    caches = build_caches(batch, t_vis, t_fp, bits, n_caches, device, seed=1234 + rank)
    g = torch.Generator(device=device).manual_seed(99 + rank)
    q_dev = torch.randn(batch, HQ, 1, D, generator=g, device=device).half()
    out = torch.empty(batch, HQ, D, dtype=torch.float16, device=device)
    t_sys = min(41, t_fp)

    # ---- parity before timing: row 0 of cache 0 is replaced by a row rebuilt on the CPU from its seed;
    # the whole batch runs on the GPU and that row is compared with the CPU oracle
    parity = None
    if rank == 0 and not args.no_parity:
        q0, kp0, vp0, kf0, vf0, o_ref = oracle_row(t_vis, t_fp, bits)
        kp, vp, kf, vf = caches[0]
        for dst, src in zip(kp + vp, kp0 + vp0):
            dst[0:1].copy_(src.to(device))
        if t_fp:
            kf[0:1].copy_(kf0.to(device)); vf[0:1].copy_(vf0.to(device))
        q_par = q_dev.clone()
        q_par[0:1].copy_(q0.to(device))
        o = ops.decode_attention(q_par, kp, vp, kf, vf, t_sys, bits).float().cpu()
        err = float((o[0].reshape(HQ, D).double() - o_ref[0, :, 0].double()).norm() / o_ref.double().norm())
        parity = {"rel_l2": round(err, 6), "rows": 1, "tolerance": 1e-2, "ok": bool(err <= 1e-2),
                  "against": "oracle.group_format.decode_attention on a seeded row of this workload, whole batch on the GPU"}
        if not parity["ok"]:
            raise RuntimeError(f"decode attention differs from the CPU oracle: rel-L2 {err}")

    def step(i, q):
        kp, vp, kf, vf = caches[i % n_caches]
        return ops.decode_attention(q, kp, vp, kf, vf, t_sys, bits, out=out)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i, q_dev)

    # The K timed steps are one CUDA graph (caches visited round-robin), so that the device-side number does
    # not depend on how fast the host can issue ~40 us Python calls; the graph is replayed until the timed
    # region is at least MIN_TIMED_MS long, each replay bracketed by its own pair of events.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            step(i, q_dev)
    ev_a, ev_b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph.replay()
    torch.cuda.synchronize()
    ev_a.record(); graph.replay(); ev_b.record(); torch.cuda.synchronize()
    n_replays = max(1, int(-(-MIN_TIMED_MS // max(ev_a.elapsed_time(ev_b), 1e-3))))
    n_replays = min(n_replays, 2000)
    n_replays = agree_max(n_replays, world, device)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_replays + 1)]
    sampler = ClockSampler(device.index)
    barrier()
    sampler.start()
    marks[0].record()
    for r in range(n_replays):
        graph.replay()
        marks[r + 1].record()
    barrier()
    clocks = sampler.stop()
    ms = marks[0].elapsed_time(marks[-1])
    per_replay = sorted(marks[r].elapsed_time(marks[r + 1]) / args.steps for r in range(n_replays))
    del graph
    # ---- the launches of one step timed one by one (events between the launches, same stream, same
    # rotation of caches), averaged over the steps
    kernel_ms = {}
    n_prof = max(5, min(args.steps, 50))
    for i in range(n_prof):
        kp, vp, kf, vf = caches[i % n_caches]
        _, t = ops.decode_attention_profile(q_dev, kp, vp, kf, vf, t_sys, bits, out=out)
        for name, v in t.items():
            kernel_ms[name] = kernel_ms.get(name, 0.0) + v / n_prof
    # ---- end to end: query from pinned host memory, output back to host, every step ----------
    # (the host-buffer entry point: query copied in, result stored into the pinned buffer by the
    # last launch, the call returns when it is there: a decode loop needs the result each step)
    q_host = q_dev.cpu().pin_memory()
    o_host = torch.empty(batch, HQ, D, dtype=torch.float16).pin_memory()

    prepared = [ops.prepare_host_decode(q_host, kp, vp, kf, vf, t_sys, bits) for kp, vp, kf, vf in caches]

    def step_host(i):
        return prepared[i % n_caches](q_host, o_host)

    n_w = max(1, min(3, args.warmup))
    for i in range(n_w):
        step_host(i)
    if not torch.equal(o_host.view(torch.int16), step(n_w - 1, q_dev).view(batch, HQ, D).cpu().view(torch.int16)):
        raise RuntimeError("host-buffer decode step differs from the device-buffer one")
    n_e2e = args.steps * max(1, min(n_replays, int(-(-MIN_TIMED_MS // max(ms / n_replays, 1e-3)))))
    n_e2e = agree_max(n_e2e, world, device)
    barrier()
    ev_a.record()
    for i in range(n_e2e):
        step_host(i)
    ev_b.record()
    barrier()
    ms_e2e = ev_a.elapsed_time(ev_b)
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, ms_e2e = t.tolist()
    pack = time_pack(batch, t_vis, bits, device) if rank == 0 else None
    n_steps_timed = args.steps * n_replays
    per_step_ms = ms / n_steps_timed
    gbs = world * step_bytes / (per_step_ms * 1e-3) / 1e9
    gbs_e2e = world * step_bytes / (ms_e2e / n_e2e * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    launches_per_step = 3 + (1 if t_fp else 0)
    # per-launch algorithmic bytes: K side (codes + scale + min) for the score launch, V side plus
    # nothing else for the attn.V launch; the logits exchanged through the workspace are not counted
    side_bytes = batch * HKV * t_vis * (D * bits // 8 + (D // GROUP) * 4)
    dom = max(("scores", "attn_v"), key=lambda k: kernel_ms[k])
    dom_gbs = side_bytes / (kernel_ms[dom] * 1e-3) / 1e9
    traffic, traffic_source = None, None
    entry = NCU_TRAFFIC.get((dom, bits, t_vis, batch))
    if entry and entry[0] is not None:
        traffic, traffic_source = entry[0], {"kernel": entry[1], "summary": entry[2]}
    line = {
        "metric": f"decode_attn_{bits}bit_GBps", "value": round(gbs, 2), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(per_step_ms, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {
            "workload": workload_name(batch, t_vis, t_fp, bits),
            "batch_per_gpu": batch, "context": t_vis, "fp_tokens": t_fp, "bits": bits,
            "l2": f"{n_caches} resident caches of {step_bytes / 1e6:.1f} MB visited round-robin "
                  f"(each larger than the 126 MB L2)" if step_bytes > L2_BYTES else
                  f"{n_caches} resident caches visited round-robin (together {n_caches * step_bytes / 1e6:.0f} MB > 3x L2)",
            "parallelism": f"batch-sharded x{world}, no collective",
            "launch": f"the {args.steps} steps are one CUDA graph, replayed {n_replays} times back to back "
                      f"({ms:.1f} ms timed); e2e: one blocking host call per step, {n_e2e} calls",
            "pct_of_8TBps": round(100 * gbs / world / 8000, 2),
            "per_replay_ms_per_step": {"median": round(statistics.median(per_replay), 5),
                                       "min": round(per_replay[0], 5), "max": round(per_replay[-1], 5)},
        },
        "roofline": {"bound": "hbm", "achieved": round(dom_gbs, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(dom_gbs / peak, 4), "traffic": traffic, "traffic_source": traffic_source,
                     "peak_kind": peak_kind, "bytes_per_launch": side_bytes, "kernel": KERNEL_NAMES[dom],
                     "ms_per_launch": round(kernel_ms[dom], 5),
                     "other_kernels": {KERNEL_NAMES.get(k, k): {"ms_per_launch": round(v, 5)}
                                       for k, v in kernel_ms.items() if k != dom},
                     "step_frac": round(gbs / world / peak, 4)},
        "e2e": {"value": round(gbs_e2e, 2), "unit": "GB/s",
                "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": o_host.numel() * 2,
                "ms_per_step": round(ms_e2e / n_e2e, 5)},
        "gpu_launches": launches_per_step * n_steps_timed,
        "parity": parity,
        "pack": pack,
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args, reps=10)
    if not args.no_model:
        try:
            line["prefill"] = prefill_key(device, world)
        except Exception as e:
            line["prefill"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    # ---- the second half of the metric: end-to-end decode tok/s of the 7B-architecture backbone on these N GPUs
    if not args.no_model:
        del caches, prepared
        torch.cuda.empty_cache()
        try:
            line["model_decode"] = model_decode(rank, world, device, steps=64)
        except Exception as e:      # the attention numbers above stand on their own
            line["model_decode"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return line


def cpu_baseline(args, reps, rows=1):
    """Time the CPU oracle (PyTorch port of the reference decode step) on `rows` batch rows of
    the workload; report GB/s with the same algorithmic byte count."""
    from oracle import generator
    from oracle import group_format as gf
    torch.set_num_threads(os.cpu_count())
    t_vis, t_fp, bits = args.context, args.fp_tokens, args.bits
    T = t_vis + t_fp
    sys_len = min(41, t_fp)
    k, v, q = generator.make_kvq(rows, HQ, HKV, T, seed=0)
    k_sys, k_vis, k_txt = generator.split_spans(k, t_vis, sys_len)
    v_sys, v_vis, v_txt = generator.split_spans(v, t_vis, sys_len)
    kp = gf.quantize_and_pack_last_dim(k_vis.transpose(2, 3).contiguous(), GROUP, bits)
    vp = gf.quantize_and_pack_last_dim(v_vis.contiguous(), GROUP, bits)
    gf.decode_attention(q, kp, vp, k_sys, k_txt, v_sys, v_txt, bits)      # warm-up
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        gf.decode_attention(q, kp, vp, k_sys, k_txt, v_sys, v_txt, bits)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    gbs = algorithmic_bytes(rows, t_vis, t_fp, bits) / sec / 1e9
    return {"value": round(gbs, 4), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{rows} of {args.batch} batch rows, full context, median of {reps} passes "
                      f"({sec * 1e3:.1f} ms per pass)", "ms_per_sample": round(sec * 1e3, 2)}


def reference_gpu_decode(args, reps=5):
    """The reference's OWN CUDA path for this step, on this GPU, beside the CPU number of the reference arm: its
    extension `quantization` (qjl/csrc/quantization.cu, built unchanged into oracle/_ref/ by oracle/build_ref.py)
    called as qjl/matmul.py:4-35 calls it (three transposed copies of the packed operand per call) on operands
    expanded to the query heads as qjl/qjl_utils.py:6-11 does, with the eager calibration and softmax of
    patch_internvl.py:376-385, 413.  2 bits: the reference kernel cannot run 1-bit codes (matmul.py:24,
    quantization.cu:89).  Returns None where the extension or a GPU is missing."""
    so = os.path.join(ROOT, "oracle", "_ref", "quantization.so")
    if not (torch.cuda.is_available() and os.path.exists(so)):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("quantization", so)
    ext = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ext)
    bits, batch, t_vis = 2, args.batch, args.context
    device = torch.device("cuda", 0)
    (kp, vp, _, _), = build_caches(batch, t_vis, 0, bits, 1, device, 5)       # set-up only, outside the timed step
    q = torch.randn(batch, HQ, 1, D, device=device).half()
    n_rep = HQ // HKV

    def rep(t):                                                             # repeat_kv_quant: a materialised copy
        b, h, a, c = t.shape
        return t[:, :, None].expand(b, h, n_rep, a, c).reshape(b, h * n_rep, a, c)

    def bmm(fA, qB, scales, zeros):                                         # qjl/matmul.py:12-31
        B, nh, M, K = fA.shape
        a = fA.view(-1, M, K).contiguous()
        w = qB.reshape(-1, K, qB.shape[-1]).transpose(1, 2).contiguous()
        sc = scales.view(B * nh, scales.shape[-2], scales.shape[-1]).transpose(1, 2).contiguous()
        z = zeros.view(B * nh, zeros.shape[-2], zeros.shape[-1]).transpose(1, 2).contiguous()
        out = ext.batchedQuantizedMultiplyAccumulate_half(a, w, sc, z, bits, GROUP, nh, False)
        return out.view(B, nh, out.shape[-2], out.shape[-1])

    def step():
        s = bmm(q, rep(kp[0]), rep(kp[1]), rep(kp[2])) / math.sqrt(D)
        mx, mn = s.amax(dim=(2, 3), keepdim=True), s.amin(dim=(2, 3), keepdim=True)
        s = (s - mn) / (mx - mn + 1e-8) * ((mx + (-3)) - mn) + mn
        att = torch.softmax(s, dim=-1, dtype=torch.float32).to(q.dtype)
        return bmm(att, rep(vp[0]), rep(vp[1]), rep(vp[2]))

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(reps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / reps
    return {"what": "the reference's own CUDA kernel and wrappers for the decode step on this GPU (informational; the "
                    "reference arm's value is the CPU number)", "bits": bits, "ms_per_step": round(ms, 3),
            "GBps": round(algorithmic_bytes(batch, t_vis, 0, bits) / (ms * 1e-3) / 1e9, 2), "reps": reps}


def run_reference(args, rank, world):
    """Reference arm: the reference's decode-step arithmetic on this host's CPU cores (its CUDA
    extension and Triton kernels need a GPU toolchain that the port replaces; the CPU oracle is
    the PyTorch restatement pinned against the reference's own outputs)."""
    if rank != 0:
        return None
    rows = 1
    t0 = time.perf_counter()
    base = cpu_baseline(args, reps=max(1, min(args.steps, 5)), rows=rows)
    step_ms = base["ms_per_sample"] * args.batch / rows
    return {
        "impl": "reference", "metric": f"decode_attn_{args.bits}bit_GBps", "value": base["value"],
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(step_ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(args.batch, args.context, args.fp_tokens, args.bits),
                   "batch_per_gpu": args.batch, "context": args.context, "fp_tokens": args.fp_tokens, "bits": args.bits,
                   "sampled": f"{rows} of {args.batch} batch rows per step on the host cores (all rows would take "
                              f"{base['ms_per_sample'] * args.batch / rows / 1e3:.1f} s per step); ms_per_step "
                              "extrapolates the sampled rows to the full batch"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "reference_gpu": _safe(lambda: reference_gpu_decode(args)),
        "wall_s": round(time.perf_counter() - t0, 1),
    }


def _safe(fn):
    try:
        return fn()
    except Exception as e:
        return {"error": f"{type(e).__name__}: {e}"[:200]}


def model_decode(rank, world, device, big=False, batch=None, steps=64, bits=1, eager=False):
    """End-to-end decode throughput of an InternLM2-architecture backbone with the quantized-KV attention path:
    random-init bf16 weights, prefill of 41 system + 3328 (6656) visual + text embeddings, then greedy decode
    steps replayed from a CUDA graph.  N > 1: tensor parallel by KV head (calibquant_b200.tp): every weight
    sliced with the heads, two sums over the ranks per layer, exchanged through peer buffers over NVLink and
    added up inside the next layer-norm launch.  tok/s = batch * steps / decode time (max over ranks)."""
    from calibquant_b200 import patch_internvl as pi, tp
    from calibquant_b200.internlm2 import INTERNLM2_5_7B, INTERNLM2_20B, ChatModelShell, GraphedDecoder
    cfg = INTERNLM2_20B if big else INTERNLM2_5_7B
    batch = batch or (64 if big else 16)
    t_vis, t_txt = (6656, 128 - 41) if big else (3328, 64 - 41)
    torch.manual_seed(1234)
    with torch.device(device):
        shell = ChatModelShell(cfg).to(torch.bfloat16)
    for prm in shell.parameters():
        if prm.dim() >= 2:
            torch.nn.init.normal_(prm, std=0.02)
    pi.patch_model(shell, "calibquant")
    bits_before, pi.BITS_KV = pi.BITS_KV, bits
    lm = shell.language_model
    comm = None
    try:
        if world > 1:
            comm = tp.PeerComm(rank, world, batch * cfg.hidden_size * 2, device)
            tp.shard_model_(lm, rank, world, comm)
        T = 41 + t_vis + t_txt
        emb = torch.randn(batch, T, cfg.hidden_size, device=device, dtype=torch.bfloat16) * 0.02
        os.environ["IMAGE_TOKEN_NUM"] = str(t_vis)
        pos = torch.arange(T, device=device).unsqueeze(0).expand(batch, T)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda.synchronize()
        ev[0].record()
        with torch.no_grad():
            logits, past = lm.forward_step(emb, pos, None)
            first = lm.next_token(logits)
            ev[1].record()
            torch.cuda.synchronize()
            prefill_ms = ev[0].elapsed_time(ev[1])
            if eager:
                tok = first
                for step in range(steps):
                    e = lm.model.tok_embeddings(tok).unsqueeze(1)
                    p1 = torch.full((batch, 1), T + step, device=device, dtype=torch.long)
                    logits, past = lm.forward_step(e, p1, past)
                    tok = lm.next_token(logits)
            else:
                dec = GraphedDecoder(lm, past, first, T, steps + 3)   # capture: not timed
                dec.run(3)                                            # warm replays
                torch.cuda.synchronize()
                if world > 1:
                    torch.distributed.barrier()
                ev[1].record()
                dec.run(steps)
        ev[2].record()
        torch.cuda.synchronize()
        t = torch.tensor([ev[1].elapsed_time(ev[2])], device=device, dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        decode_ms = float(t.item())
        status = comm.status() if comm is not None else 0
        if status:
            raise RuntimeError("a wait for a peer's partial sums timed out during the decode steps")
    finally:
        pi.BITS_KV = bits_before
        if comm is not None:
            torch.distributed.barrier()
            comm.close()
    return {
        "model": f"{'InternLM2-20B' if big else 'InternLM2.5-7B'} architecture, random-init bf16",
        "tok_s": round(batch * steps / (decode_ms * 1e-3), 1), "ms_per_step": round(decode_ms / steps, 4),
        "batch": batch, "steps": steps, "prefill_tokens": T, "prefill_ms": round(prefill_ms, 1), "kv_bits": bits,
        "parallelism": "single GPU" if world == 1 else
                       f"tensor parallel by KV head x{world}: wqkv/wo/w1/w3/w2 and the cache sliced with the heads",
        "collectives_per_layer": 0 if world == 1 else 2,
        "collective": None if world == 1 else
                      "one launch per all-reduce of the [batch, hidden] partial sums: peer stores over NVLink, bounded wait "
                      "for the peers' rows, rank-ordered sum + residual + RMSNorm (cq_comm_allreduce_add_rmsnorm); more "
                      "than 64 rows: cq_comm_push + cq_comm_reduce_add_rmsnorm",
        "decode_loop": "eager launches" if eager else "one CUDA graph replayed per token",
    }


def run_model(args, rank, world, device):
    """``--workload model7b|model20b``: the line's value is the end-to-end decode tok/s (see model_decode)."""
    big = args.workload == "model20b"
    res = model_decode(rank, world, device, big=big, batch=None if args.batch == 8 else args.batch,
                       steps=args.steps, bits=args.bits, eager=args.eager)
    return {
        "metric": "decode_tok_per_s", "value": res["tok_s"], "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": 3, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{res['model']}, batch {res['batch']}, prefill {res['prefill_tokens']} tokens, "
                               f"{args.steps} greedy steps, {args.bits}-bit KV (group 32)",
                   "parallelism": res["parallelism"], "decode_loop": res["decode_loop"],
                   "prefill_ms": res["prefill_ms"]},
        "model_decode": res,
    }


def run_pack(args, rank, world, device):
    """Quantize+pack of the visual span alone (the prefill-side kernel of the path): K per channel
    and V per token of `batch` rows per GPU, fp16 in, codes + scales + minima out."""
    peak, which = measured_peak()
    res = time_pack(args.batch, args.context, args.bits, device, reps=max(args.steps, 1))
    ms = res["k_per_channel"]["ms"] + res["v_per_token"]["ms"]
    n = args.batch * HKV * args.context * D
    nbytes = 2 * n * res["bytes_per_element"]
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t.item())
    gbps = world * nbytes / ms / 1e6
    worst = min(res["k_per_channel"]["GBps"], res["v_per_token"]["GBps"])
    return {
        "metric": f"pack_{args.bits}bit_GBps", "value": round(gbps, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": 2, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"quantize+pack K (per channel) and V (per token), batch {args.batch}/GPU, 8 KV heads, "
                               f"{args.context} tokens, head_dim 128, {args.bits}-bit, group 32",
                   "l2": "two source tensors of %.0f MB alternate" % (n * 2 / 1e6)},
        "kernels": res,
        "roofline": {"bound": "hbm", "kernel": "pack_k_per_channel_kernel / pack_last_dim_kernel",
                     "achieved": worst, "peak": peak, "unit": "GB/s", "frac": round(worst / peak, 4),
                     "peak_source": which, "traffic": None,
                     "algorithmic_bytes_per_element": res["bytes_per_element"]},
        "gpu_launches": 2 * max(args.steps, 1),
    }


def run_qjl(args, rank, world, device):
    """The QJL baseline's key path alone: sketch `batch` x 8 KV heads x `context` keys (256 + 256 sign bits per
    key, 32 outlier channels per group of 32) once, then time the score estimate of one query per head."""
    from calibquant_b200.qjl.qjl_utils import QJLSketch, QJLKeyQuantizer
    B, T = args.batch, args.context
    sk = QJLSketch((D, 256), 256, device=device, rng=torch.Generator(device=device).manual_seed(1))
    g = torch.Generator(device=device).manual_seed(2 + rank)
    k = torch.randn(B, HKV, T, D, generator=g, device=device).half()
    q = torch.randn(B, HQ, 1, D, generator=g, device=device).half()
    kq = QJLKeyQuantizer(sk, 32, 128, 32, 2)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kq.build_sketch(k)                                # first call also loads the kernels
    kq = QJLKeyQuantizer(sk, 32, 128, 32, 2)
    ev0.record()
    kq.build_sketch(k)
    ev1.record()
    torch.cuda.synchronize()
    build_ms = ev0.elapsed_time(ev1)
    for _ in range(max(args.warmup, 1)):
        kq.attention_score(q)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(args.steps):
        kq.attention_score(q)
    ev1.record()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1) / args.steps], device=device, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t.item())
    n_keys = B * HKV * (T - T % 128)
    nbytes = n_keys * (32 + 32 + 2 + 2)               # sign bits of both sketches + the two norms
    peak, which = measured_peak()
    gbps = world * nbytes / ms / 1e6
    return {
        "metric": "qjl_score_GBps", "value": round(gbps, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"QJL score estimate, batch {B}/GPU, {HQ}q/{HKV}kv heads, {T} sketched keys, "
                               "256+256-bit sketches, 32 outlier channels per group of 32 keys",
                   "build_sketch_ms": round(build_ms, 3)},
        "roofline": {"bound": "hbm", "kernel": "score_mma_kernel", "achieved": round(gbps / world, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(gbps / world / peak, 4), "peak_source": which, "traffic": None},
        "gpu_launches": args.steps,
    }


def time_prefill(device, world, B=16, T=3392, HQ=32, steps=5, warmup=3):
    """Time the dense causal prefill attention (tcgen05 kernel) on B rows x T tokens per GPU, 32 query / 8 KV
    heads, bf16.  Returns (ms per pass as the max over ranks, TFLOP/s of one GPU, peak, peak source, MB per pass)."""
    from calibquant_b200 import ops
    g = torch.Generator(device=device).manual_seed(3)
    q = torch.randn(B, T, HQ, D, generator=g, device=device).to(torch.bfloat16)
    k = torch.randn(B, T, HKV, D, generator=g, device=device).to(torch.bfloat16)
    v = torch.randn(B, T, HKV, D, generator=g, device=device).to(torch.bfloat16)
    out = torch.empty_like(q)
    for _ in range(max(warmup, 3)):
        ops.prefill_attention(q, k, v, out=out)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        ops.prefill_attention(q, k, v, out=out)
    ev1.record()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1) / steps], device=device, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t.item())
    flops = 4.0 * B * HQ * T * T * D / 2
    pk_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk_path):
        peak, which = float(json.load(open(pk_path))["bf16_tflops"]), "measured (cuBLAS bf16 burst)"
    else:
        peak, which = 1590.0, "fallback"
    return ms, flops / ms / 1e9, peak, which, (2 * q.numel() + 2 * k.numel()) * 2 / 1e6


def time_flash_attn_library(device, B=16, T=3392, HQ=32, steps=5):
    """The same shape through the third-party flash_attn package the reference calls for its prefill
    (patch_internvl.py:464-468): TFLOP/s of one GPU, or None where the package is missing or has no kernels for
    this GPU.  A library baseline beside the number, never part of it."""
    try:
        from flash_attn import flash_attn_func
        g = torch.Generator(device=device).manual_seed(3)
        q = torch.randn(B, T, HQ, D, generator=g, device=device).to(torch.bfloat16)
        k = torch.randn(B, T, HKV, D, generator=g, device=device).to(torch.bfloat16)
        v = torch.randn(B, T, HKV, D, generator=g, device=device).to(torch.bfloat16)
        for _ in range(3):
            flash_attn_func(q, k, v, causal=True)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            flash_attn_func(q, k, v, causal=True)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / steps
        return round(4.0 * B * HQ * T * T * D / 2 / ms / 1e9, 1)
    except Exception:
        return None


def prefill_key(device, world):
    """The `prefill` entry of the default line: config 2's prefill attention, batch 16 x 3392 tokens, 5 passes."""
    ms, tf, peak, which, mb = time_prefill(device, world)
    return {"flash_attn_library_TFLOPs_per_gpu": time_flash_attn_library(device),"metric": "prefill_attn_TFLOPs", "value": round(tf * world, 1), "unit": "TFLOP/s", "ms_per_pass": round(ms, 4),
            "config": "causal prefill attention, batch 16/GPU, 3392 tokens, 32q/8kv heads, head_dim 128, bf16; 5 passes "
                      f"after 3 warm-up; q+k+v+out = {mb:.0f} MB per pass (> L2)",
            "flops": "4*B*Hq*T^2*D/2 (causal half)", "kernel": "prefill_tc_kernel",
            "frac_of_peak": round(tf / peak, 4), "peak": peak, "peak_source": which}


def run_prefill(args, rank, world, device):
    """Dense causal prefill attention alone (tcgen05 kernel) on the 7B prefill shape: batch rows per
    GPU x 3392 tokens, 32 query / 8 KV heads, bf16."""
    B, T, HQ = (args.batch if args.batch != 8 else 16), 3392, 32
    ms, tf1, peak, which, mb = time_prefill(device, world, B, T, HQ, args.steps, args.warmup)
    tf = world * tf1
    return {
        "metric": "prefill_attn_TFLOPs", "value": round(tf, 1), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"causal prefill attention, batch {B}/GPU, {T} tokens, 32q/8kv heads, head_dim 128",
                   "flops": "4*B*Hq*T^2*D/2 (causal half)", "l2": "q+k+v+out = %.0f MB per pass" % mb},
        "roofline": {"bound": "tensor", "kernel": "prefill_tc_kernel", "achieved": round(tf / world, 1), "peak": peak,
                     "unit": "TFLOP/s", "frac": round(tf / world / peak, 4), "peak_source": which, "traffic": None},
        "gpu_launches": args.steps,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="attn", choices=["attn", "model7b", "model20b", "pack", "prefill", "qjl"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bits", type=int, default=1)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--fp-tokens", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of one row before timing")
    ap.add_argument("--no-model", action="store_true", help="skip the end-to-end model decode after the attention measurement")
    ap.add_argument("--eager", action="store_true", help="model workloads: no CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        torch.distributed.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=240))
    try:
        runner = {"attn": run_ours, "pack": run_pack, "prefill": run_prefill, "qjl": run_qjl}.get(args.workload, run_model)
        line = runner(args, rank, world, device)
        if rank == 0:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
