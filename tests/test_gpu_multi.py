"""Two-GPU checks: the KV-head sharding with an NCCL all-gather of head outputs, and the tensor-parallel
decode step over peer memory; skipped on one GPU."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_layer_on_two_gpus():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29617", os.path.join(root, "tests", "multi_gpu_worker.py")]
    res = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=420)
    errors = "\n".join(l for l in res.stderr.splitlines() if "Error" in l or "assert" in l)
    assert res.returncode == 0 and "MULTI_GPU_OK" in res.stdout, res.stdout[-1500:] + errors[-2500:]
