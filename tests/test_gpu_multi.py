"""GPU (two or more): the batch-sharded and head-sharded product paths over NCCL, one process per GPU.

The CPU suite checks the partition arithmetic with gloo ranks (tests/test_sharding_gloo.py); this one runs the real
thing -- `flashrnn(..., grad_allreduce_group=...)`, whose backward all-reduces the fp32 workspace slice between the
reverse loop and the cast -- and compares it with a single-GPU run and with the oracle (tests/nccl_shard_worker.py).
Skipped on a single-GPU box."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_batch_and_head_sharding_over_nccl(cuda_device):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(ROOT / "tests" / "nccl_shard_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "NCCL_SHARD_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
