"""CPU, world_size 2 (gloo): the multi-GPU partitioning logic.  Each rank runs the ORACLE on its shard (the
CUDA kernels need a GPU); what is tested is the host-side path around them: batch/head partitioning, the single
packed all-reduce of dR || db, and that the sharded result equals the unsharded one."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, mode, ret):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flashrnn_b200.sharding import allreduce_param_grads, shard_batch, shard_heads, shard_range
    from oracle import oracle_fwbw
    from tests.util import make_inputs

    function = "gru" if mode == "heads" else "lstm"
    Wx, R, b, s0 = make_inputs(function, 5, 6, 4, 16, seed=3, random_init=True)
    full = oracle_fwbw(function, Wx.numpy(), R.numpy(), b.numpy(), s0.numpy())
    if mode == "batch":
        Wl, sl = shard_batch(Wx, s0, rank, world)
        o = oracle_fwbw(function, Wl.numpy(), R.numpy(), b.numpy(), sl.numpy())
        dR, db = allreduce_param_grads(torch.from_numpy(o["dR"]), torch.from_numpy(o["db"]))
        lo, hi = shard_range(5, rank, world)
        ok = np.allclose(dR.numpy(), full["dR"], atol=1e-5) and np.allclose(db.numpy(), full["db"], atol=1e-5)
        ok = ok and np.allclose(o["states"], full["states"][:, lo:hi]) and np.allclose(o["dWx"], full["dWx"][lo:hi])
    else:
        Wl, Rl, bl, sl = shard_heads(Wx, R, b, s0, rank, world)
        o = oracle_fwbw(function, Wl.numpy(), Rl.numpy(), bl.numpy(), sl.numpy())
        lo, hi = shard_range(4, rank, world)
        ok = np.allclose(o["dR"], full["dR"][:, lo:hi]) and np.allclose(o["db"], full["db"][:, lo:hi])
        ok = ok and np.allclose(o["states"], full["states"][:, :, :, lo:hi])
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret.put(float(flag.item()))
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["batch", "heads"])
def test_sharded_equals_unsharded(mode):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29500 + (os.getpid() % 400) + (0 if mode == "batch" else 500)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert ret.get(timeout=10) == 1.0


def test_shard_range_covers_everything():
    from flashrnn_b200.sharding import shard_range

    for total in (1, 5, 8, 1024):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
