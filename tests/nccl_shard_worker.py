"""Worker of tests/test_gpu_multi.py: one process per GPU (torchrun), NCCL.

Every rank builds the same seeded full-batch problem, runs `flashrnn_batch_sharded` on its own batch slice (the
autograd function all-reduces the packed fp32 dR || db over NCCL before casting) and checks: its states / dWx / ds0
rows equal the rows of a single-GPU run over the whole batch, and the summed dR / db equal both that run's and the
oracle's.  Head sharding is checked the same way (no collective).  Prints NCCL_SHARD_OK on rank 0."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from flashrnn_b200 import flashrnn  # noqa: E402
from flashrnn_b200.sharding import flashrnn_batch_sharded, flashrnn_head_sharded, shard_batch, shard_heads  # noqa: E402
from tests.util import GRAD_REL_L2, make_inputs, rel_l2, run_oracle  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    f = lambda t: t.detach().to(torch.float64).cpu().numpy()
    for function, (B, T, N, D) in (("lstm", (16, 24, 2, 256)), ("elman", (256, 16, 4, 64)), ("gru", (12, 20, 4, 128))):
        cpu = make_inputs(function, B, T, N, D, seed=41, random_init=True)
        Wx, R, b, s0 = (t.to(dev, torch.bfloat16) for t in cpu)
        # ---- single GPU, whole batch
        full = [t.clone().requires_grad_(True) for t in (Wx, R, b, s0)]
        st_full, _ = flashrnn(*full, function=function)
        st_full[0].float().sum().backward()
        # ---- batch shard of this rank; dR/db come back summed over the ranks
        Wx_l, s0_l = shard_batch(Wx, s0, rank, world)
        lo = sum(Wx.shape[0] // world + (1 if r < Wx.shape[0] % world else 0) for r in range(rank))
        loc = [Wx_l.contiguous().clone().requires_grad_(True), R.clone().requires_grad_(True), b.clone().requires_grad_(True),
               s0_l.contiguous().clone().requires_grad_(True)]
        st_l, _ = flashrnn_batch_sharded(loc[0], loc[1], loc[2], loc[3], function=function)
        st_l[0].float().sum().backward()
        hi = lo + Wx_l.shape[0]
        assert torch.equal(st_l, st_full[:, lo:hi]), (function, "states rows")
        # a shard may run with another cluster size than the whole batch (the tile table looks at the number of batch
        # tiles), which changes the order of the fp32 sums behind dh: equal to rounding, not to the bit
        assert rel_l2(f(loc[0].grad), f(full[0].grad[lo:hi])) <= 0.5 * GRAD_REL_L2, (function, "dWx rows")
        assert rel_l2(f(loc[3].grad), f(full[3].grad[:, lo:hi])) <= 0.5 * GRAD_REL_L2, (function, "ds0 rows")
        ref = run_oracle(function, *cpu)
        for name, got, one in (("dR", loc[1].grad, full[1].grad), ("db", loc[2].grad, full[2].grad)):
            assert rel_l2(f(got), f(one)) <= GRAD_REL_L2, (function, name, "vs single GPU", rel_l2(f(got), f(one)))
            assert rel_l2(f(got), ref[name]) <= GRAD_REL_L2, (function, name, "vs oracle", rel_l2(f(got), ref[name]))
        # ---- head shard of this rank: no collective, gradients stay sharded like R and b
        if N % world == 0:
            Wx_h, R_h, b_h, s0_h = (t.contiguous().clone().requires_grad_(True) for t in shard_heads(Wx, R, b, s0, rank, world))
            st_h, _ = flashrnn_head_sharded(Wx_h, R_h, b_h, s0_h, function=function)
            st_h[0].float().sum().backward()
            h0, h1 = rank * (N // world), (rank + 1) * (N // world)
            assert torch.equal(st_h, st_full[:, :, :, h0:h1]), (function, "head-shard states")
            assert rel_l2(f(R_h.grad), f(full[1].grad[:, h0:h1])) <= GRAD_REL_L2, (function, "head-shard dR")
            assert rel_l2(f(b_h.grad), f(full[2].grad[:, h0:h1])) <= GRAD_REL_L2, (function, "head-shard db")
    dist.barrier()
    if rank == 0:
        print("NCCL_SHARD_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
