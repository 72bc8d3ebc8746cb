"""Multi-GPU partitioning of the recurrent path: one process per GPU, torch.distributed for the plumbing.

The recurrence shards naturally (the reference itself is single-GPU; it has no counterpart of this file):

* batch sharding -- rank r owns the batch rows ``[r*B/k, (r+1)*B/k)``; R and b are replicated; forward and
  backward are local; the only exchange is one all-reduce (sum) of the packed fp32 ``dR || db`` after the
  backward loop, issued from inside the autograd function on the compute stream;
* head sharding -- rank r owns heads ``[r*N/k, (r+1)*N/k)`` of Wx, R, b and the states; heads never interact
  (block-diagonal R), so there is no collective at all and dR/db stay sharded like R/b.
"""
from __future__ import annotations

import torch


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open index range of shard ``rank``; the first ``total % world`` shards get one extra element."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(Wx, states, rank: int, world: int):
    """Batch slice of the per-sample tensors (Wx[B,...], states[S,B,...]); R and b are replicated."""
    lo, hi = shard_range(Wx.shape[0], rank, world)
    return Wx[lo:hi], (None if states is None else states[:, lo:hi])


def shard_heads(Wx, R, b, states, rank: int, world: int):
    """Head slice of every tensor (Wx dim 3, R dim 1, b dim 1, states dim 3)."""
    lo, hi = shard_range(Wx.shape[3], rank, world)
    return Wx[:, :, :, lo:hi], R[:, lo:hi], b[:, lo:hi], (None if states is None else states[:, :, :, lo:hi])


def allreduce_param_grads(dR: torch.Tensor, db: torch.Tensor, group=None):
    """Sum dR and db over the batch shards with ONE collective on a packed fp32 buffer; returns fp32 tensors.
    The native path does the same on its fp32 workspace before casting; this helper serves host-side callers."""
    flat = torch.cat([dR.reshape(-1).float(), db.reshape(-1).float()])
    torch.distributed.all_reduce(flat, group=group)
    return flat[: dR.numel()].view_as(dR), flat[dR.numel():].view_as(db)


def flashrnn_batch_sharded(Wx_local, R, b, states_local=None, function="lstm", group=None, **kw):
    """``flashrnn`` on this rank's batch slice; dR/db come back already summed over all ranks of ``group``."""
    from .flashrnn import flashrnn

    return flashrnn(Wx_local, R, b, states_local, function=function,
                    grad_allreduce_group=(group if group is not None else True), **kw)


def flashrnn_head_sharded(Wx_local, R_local, b_local, states_local=None, function="lstm", **kw):
    """``flashrnn`` on this rank's heads; no collective is needed."""
    from .flashrnn import flashrnn

    return flashrnn(Wx_local, R_local, b_local, states_local, function=function, **kw)
