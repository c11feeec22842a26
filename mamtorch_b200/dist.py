"""Row-sharded data parallelism for MAM layers.

The MAM path shards by rows of the activation matrix: an output row needs its own input row and
the whole weight, nothing else.  So every rank keeps a full replica of the weights, owns a
contiguous block of rows, and runs forward, index selection and dX without talking to anyone; the
only exchange is the sum of the per-rank weight gradients (and, if wanted, of the integer
selection hits) after the backward.  The reference has no distributed code at all; this module is
what its data-parallel use looks like.

One process per GPU, `torch.distributed` (NCCL on GPUs; the helpers are backend-agnostic and are
tested with gloo on CPU).
"""
from __future__ import annotations

from typing import Iterable, Sequence

import torch
import torch.distributed as dist

__all__ = ["row_shard", "shard_rows", "broadcast_parameters", "allreduce_gradients", "allreduce_counts"]


def row_shard(total_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the rows rank `rank` owns: blocks differ by at most one row and cover
    0..total_rows exactly once, in rank order."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(total_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, world_size: int | None = None, rank: int | None = None) -> torch.Tensor:
    """The block of rows (first dimension) of `x` that this rank owns."""
    world_size = dist.get_world_size() if world_size is None else world_size
    rank = dist.get_rank() if rank is None else rank
    lo, hi = row_shard(x.shape[0], world_size, rank)
    return x[lo:hi]


def broadcast_parameters(module: torch.nn.Module, src: int = 0) -> None:
    """Replicates rank `src`'s parameters into every rank's own memory (one-time set-up)."""
    for p in module.parameters():
        dist.broadcast(p.data, src)


def _flat_allreduce(tensors: Sequence[torch.Tensor], bucket_bytes: int) -> None:
    """Sum over ranks, packing small tensors into buckets so each collective amortises its launch."""
    bucket, size = [], 0

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        if len(bucket) == 1:
            dist.all_reduce(bucket[0])
        else:
            flat = torch.cat([t.reshape(-1) for t in bucket])
            dist.all_reduce(flat)
            off = 0
            for t in bucket:
                t.copy_(flat[off:off + t.numel()].view_as(t))
                off += t.numel()
        bucket, size = [], 0

    for t in tensors:
        nbytes = t.numel() * t.element_size()
        if bucket and (size + nbytes > bucket_bytes or t.dtype != bucket[0].dtype):
            flush()
        bucket.append(t)
        size += nbytes
    flush()


def allreduce_gradients(params: Iterable[torch.nn.Parameter], average: bool = False,
                        bucket_bytes: int = 32 << 20) -> None:
    """Sums `.grad` of the given parameters over all ranks, in place.  With row sharding the sum
    (not the mean) is the gradient of the un-sharded batch."""
    grads = [p.grad for p in params if p.grad is not None]
    _flat_allreduce(grads, bucket_bytes)
    if average:
        w = dist.get_world_size()
        for g in grads:
            g.div_(w)


def allreduce_counts(modules: Iterable[torch.nn.Module]) -> None:
    """Sums the integer selection-hit matrices a rank accumulated (`hit_max`, `hit_min` attributes,
    if a caller keeps them) or, for the reference-style counters, nothing: the 0/1-per-call rule of
    `update_selection_count` is not additive over ranks, so callers that need global counts
    all-reduce true hits and derive the indicator afterwards."""
    tensors = []
    for m in modules:
        for name in ("hit_max", "hit_min"):
            t = getattr(m, name, None)
            if isinstance(t, torch.Tensor):
                tensors.append(t)
    _flat_allreduce(tensors, 32 << 20)
