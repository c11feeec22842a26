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

__all__ = ["row_shard", "shard_rows", "broadcast_parameters", "allreduce_gradients", "allreduce_counts",
           "OverlappedGradSync"]


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
    """Sum over ranks, in place.  Tensors of `bucket_bytes` or more (a layer's weight gradient) go as they
    are -- no staging copy; smaller ones (biases, counters) of one dtype are grouped into one coalesced
    launch, or, where the backend has no coalescing, packed into one flat buffer and copied back."""
    small: dict[torch.dtype, list[torch.Tensor]] = {}
    for t in tensors:
        if t.numel() * t.element_size() >= bucket_bytes or not t.is_contiguous():
            dist.all_reduce(t)
        else:
            small.setdefault(t.dtype, []).append(t)
    for group in small.values():
        if len(group) == 1:
            dist.all_reduce(group[0])
            continue
        flat = torch.cat([t.reshape(-1) for t in group])
        dist.all_reduce(flat)
        off = 0
        for t in group:
            t.copy_(flat[off:off + t.numel()].view_as(t))
            off += t.numel()


class OverlappedGradSync:
    """All-reduces every parameter's gradient without a staging copy, off the compute stream.

    A hook on each parameter (`register_post_accumulate_grad_hook`) fires as soon as autograd has finished
    accumulating its gradient.  In the default mode the hook starts an asynchronous, in-place all-reduce of
    `param.grad` right away; with NCCL it runs on the process group's own stream, ordered after the kernel that
    produced the gradient, while the backward of the earlier layers carries on on the compute stream: the
    weight gradient of the last layer crosses NVLink under the backward of the layers before it.

    `deferred=True` only notes the gradients in the hooks; `start()` then launches all the (asynchronous)
    all-reduces at once.  That is for a backward whose own kernels are bound by the same L2 / memory system the
    collective's kernels use -- the MAM scatter backward is -- where running the two side by side costs more
    than it hides, and the exchange is better put under whatever follows the backward (bookkeeping kernels,
    the next data copy).

    `finish()` makes the current stream wait for all started collectives -- call it once after `backward()`,
    before the gradients are read.  Sums, like `allreduce_gradients` (pass `average=True` for the mean).
    `enabled = False` turns the hooks into no-ops."""

    def __init__(self, params: Iterable[torch.nn.Parameter], average: bool = False, group=None,
                 deferred: bool = False):
        self.average, self.group, self.enabled, self.deferred = average, group, True, deferred
        self._works: list = []
        self._grads: list[torch.Tensor] = []
        self._pending: list[torch.Tensor] = []
        self._handles = [p.register_post_accumulate_grad_hook(self._hook) for p in params if p.requires_grad]

    def _hook(self, param: torch.nn.Parameter) -> None:
        if not self.enabled or param.grad is None:
            return
        if self.deferred:
            self._pending.append(param.grad)
            return
        self._works.append(dist.all_reduce(param.grad, group=self.group, async_op=True))
        self._grads.append(param.grad)

    def start(self) -> None:
        """Deferred mode: launch the all-reduces of every gradient noted since the last finish()."""
        for g in self._pending:
            self._works.append(dist.all_reduce(g, group=self.group, async_op=True))
            self._grads.append(g)
        self._pending.clear()

    def finish(self) -> None:
        self.start()
        for w in self._works:
            w.wait()
        if self.average:
            n = dist.get_world_size(self.group)
            for g in self._grads:
                g.div_(n)
        self._works.clear()
        self._grads.clear()

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles.clear()


def allreduce_gradients(params: Iterable[torch.nn.Parameter], average: bool = False,
                        bucket_bytes: int = 1 << 20) -> None:
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
    _flat_allreduce(tensors, 1 << 20)
