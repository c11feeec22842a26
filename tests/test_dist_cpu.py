"""Sharding and reduction bookkeeping of the row-sharded layer, with gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mamtorch_b200.dist import OverlappedGradSync, allreduce_gradients, row_shard, shard_rows
from oracle import mam_oracle


def test_row_shard_partitions_exactly():
    for total in (0, 1, 7, 64, 12608, 65536, 65537):
        for world in (1, 2, 3, 8):
            spans = [row_shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_shard(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        M, K, N = 37, 24, 10
        x = torch.randn(M, K, generator=g)
        w = torch.randn(N, K, generator=g)
        gy = torch.randn(M, N, generator=g)
        xs, gs = shard_rows(x), shard_rows(gy)
        b = w.T.contiguous()
        y, imax, imin = mam_oracle.mam_forward(xs, b)      # stand-in for the rank-local GPU forward
        dx, db = mam_oracle.mam_backward(xs, b, gs, imax, imin)
        wp = torch.nn.Parameter(w.clone())
        bp = torch.nn.Parameter(torch.zeros(N))
        wp.grad = db.T.contiguous()
        bp.grad = gs.sum(0)
        wp2 = torch.nn.Parameter(w.clone())
        wp2.grad = db.T.contiguous()
        allreduce_gradients([wp, bp], bucket_bytes=4096)     # both below the bucket size: packed into one launch
        allreduce_gradients([wp2], bucket_bytes=64)          # at or above it: reduced in place, no staging copy
        # gradient hooks: the all-reduce starts when autograd has accumulated the gradient, finish() waits
        lin_w = torch.nn.Parameter(w.clone())
        lin_b = torch.nn.Parameter(torch.zeros(N))
        sync = OverlappedGradSync([lin_w, lin_b])
        ((xs @ lin_w.T + lin_b) * gs).sum().backward()
        sync.finish()
        hooked_ok = torch.allclose(lin_w.grad, gy.T @ x, rtol=1e-5, atol=1e-5) and \
            torch.allclose(lin_b.grad, gy.sum(0), rtol=1e-5, atol=1e-6)
        sync.enabled = False
        lin_w.grad = None
        ((xs @ lin_w.T) * gs).sum().backward()
        sync.finish()
        hooked_ok &= torch.allclose(lin_w.grad, gs.T @ xs, rtol=1e-5, atol=1e-5)   # disabled: the rank's own gradient
        sync.remove()
        # deferred mode: the hooks only note the gradients, start() launches, finish() waits
        lin_w.grad = None
        sync = OverlappedGradSync([lin_w], deferred=True)
        ((xs @ lin_w.T) * gs).sum().backward()
        hooked_ok &= torch.allclose(lin_w.grad, gs.T @ xs, rtol=1e-5, atol=1e-5)   # nothing exchanged yet
        sync.start()
        sync.finish()
        hooked_ok &= torch.allclose(lin_w.grad, gy.T @ x, rtol=1e-5, atol=1e-5)
        sync.remove()
        if rank == 0:
            y_full, imax_f, imin_f = mam_oracle.mam_forward(x, b)
            _, db_full = mam_oracle.mam_backward(x, b, gy, imax_f, imin_f)
            lo, hi = row_shard(M, world, rank)
            ok = torch.equal(y, y_full[lo:hi])
            ok &= torch.allclose(wp.grad, db_full.T, rtol=1e-5, atol=1e-6)
            ok &= torch.allclose(bp.grad, gy.sum(0), rtol=1e-5, atol=1e-6)
            ok &= torch.allclose(wp2.grad, db_full.T, rtol=1e-5, atol=1e-6)
            ok &= bool(hooked_ok)
            out.put(bool(ok))
    finally:
        dist.destroy_process_group()


def test_sharded_backward_equals_unsharded_world2():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) is True
