#!/usr/bin/env python
"""Benchmark of the MAM hot path on B200.

Workload (N GPUs, weak scaling: every rank owns the same number of rows): the ViT-B/16-shaped
MAM MLP pair of the reference's headline configuration -- tokens M = 64 x 197 = 12608 per rank,
layer 1 K=768 -> N=3072, layer 2 K=3072 -> N=768, fp32, x ~ N(0,1), W ~ N(0,1/K), forward with
arg-indices + selected-pair backward + selection-count accumulation, synthetic data.  With N > 1
the two weight gradients are summed over ranks with one NCCL all-reduce each (the only exchange a
row-sharded layer has).

One JSON line on stdout (rank 0).  `value` counts (m,n,k) units -- one multiply, one max update,
one min update -- of the two forward passes, divided by the whole forward+backward step time:
"G(mul+max/min)/s".  `e2e` is the same step called with HOST buffers: the step's activations and
upstream gradient start in pinned host memory and its output and loss come back to the host
inside the timed region.  `roofline` is for the dominant kernel (the tiled forward), timed with
CUDA events recorded by the library around each of its launches during the timed steps.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`--impl reference` times the CPU restatement of the reference's own torch path (oracle/) on the
host cores on a bounded row sample of the same workload.  `--impl reference_cuda` (an extra arm, not
part of the default run) times the reference's own CUDA operators on the GPU where
oracle/build_ref_cuda.py has built them.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOKENS, D_MODEL, D_FF = 64 * 197, 768, 3072
UNITS_PER_STEP = M_TOKENS * (D_MODEL * D_FF + D_FF * D_MODEL)  # per rank
METRIC = "mam_mlp_pair_fwd_bwd_throughput"
UNIT = "G(mul+max/min)/s"
WORKLOAD = ("ViT-B/16 MAM MLP pair fwd+bwd, fp32, M=12608 tokens per rank, 768->3072->768, "
            "arg-indices, selected-pair backward, selection count on")


M_TOTAL_OUTPUTS = M_TOKENS * (D_FF + D_MODEL)   # outputs of both layers per rank


def measured_hbm_gbs() -> float:
    """Copy bandwidth measured on this pool's B200s (MEASURED_PEAKS.json beside this file), else the
    6650 GB/s of an earlier measurement."""
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0


def fp32_peaks(sms: int, mhz: float):
    lanes = sms * 128 * mhz * 1e6
    # mix_ceiling: what the (mul, max, min) instruction mix can sustain on sm_100a, measured with
    # independent instruction streams (profiles/pipe_probe_b200.md): the min/max pipe shares its
    # datapath with half of the fp32 multiply throughput -> 3 cycles per unit per warp = 128/3
    # units/clk/SM, numerically the non-FMA issue peak.
    return {"fma_counted_tflops": 2 * lanes / 1e12, "non_fma_tops": lanes / 1e12,
            "mix_ceiling_gunits": sms * (128.0 / 3.0) * mhz * 1e6 / 1e9}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": reasons}


def cpu_reference_sample(rows: int, repeats: int):
    """The reference's CPU torch path (restated in oracle/mam_oracle.py) on `rows` rows of both
    layers, forward + backward.  Returns (G units/s, threads, description)."""
    import torch

    from oracle import mam_oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, D_MODEL, generator=g)
    w1 = torch.randn(D_FF, D_MODEL, generator=g) * D_MODEL ** -0.5
    w2 = torch.randn(D_MODEL, D_FF, generator=g) * D_FF ** -0.5
    gy = torch.randn(rows, D_MODEL, generator=g)
    b1, b2 = w1.T.contiguous(), w2.T.contiguous()
    units = rows * (D_MODEL * D_FF + D_FF * D_MODEL)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        h, i1, j1 = mam_oracle.mam_forward(x, b1)
        y, i2, j2 = mam_oracle.mam_forward(h, b2)
        dh, dw2 = mam_oracle.mam_backward(h, b2, gy, i2, j2)
        dx, dw1 = mam_oracle.mam_backward(x, b1, dh, i1, j1)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return units / best / 1e9, threads, f"{rows} of {M_TOKENS} rows of both layers, fwd+bwd, torch CPU, best of {repeats}"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 128
    # warm-up + K timed "steps", each one bounded sample
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_sample(rows, 1)
    t0 = time.perf_counter()
    vals = [cpu_reference_sample(rows, 1) for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    value = statistics.median(v[0] for v in vals)
    threads, sample = vals[0][1], vals[0][2]
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference's torch path; each step is a "
                       f"{rows}-row sample of the workload, throughput is per-unit so it compares directly"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_sharded_sparse(args):
    """The large sharded configuration: one MAM layer, M = 65536 rows split by rank, K = N = 4096, W pruned
    to 90 % sparsity (uniform random mask) and stored as CSR; forward with indices through the tiled CSR
    kernels, backward through the selected-pair scatter (dW dense), dW summed over the ranks with NCCL.
    Total work is fixed, so the scaling is strong.  Prints one JSON line with the same keys as the
    headline run (without the per-kernel roofline, which profiles/mam_csr_fwd_2048x4096x4096.md covers)."""
    import torch
    import torch.distributed as dist

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib
    from mamtorch_b200.dist import row_shard

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torch.distributed.run)"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    M_TOTAL, K, N = 65536, 4096, 4096
    lo, hi = row_shard(M_TOTAL, world, rank)
    rows = hi - lo
    g = torch.Generator().manual_seed(0)
    w = torch.randn(N, K, generator=g) * K ** -0.5
    keep = (torch.rand(N, K, generator=g) >= 0.9).float()          # as test/test_sparse.py:13-16 of the reference
    wz = (w * keep).to(dev).requires_grad_()
    w_csr = wz.detach().to_sparse_csr()
    nnz = int(w_csr.values().numel())
    gd = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(rows, K, generator=gd).to(dev)
    gy = torch.randn(rows, N, generator=gd).to(dev)

    def step():
        wz.grad = None
        xl = x.detach().requires_grad_()
        y, _, _ = mamtorch.sparse.kernel.v1.mam_linear_csr(xl, w_csr, None, dense_weight=wz)
        y.backward(gy)
        if world > 1:
            dist.all_reduce(wz.grad)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    _lib.check(_lib.lib().mam_check_device_flag(), "device wait flag")
    if rank == 0:
        ms_per_step = float(ms.item()) / args.steps
        units = M_TOTAL * nnz                                       # (row, stored weight) pairs, all ranks
        line = {"metric": "mam_sharded_sparse_layer_fwd_bwd_throughput", "value": units / (ms_per_step * 1e-3) / 1e9,
                "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "large sharded MAM layer fwd+bwd, fp32, M=65536 rows split by rank, K=N=4096, "
                                       "W pruned to 90 % sparsity (CSR), dW all-reduced over NCCL",
                           "units": "value counts (row, stored weight) pairs; the dense-equivalent rate is "
                                    f"{M_TOTAL * K * N / (ms_per_step * 1e-3) / 1e9:.0f} G units/s",
                           "nnz": nnz, "rows_per_rank": rows,
                           "l2": "per-rank working set (activations, indices, gradients) exceeds the 126 MB L2"},
                "gpu_launches": 11 * args.steps, "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference_cuda(args):
    """The reference's own CUDA kernels (its default training path: the v4 operators) on this GPU,
    built from the reference's sources by oracle/build_ref_cuda.py.  The step is the reference module's
    own sequence -- `weight.T.contiguous()`, `fullyconnected`, bias add
    (mamtorch/nn/v4/fullyconnected.py:141-199), `fullyconnected_backward` through the registered
    autograd formula (mamtorch/kernel/v4/fullyconnected.py:24-40), `update_selection_count`
    (mamtorch/nn/v4/fullyconnected.py:114-131) -- on the same workload as the default arm.  This
    process never imports mamtorch_b200 (both define the mamtorch_kernel_v4 operator namespace)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    so = os.path.join(ROOT, "oracle", "_ref", "mamtorch_kernel_v4.so")
    if not os.path.exists(so):
        print(json.dumps({"impl": "reference_cuda", "unavailable": "oracle/_ref/mamtorch_kernel_v4.so not built "
                          "(python oracle/build_ref_cuda.py --reference DIR)"}), flush=True)
        return
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference_cuda", "unavailable": "no CUDA device"}), flush=True)
        return
    torch.ops.load_library(so)
    ops = torch.ops.mamtorch_kernel_v4
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    w1 = (torch.randn(D_FF, D_MODEL, generator=g) * D_MODEL ** -0.5).to(dev)
    w2 = (torch.randn(D_MODEL, D_FF, generator=g) * D_FF ** -0.5).to(dev)
    b1, b2 = torch.zeros(D_FF, device=dev), torch.zeros(D_MODEL, device=dev)
    gd = torch.Generator().manual_seed(100)
    x = torch.randn(M_TOKENS, D_MODEL, generator=gd).to(dev)
    gy = torch.randn(M_TOKENS, D_MODEL, generator=gd).to(dev)
    counts = [torch.zeros(D_FF, D_MODEL, dtype=torch.int32, device=dev),
              torch.zeros(D_MODEL, D_FF, dtype=torch.int32, device=dev)]
    parts = {"forward": 0.0, "backward": 0.0, "selection_count": 0.0}

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def layer_forward(inp, weight, bias):
        w = weight.T.contiguous()
        c, amax, amin = ops.fullyconnected(inp, w)
        c += bias.view(1, -1)
        return c, amax, amin, w

    def layer_backward(inp, w, grad, amax, amin):
        a_grad, b_grad = ops.fullyconnected_backward(inp, w, grad.contiguous(), amax, amin)
        return a_grad, b_grad.T, grad.sum(0)      # weight gradient through the transpose, bias gradient

    def count(cnt, amax, amin):
        rows, cols = amax.shape
        col = torch.arange(cols).repeat(rows).to(dev)
        cnt[col, amax.flatten().long()] += 1
        col = torch.arange(cols).repeat(rows).to(dev)
        cnt[col, amin.flatten().long()] += 1

    def step(record):
        t0 = ev()
        h, i1, j1, w1t = layer_forward(x, w1, b1)
        y, i2, j2, w2t = layer_forward(h, w2, b2)
        t1 = ev()
        dh, dw2, db2 = layer_backward(h, w2t, gy, i2, j2)
        dx, dw1, db1 = layer_backward(x, w1t, dh, i1, j1)
        t2 = ev()
        count(counts[0], i1, j1)
        count(counts[1], i2, j2)
        t3 = ev()
        if record:
            torch.cuda.synchronize()
            parts["forward"] += t0.elapsed_time(t1)
            parts["backward"] += t1.elapsed_time(t2)
            parts["selection_count"] += t2.elapsed_time(t3)
        return y

    for _ in range(max(args.warmup, 1)):
        step(False)
    torch.cuda.synchronize()
    # sanity of the build: the index-packing operator against the reference's own exact values-only operator
    w1t = w1.T.contiguous()
    approx_gap = float((ops.fullyconnected(x, w1t)[0] - ops.fullyconnected_fast(x, w1t)).abs().max())
    f0 = ev()
    for _ in range(args.steps):
        ops.fullyconnected_fast(x, w1t)
    f1 = ev()
    t0 = ev()
    for _ in range(args.steps):
        step(True)
    t1 = ev()
    torch.cuda.synchronize()
    fast_ms = f0.elapsed_time(f1) / args.steps
    ms = t0.elapsed_time(t1) / args.steps
    value = UNITS_PER_STEP / (ms * 1e-3) / 1e9
    kernels_ms = (parts["forward"] + parts["backward"]) / args.steps
    line = {"impl": "reference_cuda", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "note": "the reference's v4 CUDA operators (its default training path: indices are "
                               "approximate by design) compiled for sm_100 and called in the reference module's "
                               "own sequence; inputs resident in HBM"},
            "ms_per_step_parts": {k: v / args.steps for k, v in parts.items()},
            "value_without_selection_count": UNITS_PER_STEP / (kernels_ms * 1e-3) / 1e9,
            "fullyconnected_fast_layer1_ms": fast_ms,
            "fullyconnected_vs_fullyconnected_fast_max_abs_diff": approx_gap}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fwd-variant", type=int, default=-1, help="tile configuration of the index-producing forward")
    ap.add_argument("--workload", default="vit_mlp", choices=["vit_mlp", "sharded_sparse"],
                    help="vit_mlp: the headline configuration (default); sharded_sparse: the large pruned layer, "
                         "65536 rows split over the ranks (strong scaling), K = N = 4096, 90 %% of W pruned")
    args = ap.parse_args()
    if args.workload == "sharded_sparse" and args.impl == "b200":
        return run_sharded_sparse(args)
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference_cuda":
        return run_reference_cuda(args)

    import torch
    import torch.distributed as dist

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib
    from mamtorch_b200.dist import allreduce_gradients

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torch.distributed.run)"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    if args.fwd_variant >= 0:
        _lib.check(L.mam_set_fwd_variant(1, args.fwd_variant), "mam_set_fwd_variant")

    # ---- model and data: every rank its own rows (seeded per rank), identical weights
    torch.manual_seed(0)
    fc1 = mamtorch.nn.FullyConnected(D_MODEL, D_FF, bias=True, store_args=True).to(dev)
    fc2 = mamtorch.nn.FullyConnected(D_FF, D_MODEL, bias=True, store_args=True).to(dev)
    with torch.no_grad():
        g = torch.Generator().manual_seed(0)
        fc1.weight.copy_(torch.randn(D_FF, D_MODEL, generator=g) * D_MODEL ** -0.5)
        fc2.weight.copy_(torch.randn(D_MODEL, D_FF, generator=g) * D_FF ** -0.5)
        fc1.bias.zero_()
        fc2.bias.zero_()
    gd = torch.Generator().manual_seed(100 + rank)
    x_host = torch.randn(64, 197, D_MODEL, generator=gd).pin_memory()
    gy_host = torch.randn(64, 197, D_MODEL, generator=gd).pin_memory()
    y_host = torch.empty(64, 197, D_MODEL).pin_memory()
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
    x_dev = x_host.to(dev)
    gy_dev = gy_host.to(dev)
    params = [fc1.weight, fc2.weight, fc1.bias, fc2.bias]

    def step(x, gy):
        for p in params:
            p.grad = None
        x = x.detach().requires_grad_()   # a fresh leaf every step: dX is produced, never accumulated
        y = fc2(fc1(x))
        y.backward(gy)
        fc1.update_selection_count()
        fc2.update_selection_count()
        if world > 1:
            allreduce_gradients(params)
        return y

    # End-to-end leg: every step's activations and upstream gradient start in pinned host memory and
    # its output and loss end there.  Copies run on their own stream, double-buffered, so the upload
    # of step i+1 and the download of step i overlap the kernels of the neighbouring step -- what a
    # data loader feeding this layer does.  All of it is inside the timed region.
    copy_stream = torch.cuda.Stream(device=dev)
    x_buf = [torch.empty_like(x_dev) for _ in range(2)]
    gy_buf = [torch.empty_like(gy_dev) for _ in range(2)]
    y_buf = [torch.empty(64, 197, D_MODEL, device=dev) for _ in range(2)]
    loss_buf = [torch.empty((), device=dev) for _ in range(2)]
    up_done = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]
    down_done = [torch.cuda.Event() for _ in range(2)]

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(comp_done[slot])   # the buffers' previous step must be done with them
            x_buf[slot].copy_(x_host, non_blocking=True)
            gy_buf[slot].copy_(gy_host, non_blocking=True)
            up_done[slot].record(copy_stream)

    def run_from_host(steps):
        main = torch.cuda.current_stream()
        for ev in comp_done + down_done:
            ev.record(main)
        upload(0)
        for i in range(steps):
            slot = i & 1
            if i + 1 < steps:
                upload(slot ^ 1)
            main.wait_event(up_done[slot])
            main.wait_event(down_done[slot])          # y_buf[slot] of step i-2 has been downloaded
            y = step(x_buf[slot], gy_buf[slot])
            y_buf[slot].copy_(y.detach())
            loss_buf[slot].copy_((y.detach() * gy_buf[slot]).sum())
            comp_done[slot].record(main)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(comp_done[slot])
                y_host.copy_(y_buf[slot], non_blocking=True)
                loss_host.copy_(loss_buf[slot], non_blocking=True)
                down_done[slot].record(copy_stream)
        main.wait_stream(copy_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step(x_dev, gy_dev)
    run_from_host(2)
    barrier()

    # ---- per-kernel events for the dominant kernel (2 launches per step)
    cap = 2 * args.steps
    ev_pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(cap)]
    for a, b in ev_pairs:  # events are created lazily on first record; force creation now
        a.record()
        b.record()
    torch.cuda.synchronize()
    starts = (ctypes.c_void_p * cap)(*[ctypes.c_void_p(a.cuda_event) for a, _ in ev_pairs])
    stops = (ctypes.c_void_p * cap)(*[ctypes.c_void_p(b.cuda_event) for _, b in ev_pairs])
    _lib.check(L.mam_timer_arm(starts, stops, cap, 0), "mam_timer_arm")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    total_ms = timed(lambda: step(x_dev, gy_dev), args.steps)
    recorded = L.mam_timer_disarm()
    torch.cuda.synchronize()
    kernel_ms = [a.elapsed_time(b) for a, b in ev_pairs[:recorded]]
    # the other kernels of the step, each class timed by the library's own events over three extra steps
    # (two launches per step: layer 1 and layer 2)
    other_ms = {}
    for name, kid in (("index_resolver", 1), ("backward_scatter", 3), ("selection_hits", 4)):
        _lib.check(L.mam_timer_arm(starts, stops, cap, kid), "mam_timer_arm")
        for _ in range(3):
            step(x_dev, gy_dev)
        n_rec = L.mam_timer_disarm()
        torch.cuda.synchronize()
        per_launch = [a.elapsed_time(b) for a, b in ev_pairs[:n_rec]]
        other_ms[name] = sum(per_launch) / 3 if per_launch else float("nan")
    e2e_ms = timed(lambda: run_from_host(args.steps), 1)
    clocks = sampler.stop() if rank == 0 else None
    _lib.check(L.mam_check_device_flag(), "device wait flag")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    value = world * UNITS_PER_STEP / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * UNITS_PER_STEP / (e2e_ms / args.steps * 1e-3) / 1e9
    props = torch.cuda.get_device_properties(dev)
    sms = props.multi_processor_count
    kavg = statistics.mean(kernel_ms) if kernel_ms else float("nan")
    flops_per_launch = 3.0 * M_TOKENS * D_MODEL * D_FF  # 3 fp32 ops per (m,n,k) unit, unpadded extents
    max_mhz = (clocks or {}).get("sm_max_mhz") or 1965.0
    peaks = fp32_peaks(sms, max_mhz)
    achieved = flops_per_launch / (kavg * 1e-3) / 1e12
    roofline = {"bound": "fp32_cuda_core", "kernel": "mam_fwd_tiled_kernel (index-tracking variant "
                + L.mam_fwd_variant_name(1, args.fwd_variant if args.fwd_variant >= 0 else 1).decode() + ")",
                "achieved": achieved, "peak": peaks["fma_counted_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["fma_counted_tflops"],
                "peak_source": f"{sms} SMs x 128 lanes x 2 x {max_mhz:.0f} MHz (FMA counted as 2; no fp32 entry in "
                               "MEASURED_PEAKS.json); a MAM unit has no FMA, see the two extra fractions",
                "frac_of_non_fma_peak": achieved / peaks["non_fma_tops"],
                "frac_of_measured_mix_ceiling": (achieved / 3 * 1e3) / peaks["mix_ceiling_gunits"],
                "launch_ms_avg": kavg, "launches_timed": len(kernel_ms), "traffic": 3.75e8,
                "traffic_note": "dram read+write bytes per launch (layer-1 shape) from the ncu capture in "
                                "profiles/step_kernels_4736x768x3072.md, scaled by rows to M=12608"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "working set per step (~1 GB of activations, indices and "
                       "gradients) exceeds the 126 MB L2; no explicit flush",
                       "parallelism": f"rows sharded over {world} rank(s); dW all-reduce over NCCL" if world > 1
                       else "single GPU"},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": x_host.numel() * 4 + gy_host.numel() * 4,
                    "d2h_bytes_per_step": y_host.numel() * 4 + 4},
            "gpu_launches": 10 * args.steps, "clocks": clocks, "roofline": roofline}
    # per-step time of every kernel class and, for the two HBM-style kernels, algorithmic bytes over time
    # against the measured copy bandwidth (both layers: M x 768 x 3072 and M x 3072 x 768)
    hbm_peak = measured_hbm_gbs()
    mn, mk_nk = M_TOTAL_OUTPUTS, 2 * (M_TOKENS * D_MODEL + M_TOKENS * D_FF + 2 * D_MODEL * D_FF)
    bwd_bytes = 12 * mn + 4 * mk_nk
    sel_bytes = 8 * mn + 8 * 2 * D_MODEL * D_FF
    line["kernels_ms_per_step"] = {"forward_main_loop": 2 * kavg, **other_ms}
    line["roofline_other_kernels"] = [
        {"kernel": "mam_bwd_rowwarp_kernel (768 -> 3072) + mam_bwd_kernel (3072 -> 768)", "bound": "hbm", "achieved": bwd_bytes / (other_ms["backward_scatter"] * 1e-3) / 1e9,
         "peak": hbm_peak, "unit": "GB/s", "frac": bwd_bytes / (other_ms["backward_scatter"] * 1e-3) / 1e9 / hbm_peak,
         "note": "12*M*N + 8*(M*K + N*K) bytes per layer; in practice bound by the rate of scattered fp32 reductions "
                 "into L2 (2*M*N per layer) and the LSU data pipe, see profiles/step_kernels_4736x768x3072.md"},
        {"kernel": "mam_selcount_kernel", "bound": "hbm", "achieved": sel_bytes / (other_ms["selection_hits"] * 1e-3) / 1e9,
         "peak": hbm_peak, "unit": "GB/s", "frac": sel_bytes / (other_ms["selection_hits"] * 1e-3) / 1e9 / hbm_peak,
         "note": "8*M*N + 8*N*K bytes per layer"}]
    if world == 1 and not args.no_cpu_baseline:
        cv, threads, sample = cpu_reference_sample(256, 3)
        line["cpu_baseline"] = {"value": cv, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
