#!/usr/bin/env python
"""Benchmark of the MAM hot path on B200.

Headline workload (N GPUs, weak scaling: every rank owns the same number of rows): the
ViT-B/16-shaped MAM MLP pair -- tokens M = 64 x 197 = 12608 per rank, layer 1 K=768 -> N=3072,
layer 2 K=3072 -> N=768, fp32, x ~ N(0,1), W ~ N(0,1/K), forward with arg-indices + selected-pair
backward + selection-count accumulation, synthetic data.  With N > 1 the weight gradients are
summed over ranks with NCCL, each as soon as its layer's backward has produced it, on NCCL's own
stream, so that the exchange runs under the rest of the backward.

One JSON line on stdout (rank 0).  `value` counts (m,n,k) units -- one multiply, one max update,
one min update -- of the two forward passes, divided by the whole forward+backward step time:
"G(mul+max/min)/s".  `e2e` is the same step called with HOST buffers: the step's activations and
upstream gradient start in pinned host memory and its output and loss come back to the host
inside the timed region.  `roofline` is for the dominant kernel (the tiled forward), timed with
CUDA events recorded by the library around each of its launches during the timed steps.

The same line carries `north_star_configs`: the other configurations the path is specified on,
each measured in this run with CUDA events (max over ranks) -- the 4096^3 forward (values only;
with indices: main loop and index resolver), the convolution and the beta-blended training step
(one GPU only), and the large sharded pruned layer at this N (65536 rows split over the ranks,
strong scaling, dW all-reduced) with the time of its all-reduce alone.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`--impl reference` times the reference's own CPU torch path on the host cores on a bounded row
sample of the same workload: the reference's checker functions byte-compiled into oracle/_ref/ where
that was built, else their restatement in oracle/mam_oracle.py.  `--impl reference_cuda` (an extra
arm, not part of the default run) times the reference's own CUDA operators on the GPU where
oracle/build_ref_cuda.py has built them.  `--case OP --shape ...` runs one operation a few times and
prints its time: the small, bounded command that profiler captures are taken on.
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

# DRAM bytes (read + write) of one launch of the index-tracking forward at M=4736, K=768, N=3072, from a
# profiler capture of `bench.py --case step --shape 4736x768x3072 --reps 1`: 24.2 MB read (of which the
# 9.4 MB weight does not depend on M) + 64.4 MB written.  The rest grows with the rows, so a launch at M rows
# moves about 9.4 MB + 79.2 MB * M / 4736.
TRAFFIC_CAPTURED_ROWS, TRAFFIC_CAPTURED_BYTES, TRAFFIC_WEIGHT_BYTES = 4736, 7.92e7, 9.4e6

SHARDED_M, SHARDED_K, SHARDED_N, SHARDED_SPARSITY = 65536, 4096, 4096, 0.9
CONV_SHAPE = (128, 64, 56, 56, 128)      # B, C, H, W, F; 3x3, stride 1, padding 1


def measured_hbm_gbs() -> float:
    """Copy bandwidth measured on this pool's B200s (MEASURED_PEAKS.json beside this file), else the
    6650 GB/s of an earlier measurement."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0


def fp32_peaks(sms: int, mhz: float):
    lanes = sms * 128 * mhz * 1e6
    # mix_ceiling: what the (mul, max, min) instruction mix can sustain on sm_100a, measured with
    # independent instruction streams: the min/max pipe shares its datapath with half of the fp32
    # multiply throughput -> 3 cycles per unit per warp = 128/3 units/clk/SM, numerically the
    # non-FMA issue peak.
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


def bind_to_gpu_numa_node(local: int):
    """Best effort: run this rank's host threads on the NUMA node its GPU hangs off and ask the kernel to place
    this process's memory there (the pinned buffers are allocated afterwards), so that eight ranks do not pull
    their host copies through one node or across the socket link.  Returns what was done:
    {"gpu_node", "cpus_bound", "memory_preferred"}, or None where the system does not name a node."""
    try:
        import torch

        props = torch.cuda.get_device_properties(local)
        path = f"/sys/bus/pci/devices/{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return None
        done = {"gpu_node": node, "cpus_bound": False, "memory_preferred": False}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            done["cpus_bound"] = True
        if node < 63 and sys.platform.startswith("linux") and os.uname().machine == "x86_64":
            # set_mempolicy(MPOL_PREFERRED, {node}): also helps where this rank's cores are all on another node
            mask = ctypes.c_ulong(1 << node)
            rc = ctypes.CDLL(None, use_errno=True).syscall(238, 1, ctypes.byref(mask), ctypes.c_ulong(64))
            done["memory_preferred"] = rc == 0
        return done
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


# ------------------------------------------------------------------------------------------------
# CPU legs: the reference's own torch path on the host cores
# ------------------------------------------------------------------------------------------------
class CpuPath:
    """The reference's CPU functions: its own checker (`test/reference.py`, byte-compiled into
    oracle/_ref/reference_checker.bin by oracle/build_ref_py.py where a checkout was at hand when the tree was
    built; kind "reference") or their restatement in oracle/mam_oracle.py (kind "port")."""

    def __init__(self):
        import torch

        self.threads = os.cpu_count() or 1
        torch.set_num_threads(self.threads)
        self.kind, self._ref = "port", None
        pyc = os.path.join(ROOT, "oracle", "_ref", "reference_checker.bin")
        if os.path.exists(pyc):
            try:
                import importlib.machinery
                import importlib.util

                loader = importlib.machinery.SourcelessFileLoader("mamtorch_reference_checker", pyc)
                spec = importlib.util.spec_from_loader("mamtorch_reference_checker", loader)
                mod = importlib.util.module_from_spec(spec)
                loader.exec_module(mod)
                self._ref, self.kind = mod, "reference"
            except Exception:  # noqa: BLE001  (a .pyc of another interpreter version: fall back to the port)
                self._ref = None
        if self._ref is None:
            from oracle import mam_oracle

            self._port = mam_oracle

    def forward(self, a, b, beta=0.0):
        if self._ref is not None:
            return self._ref.fullyconnected_reference(a, b, 0.0, beta)
        return self._port.mam_forward(a, b, beta=beta)

    def backward(self, a, b, g, imax, imin, beta=0.0):
        if self._ref is not None:
            return self._ref.fullyconnected_backward_reference(a, b, g, imax, imin, beta)
        return self._port.mam_backward(a, b, g, imax, imin, beta=beta)


def cpu_mlp_pair_sample(cpu: CpuPath, rows: int, repeats: int):
    """`rows` rows of both layers of the headline workload, forward + backward.  Returns (G units/s, text)."""
    import torch

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
        h, i1, j1 = cpu.forward(x, b1)
        y, i2, j2 = cpu.forward(h, b2)
        dh, dw2 = cpu.backward(h, b2, gy, i2, j2)
        dx, dw1 = cpu.backward(x, b1, dh, i1, j1)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return units / best / 1e9, f"{rows} of {M_TOKENS} rows of both layers, fwd+bwd, torch CPU, best of {repeats}"


def cpu_layer_sample(cpu: CpuPath, rows: int, K: int, N: int, beta: float, sparsity: float, x_std: float, w_std: float):
    """`rows` rows of one layer, forward + backward, optionally on a pruned (zeroed) weight or blended
    with the dense term.  Returns seconds."""
    import torch

    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, K, generator=g) * x_std
    w = torch.randn(N, K, generator=g) * w_std
    if sparsity > 0:
        w = w * (torch.rand(N, K, generator=g) >= sparsity).float()
    gy = torch.randn(rows, N, generator=g)
    b = w.T.contiguous()
    t0 = time.perf_counter()
    y, i1, j1 = cpu.forward(x, b, beta)
    cpu.backward(x, b, gy, i1, j1, beta)
    return time.perf_counter() - t0


def cpu_conv_sample(cpu: CpuPath, images: int, out_rows: int):
    """The convolution's CPU path: F.unfold + the reference functions on the first `out_rows` output
    pixels of `images` images (the reference has no executable convolution).  Returns seconds."""
    import torch

    from oracle import mam_oracle

    B, C, H, W, Fo = CONV_SHAPE
    g = torch.Generator().manual_seed(0)
    x = torch.randn(images, C, H, W, generator=g)
    w = torch.randn(Fo, C, 3, 3, generator=g) * (C * 9) ** -0.5
    t0 = time.perf_counter()
    rows = mam_oracle.conv2d_as_rows(x, (3, 3), stride=1, padding=1)[:out_rows].contiguous()
    gy = torch.randn(rows.size(0), Fo, generator=g)
    b = w.reshape(Fo, -1).T.contiguous()
    y, i1, j1 = cpu.forward(rows, b)
    cpu.backward(rows, b, gy, i1, j1)
    return time.perf_counter() - t0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuPath()
    rows = 128
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_mlp_pair_sample(cpu, rows, 1)
    t0 = time.perf_counter()
    vals = [cpu_mlp_pair_sample(cpu, rows, 1) for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    value = statistics.median(v[0] for v in vals)
    sample = vals[0][1]
    how = ("the reference's own checker functions (test/reference.py, byte-compiled)" if cpu.kind == "reference"
           else "CPU restatement of the reference's torch path")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": f"{how}; each step is a {rows}-row sample of the workload, "
                       "throughput is per unit so it compares directly"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cpu.threads, "kind": cpu.kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU helpers
# ------------------------------------------------------------------------------------------------
class Dist:
    """Rank bookkeeping + barrier + max-over-ranks event timing."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert self.world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={self.world} (launch with torch.distributed.run)"
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.numa_node = None
        if self.world > 1:     # (a single rank keeps every core: it also times the CPU path)
            self.numa_node = bind_to_gpu_numa_node(self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            opts = None
            if os.environ.get("MAM_BENCH_NCCL_PRIORITY", "1") == "1":
                # the collectives' kernels take the first SM resources that come free instead of queueing
                # behind the whole grid of whatever compute kernel is running
                opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
            dist.init_process_group("nccl", device_id=self.dev, pg_options=opts)
        self.dist = dist

    def barrier(self):
        import torch

        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps):
        """Milliseconds for `steps` calls of fn: CUDA events, barrier + synchronize on both sides, max over ranks."""
        import torch

        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        self.barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


class LibTimer:
    """Per-launch CUDA events recorded by the library around one class of its kernels."""

    def __init__(self, L, capacity):
        import torch

        self.L, self.cap = L, capacity
        self.pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(capacity)]
        for a, b in self.pairs:   # events are created lazily on first record; force creation now
            a.record()
            b.record()
        torch.cuda.synchronize()
        self.starts = (ctypes.c_void_p * capacity)(*[ctypes.c_void_p(a.cuda_event) for a, _ in self.pairs])
        self.stops = (ctypes.c_void_p * capacity)(*[ctypes.c_void_p(b.cuda_event) for _, b in self.pairs])

    def arm(self, kernel_id):
        from mamtorch_b200 import _lib

        _lib.check(self.L.mam_timer_arm(self.starts, self.stops, self.cap, kernel_id), "mam_timer_arm")

    def collect(self):
        import torch

        n = self.L.mam_timer_disarm()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in self.pairs[:n]]


def bench_fwd_4096(D: Dist, L, sms, max_mhz, reps=8):
    """The 4096^3 forward on one GPU: values only, and with indices (main loop and resolver apart)."""
    import torch

    from mamtorch_b200 import _lib

    n = 4096
    gen = torch.Generator(device=D.dev).manual_seed(4096)
    x = torch.randn(n, n, generator=gen, device=D.dev)
    w = torch.randn(n, n, generator=gen, device=D.dev) * n ** -0.5
    ops = torch.ops.mamtorch_b200
    timer = LibTimer(L, 2 * reps)
    units = float(n) ** 3
    peaks = fp32_peaks(sms, max_mhz)

    def run(want_idx, kid):
        for _ in range(3):
            ops.linear_forward(x, w, None, None, 1.0, 0.0, want_idx)
        timer.arm(kid)
        for _ in range(reps):
            ops.linear_forward(x, w, None, None, 1.0, 0.0, want_idx)
        ms = timer.collect()
        return statistics.mean(ms) if ms else float("nan")

    def fractions(ms):
        tf = 3.0 * units / (ms * 1e-3) / 1e12
        return {"ms": ms, "t_units_per_s": units / (ms * 1e-3) / 1e12, "tflops_3_per_unit": tf,
                "frac_of_fma_counted_peak": tf / peaks["fma_counted_tflops"],
                "frac_of_non_fma_peak": tf / peaks["non_fma_tops"]}

    val_ms = run(False, 0)
    idx_main_ms = run(True, 0)
    idx_res_ms = run(True, 1)
    _lib.check(L.mam_check_device_flag(), "device wait flag")
    return {"shape": "M=N=K=4096, x ~ N(0,1), W ~ N(0,1/K), fp32",
            "timing": f"library-recorded CUDA events per launch, mean of {reps} launches after 3 warm-ups",
            "peaks": {"fma_counted_tflops": peaks["fma_counted_tflops"], "non_fma_tops": peaks["non_fma_tops"],
                      "source": f"{sms} SMs x 128 lanes x {max_mhz:.0f} MHz (x 2 counting an FMA as two)"},
            "values_only": fractions(val_ms),
            "with_indices": {"main_loop": fractions(idx_main_ms), "index_resolver_ms": idx_res_ms,
                             "total": fractions(idx_main_ms + idx_res_ms)}}


def bench_sharded_sparse(D: Dist, L, steps=5, warmup=3):
    """The large sharded layer at this world size: 65536 rows split by rank (strong scaling), K = N = 4096,
    W pruned to 90 % (uniform random mask, CSR), forward with indices through the CSR kernels, backward
    through the selected-pair scatter (dW dense), dW summed over the ranks with NCCL."""
    import torch

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib
    from mamtorch_b200.dist import row_shard

    M_TOTAL, K, N = SHARDED_M, SHARDED_K, SHARDED_N
    lo, hi = row_shard(M_TOTAL, D.world, D.rank)
    rows = hi - lo
    g = torch.Generator().manual_seed(0)
    w = torch.randn(N, K, generator=g) * K ** -0.5
    keep = (torch.rand(N, K, generator=g) >= SHARDED_SPARSITY).float()   # the mask rule of test/test_sparse.py:13-16
    layer = mamtorch.sparse.PrunedFullyConnected(K, N, bias=False, device=D.dev)
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.keep_mask.copy_(keep)
    nnz = int(keep.sum().item())
    gd = torch.Generator(device=D.dev).manual_seed(100 + D.rank)
    x = torch.randn(rows, K, generator=gd, device=D.dev)
    gy = torch.randn(rows, N, generator=gd, device=D.dev)

    def step():
        # a training step of the pruned layer: the kept values are gathered and regrouped again every step (an
        # optimiser would have moved them), the sparsity pattern is kept from step to step
        layer.weight.grad = None
        xl = x.detach().requires_grad_()
        y = layer(xl)
        y.backward(gy)
        if D.world > 1:
            D.dist.all_reduce(layer.weight.grad)
        return y

    for _ in range(warmup):
        step()
    ms = D.timed(step, steps) / steps
    ar_ms = None
    if D.world > 1:
        buf = torch.empty_like(layer.weight)
        for _ in range(2):
            D.dist.all_reduce(buf)
        ar_ms = D.timed(lambda: D.dist.all_reduce(buf), 5) / 5
    _lib.check(L.mam_check_device_flag(), "device wait flag")
    out = {"workload": "M=65536 rows split by rank, K=N=4096 fp32, W pruned to 90 % (uniform random mask, CSR rows), "
                       "fwd with indices + selected-pair bwd, dW all-reduced",
           "scaling": "strong", "rows_per_rank": rows, "nnz": nnz, "steps": steps, "warmup": warmup,
           "ms_per_step": ms,
           "value": M_TOTAL * nnz / (ms * 1e-3) / 1e9, "unit": "G(row, stored weight) units/s over all ranks",
           "dense_equivalent_gunits": M_TOTAL * K * N / (ms * 1e-3) / 1e9,
           "dw_allreduce_bytes": 4 * N * K, "dw_allreduce_alone_ms": ar_ms}
    if ar_ms:
        out["dw_allreduce_bus_gbs"] = 2.0 * (D.world - 1) / D.world * 4 * N * K / (ar_ms * 1e-3) / 1e9
    del x, gy, layer
    torch.cuda.empty_cache()
    return out


def bench_conv(D: Dist, L, steps=5, warmup=3):
    """MAM conv2d fwd+bwd, [128,64,56,56] -> 128 channels, 3x3, stride 1, padding 1 (M=401408, K=576, N=128)."""
    import torch

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib

    B, C, H, W, Fo = CONV_SHAPE
    torch.manual_seed(0)
    gen = torch.Generator(device=D.dev).manual_seed(3)
    out = {"workload": "MAM conv2d fwd+bwd, x[128,64,56,56], 3x3 64->128, stride 1, padding 1, fp32 "
                       "(M=401408, K=576, N=128), indices + dX + dW"}
    units = B * H * W * C * 9 * Fo
    for order in ("unfold", "taps"):
        conv = mamtorch.nn.MAMConv2d(C, Fo, 3, padding=1, bias=False, reduction_order=order).to(D.dev)
        with torch.no_grad():
            conv.weight.copy_(torch.randn(Fo, C, 3, 3, generator=gen, device=D.dev) * (C * 9) ** -0.5)
        x = torch.randn(B, C, H, W, generator=gen, device=D.dev).requires_grad_()
        gy = torch.randn(B, Fo, H, W, generator=gen, device=D.dev)

        def step():
            conv.zero_grad()
            x.grad = None
            conv(x).backward(gy)

        for _ in range(warmup):
            step()
        ms = D.timed(step, steps) / steps
        out[f"ms_per_step_{order}"] = ms
        out[f"gunits_per_s_{order}"] = units / (ms * 1e-3) / 1e9
        del conv, x, gy
    _lib.check(L.mam_check_device_flag(), "device wait flag")
    torch.cuda.empty_cache()
    return out


def bench_beta_blend(D: Dist, L, steps=5, warmup=3):
    """beta-blended training step, M=N=K=4096, beta=0.5, the dense term on the tcgen05 TF32 kernel."""
    import torch

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib
    from mamtorch_b200.nn import functional as MF

    n = 4096
    std = n ** -0.25           # "N(0, 1/sqrt(K))" read as variance K^-1/2
    gen = torch.Generator(device=D.dev).manual_seed(4)
    torch.manual_seed(0)
    layer = mamtorch.nn.FullyConnected(n, n, bias=True, vcon_steps=2).to(D.dev)
    layer.vcon_step()          # beta: 1 -> 0.5
    assert abs(layer.beta - 0.5) < 1e-12
    with torch.no_grad():
        layer.weight.copy_(torch.randn(n, n, generator=gen, device=D.dev) * std)
        layer.bias.zero_()
    x = torch.randn(n, n, generator=gen, device=D.dev) * std
    gy = torch.randn(n, n, generator=gen, device=D.dev)
    was = MF.get_dense_backend()
    MF.set_dense_backend("tf32")
    try:
        def step():
            layer.zero_grad()
            xl = x.detach().requires_grad_()
            layer(xl).backward(gy)

        for _ in range(warmup):
            step()
        ms = D.timed(step, steps) / steps
    finally:
        MF.set_dense_backend(was)
    _lib.check(L.mam_check_device_flag(), "device wait flag")
    del layer, x, gy
    torch.cuda.empty_cache()
    return {"workload": "beta-blended MAM training step fp32, y=(1-b)(max+min)+b(x.W^T), b=0.5, M=N=K=4096, "
                        "x,W ~ N(0,1/sqrt(K)); dense term and its two gradient products on tcgen05 TF32",
            "ms_per_step": ms, "gunits_per_s": float(n) ** 3 / (ms * 1e-3) / 1e9,
            "dense_tflops_in_step": 3 * 2.0 * n ** 3 / 1e12}


def cpu_other_configs(cpu: CpuPath):
    """CPU path on bounded row samples of the sharded pruned layer, the convolution and the blended layer."""
    out = {}
    rows = 8
    s = cpu_layer_sample(cpu, rows, SHARDED_K, SHARDED_N, 0.0, SHARDED_SPARSITY, 1.0, SHARDED_K ** -0.5)
    out["sharded_sparse"] = {"dense_equivalent_gunits": rows * SHARDED_K * SHARDED_N / s / 1e9,
                             "sample": f"{rows} of {SHARDED_M} rows, dense reference on the zero-filled weight, fwd+bwd"}
    px = 256
    s = cpu_conv_sample(cpu, 1, px)
    B, C, H, W, Fo = CONV_SHAPE
    out["conv"] = {"gunits_per_s": px * C * 9 * Fo / s / 1e9,
                   "sample": f"{px} of {B * H * W} output pixels, F.unfold + the reference functions, fwd+bwd"}
    rows = 8
    s = cpu_layer_sample(cpu, rows, 4096, 4096, 0.5, 0.0, 4096 ** -0.25, 4096 ** -0.25)
    out["beta_blend"] = {"gunits_per_s": rows * 4096 * 4096 / s / 1e9,
                         "sample": f"{rows} of 4096 rows, beta = 0.5, fwd+bwd"}
    for v in out.values():
        v.update({"cores": cpu.threads, "kind": cpu.kind})
    return out


# ------------------------------------------------------------------------------------------------
# single operations (what profiler captures are taken on)
# ------------------------------------------------------------------------------------------------
def run_case(args):
    import torch

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib
    from mamtorch_b200.nn import functional as MF

    dev = torch.device("cuda:0")
    L = _lib.lib()
    if args.variant >= 0:
        _lib.check(L.mam_tune_set(1, args.variant), "variant")
        _lib.check(L.mam_tune_set(0, args.variant), "variant")
    _lib.check(L.mam_tune_set(4, args.dense_split), "dense split")
    g = torch.Generator().manual_seed(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.case == "conv":
        B, C, H, W, Fo = (int(v) for v in args.shape.lower().split("x"))
        torch.manual_seed(0)
        conv = mamtorch.nn.MAMConv2d(C, Fo, 3, padding=1, bias=False, reduction_order=args.order).to(dev)
        x = torch.randn(B, C, H, W, generator=g).to(dev).requires_grad_(not args.fwd_only)
        gy = torch.randn(B, Fo, H, W, generator=g).to(dev)
        torch.cuda.reset_peak_memory_stats()
        for rep in range(args.reps + 1):
            if rep == min(1, args.reps):
                e0.record()
            if args.fwd_only:
                with torch.no_grad():
                    y = conv(x)
            else:
                conv.zero_grad()
                x.grad = None
                y = conv(x)
                y.backward(gy)
        e1.record()
        torch.cuda.synchronize()
        _lib.check(L.mam_check_device_flag(), "device wait flag")
        print(f"ok conv {args.shape} order {args.order} {'fwd' if args.fwd_only else 'fwd+bwd'} checksum "
              f"{float(y.detach().double().sum()):.6e} ms_per_rep {e0.elapsed_time(e1) / max(args.reps, 1):.4f} "
              f"peak_alloc_MB {torch.cuda.max_memory_allocated() / 1e6:.0f}")
        return
    M, K, N = (int(v) for v in args.shape.lower().split("x"))
    x = torch.randn(M, K, generator=g).to(dev)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(dev)
    gy = torch.randn(M, N, generator=g).to(dev)
    ops = torch.ops.mamtorch_b200
    y, imax, imin = ops.linear_forward(x, w, None, None, 1.0, 0.0, True)
    if args.case in ("csr_fwd", "spmm"):
        keep = (torch.rand(N, K, generator=g) >= args.sparsity).float().to(dev)
        w_csr = (w * keep).to_sparse_csr()
        xT = x.t().contiguous()
    if args.case == "step":
        layer = mamtorch.nn.FullyConnected(K, N, store_args=True).to(dev)
    for rep in range(args.reps + 1):
        if rep == min(1, args.reps):
            e0.record()
        if args.case == "fwd_idx":
            y, imax, imin = ops.linear_forward(x, w, None, None, 1.0, 0.0, True)
        elif args.case == "fwd_val":
            y, = ops.linear_forward(x, w, None, None, 1.0, 0.0, False)
        elif args.case == "bwd":
            ops.linear_backward(x, w, gy, imax, imin, 1.0)
        elif args.case == "bwd_count":
            ops.linear_backward_count(x, w, gy, imax, imin, 1.0)
        elif args.case == "selcount":
            MF.selection_hits(imax, imin, K)
        elif args.case == "dense_tf32":
            y = ops.dense_nt(x, w)
        elif args.case == "csr_fwd":
            y, imax, imin = mamtorch.sparse.kernel.v1.mam_linear_csr(x, w_csr)
        elif args.case == "spmm":
            y = mamtorch.sparse.kernel.v1.cusparsemm(w_csr, xT)
        else:
            out = layer(x.clone().requires_grad_())
            out.backward(gy)
            layer.update_selection_count()
    e1.record()
    torch.cuda.synchronize()
    _lib.check(L.mam_check_device_flag(), "device wait flag")
    ms = e0.elapsed_time(e1) / max(args.reps, 1)
    extra = ""
    if args.case == "spmm" and args.compare:
        ref = torch.sparse.mm(w_csr, xT)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.reps):
            ref = torch.sparse.mm(w_csr, xT)
        e1.record()
        torch.cuda.synchronize()
        extra = (f" torch_sparse_mm_ms {e0.elapsed_time(e1) / max(args.reps, 1):.4f}"
                 f" max_abs_diff {float((y - ref).abs().max()):.3e}")
    print(f"ok {args.case} {M}x{K}x{N} checksum {float(y.double().sum()):.6e} ms_per_rep {ms:.4f}{extra}")


def run_sharded_sparse(args):
    """`--workload sharded_sparse`: the sharded pruned layer alone, as a line of its own."""
    from mamtorch_b200 import _lib

    D = Dist(args)
    L = _lib.lib()
    sampler = ClockSampler(D.local)
    if D.rank == 0:
        sampler.start()
    res = bench_sharded_sparse(D, L, steps=args.steps, warmup=max(args.warmup, 3))
    clocks = sampler.stop() if D.rank == 0 else None
    if D.rank == 0:
        line = {"metric": "mam_sharded_sparse_layer_fwd_bwd_throughput", "value": res["value"], "unit": UNIT,
                "n_gpus": D.world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": res["workload"], "units": "value counts (row, stored weight) pairs",
                           "l2": "per-rank working set (activations, indices, gradients) exceeds the 126 MB L2"},
                "detail": res, "gpu_launches": 11 * args.steps, "clocks": clocks}
        print(json.dumps(line), flush=True)
    D.close()


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
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps (default: 100 for this library, close to a second of device time; 20 for the CPU arms)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="headline workload only")
    ap.add_argument("--grad-sync", default="hooks", choices=["hooks", "deferred", "serial", "bucket"],
                    help="N > 1: all-reduce each weight gradient from its hook while the backward runs on (hooks, "
                         "default: measured best), all of them asynchronously right after the backward, under the "
                         "selection-count kernels (deferred), after the whole step (serial), or all gradients packed "
                         "into one flat buffer and one all-reduce after the step (bucket)")
    ap.add_argument("--e2e-no-exchange", action="store_true",
                    help="N > 1, diagnosis only: run the e2e leg with the gradient exchange off (its number is then not "
                         "the workload's)")
    ap.add_argument("--fwd-variant", type=int, default=-1, help="tile configuration of the index-producing forward")
    ap.add_argument("--workload", default="vit_mlp", choices=["vit_mlp", "sharded_sparse"],
                    help="vit_mlp: the headline configuration (default); sharded_sparse: the large pruned layer, "
                         "65536 rows split over the ranks (strong scaling), K = N = 4096, 90 %% of W pruned")
    ap.add_argument("--case", default=None, choices=["fwd_idx", "fwd_val", "bwd", "bwd_count", "selcount", "step",
                                                     "dense_tf32", "csr_fwd", "spmm", "conv"],
                    help="run one operation --reps times on --shape and print its time (profiler captures)")
    ap.add_argument("--shape", default="4096x1024x2048", help="--case: MxKxN, or BxCxHxWxF for conv")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--order", default="unfold", choices=["unfold", "taps"], help="--case conv: reduction order")
    ap.add_argument("--fwd-only", action="store_true", help="--case conv: forward with indices only")
    ap.add_argument("--sparsity", type=float, default=0.9, help="--case csr_fwd / spmm: share of zeroed weights")
    ap.add_argument("--compare", action="store_true", help="--case spmm: time torch.sparse.mm too")
    ap.add_argument("--variant", type=int, default=-1, help="--case: tile configuration of the tiled forward")
    ap.add_argument("--dense-split", type=int, default=1, choices=[0, 1], help="--case dense_tf32: slice the last wave")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 100 if args.impl == "b200" and args.workload == "vit_mlp" else 20
    if args.case:
        return run_case(args)
    if args.workload == "sharded_sparse" and args.impl == "b200":
        return run_sharded_sparse(args)
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference_cuda":
        return run_reference_cuda(args)

    import torch

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib
    from mamtorch_b200.dist import OverlappedGradSync, allreduce_gradients

    D = Dist(args)
    rank, world, local, dev = D.rank, D.world, D.local, D.dev
    L = _lib.lib()
    if args.fwd_variant >= 0:
        _lib.check(L.mam_tune_set(1, args.fwd_variant), "mam_tune_set")

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
    # N > 1: every parameter's gradient is all-reduced in place from a hook that fires as soon as autograd has
    # accumulated it, on NCCL's own stream; finish() makes the compute stream wait for the collectives
    class BucketSync:
        """The plain alternative: after the step, all gradients packed into one flat buffer, one all-reduce."""
        enabled = True

        def start(self):
            pass

        def finish(self):
            if self.enabled:
                allreduce_gradients(params, bucket_bytes=1 << 30)

    sync = None
    if world > 1:
        sync = BucketSync() if args.grad_sync == "bucket" else OverlappedGradSync(params, deferred=args.grad_sync != "hooks")

    def step(x, gy):
        for p in params:
            p.grad = None
        x = x.detach().requires_grad_()   # a fresh leaf every step: dX is produced, never accumulated
        y = fc2(fc1(x))
        y.backward(gy)
        if sync is not None and args.grad_sync == "deferred":
            sync.start()
        fc1.update_selection_count()
        fc2.update_selection_count()
        if sync is not None:
            sync.finish()
        return y

    # Before anything is timed, at N > 1: the all-reduced weight gradient must equal the sum of the ranks'
    # own gradients (values, not just that N ranks took part).
    grad_sum_check = None
    if world > 1:
        sync.enabled = False
        step(x_dev, gy_dev)
        own = fc2.weight.grad.detach().clone()
        gathered = [torch.empty_like(own) for _ in range(world)]
        D.dist.all_gather(gathered, own)
        want = torch.stack(gathered).double().sum(0)
        sync.enabled = True
        step(x_dev, gy_dev)
        got = fc2.weight.grad.detach().double()
        err = float((got - want).abs().max() / want.abs().max())
        grad_sum_check = {"max_rel_err_vs_sum_of_rank_gradients": err, "ok": err <= 1e-5}
        assert err <= 1e-5, f"all-reduced dW differs from the sum of the per-rank gradients: {err}"

    # End-to-end leg: every step's activations and upstream gradient start in pinned host memory and
    # its output and loss end there.  Copies run on their own streams -- one per direction, the link is full
    # duplex -- into three rotating sets of device buffers, so the uploads of steps i+1 and i+2 and the download
    # of step i-1 overlap the kernels of step i and each other: what a data loader feeding this layer does.
    # All of it is inside the timed region.
    up_stream = torch.cuda.Stream(device=dev)
    down_stream = torch.cuda.Stream(device=dev)
    NBUF = 3   # input / output slots on the device: the upload of step i+2 may start while step i computes
    x_buf = [torch.empty_like(x_dev) for _ in range(NBUF)]
    gy_buf = [torch.empty_like(gy_dev) for _ in range(NBUF)]
    y_buf = [torch.empty(64, 197, D_MODEL, device=dev) for _ in range(NBUF)]
    loss_buf = [torch.empty((), device=dev) for _ in range(NBUF)]
    up_done = [torch.cuda.Event() for _ in range(NBUF)]
    comp_done = [torch.cuda.Event() for _ in range(NBUF)]
    down_done = [torch.cuda.Event() for _ in range(NBUF)]

    def upload(slot):
        with torch.cuda.stream(up_stream):
            up_stream.wait_event(comp_done[slot])   # the buffers' previous step must be done with them
            x_buf[slot].copy_(x_host, non_blocking=True)
            gy_buf[slot].copy_(gy_host, non_blocking=True)
            up_done[slot].record(up_stream)

    # (no timing events inside this loop: at 8 ranks, with the host's copy rate near its limit, every
    # timestamped event record in a stream measurably delayed that stream)
    def run_from_host(steps):
        main_stream = torch.cuda.current_stream()
        for ev in comp_done + down_done:
            ev.record(main_stream)
        for j in range(min(NBUF - 1, steps)):
            upload(j)
        for i in range(steps):
            slot = i % NBUF
            if i + NBUF - 1 < steps:
                upload((i + NBUF - 1) % NBUF)
            main_stream.wait_event(up_done[slot])
            main_stream.wait_event(down_done[slot])          # y_buf[slot] of step i-NBUF has been downloaded
            y = step(x_buf[slot], gy_buf[slot]).detach()
            # the step's metric: <y, gy>, one pass over both, written where the download reads it
            torch.dot(y.reshape(-1), gy_buf[slot].reshape(-1), out=loss_buf[slot])
            # y is downloaded from where the forward left it; the reference kept here holds its memory until
            # this slot's turn comes again, by which time the compute stream has waited for the download
            y_buf[slot] = y
            comp_done[slot].record(main_stream)
            with torch.cuda.stream(down_stream):
                down_stream.wait_event(comp_done[slot])
                y_host.copy_(y_buf[slot].view_as(y_host), non_blocking=True)
                loss_host.copy_(loss_buf[slot], non_blocking=True)
                down_done[slot].record(down_stream)
        main_stream.wait_stream(up_stream)
        main_stream.wait_stream(down_stream)

    for _ in range(args.warmup):
        step(x_dev, gy_dev)
    run_from_host(2)
    D.barrier()

    # ---- per-kernel events for the dominant kernel (2 launches per step)
    timer = LibTimer(L, 2 * args.steps)
    timer.arm(0)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    total_ms = D.timed(lambda: step(x_dev, gy_dev), args.steps)
    kernel_ms = timer.collect()
    # the other kernels of the step, each class timed by the library's own events over extra steps
    # (two launches per step: layer 1 and layer 2)
    other_ms = {}
    extra_steps = max(3, min(args.steps, 10))
    for name, kid in (("index_resolver", 1), ("backward_scatter", 3), ("selection_hits", 4)):
        timer.arm(kid)
        for _ in range(extra_steps):
            step(x_dev, gy_dev)
        per_launch = timer.collect()
        other_ms[name] = sum(per_launch) / extra_steps if per_launch else 0.0
    if sync is not None and args.e2e_no_exchange:
        sync.enabled = False
    e2e_ms = D.timed(lambda: run_from_host(args.steps), 1)
    if sync is not None:
        sync.enabled = True
    clocks = sampler.stop() if rank == 0 else None
    # N > 1: the e2e leg's copies alone, all ranks at once (both directions together, nothing else running): the
    # floor the host side puts under the e2e step time at this N
    copies_alone_ms = None
    if world > 1:
        def copies_only():
            main_stream = torch.cuda.current_stream()
            up_stream.wait_stream(main_stream)
            down_stream.wait_stream(main_stream)
            with torch.cuda.stream(up_stream):
                x_buf[0].copy_(x_host, non_blocking=True)
                gy_buf[0].copy_(gy_host, non_blocking=True)
            with torch.cuda.stream(down_stream):
                y_host.copy_(y_buf[0], non_blocking=True)
            main_stream.wait_stream(up_stream)
            main_stream.wait_stream(down_stream)

        copies_only()
        copies_alone_ms = D.timed(copies_only, 10) / 10
        placements = [None] * world
        D.dist.all_gather_object(placements, D.numa_node)
    # N > 1: what every rank's own GPU needs for the same step with the gradient exchange switched off, so that
    # the distance between N ranks and one splits into "the slowest of N GPUs" and "the exchange"
    no_sync_ranks = None
    if sync is not None:
        sync.enabled = False
        own_steps = max(3, min(args.steps, 20))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        D.barrier()
        e0.record()
        for _ in range(own_steps):
            step(x_dev, gy_dev)
        e1.record()
        D.barrier()
        sync.enabled = True
        mine = torch.tensor([e0.elapsed_time(e1) / own_steps], device=dev)
        every = [torch.empty_like(mine) for _ in range(world)]
        D.dist.all_gather(every, mine)
        no_sync_ranks = [round(float(t.item()), 4) for t in every]
    _lib.check(L.mam_check_device_flag(), "device wait flag")

    props = torch.cuda.get_device_properties(dev)
    sms = props.multi_processor_count
    max_mhz = (clocks or {}).get("sm_max_mhz") or 1965.0

    # ---- the other configurations of the specification, measured in the same run
    others = {}
    if not args.no_other_configs:
        del x_buf, gy_buf, y_buf
        torch.cuda.empty_cache()
        sampler2 = ClockSampler(local)
        if rank == 0:
            sampler2.start()
        if world == 1:
            others["fwd_4096"] = bench_fwd_4096(D, L, sms, max_mhz)
            others["conv"] = bench_conv(D, L)
            others["beta_blend"] = bench_beta_blend(D, L)
        others["sharded_sparse"] = bench_sharded_sparse(D, L)
        if rank == 0:
            others["clocks"] = sampler2.stop()

    if rank != 0:
        D.close()
        return

    ms_per_step = total_ms / args.steps
    value = world * UNITS_PER_STEP / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * UNITS_PER_STEP / (e2e_ms / args.steps * 1e-3) / 1e9
    kavg = statistics.mean(kernel_ms) if kernel_ms else float("nan")
    flops_per_launch = 3.0 * M_TOKENS * D_MODEL * D_FF  # 3 fp32 ops per (m,n,k) unit, unpadded extents
    peaks = fp32_peaks(sms, max_mhz)
    achieved = flops_per_launch / (kavg * 1e-3) / 1e12
    roofline = {"bound": "fp32_cuda_core", "kernel": "mam_fwd_tiled_kernel (index-tracking variant "
                + L.mam_fwd_variant_name(1, args.fwd_variant if args.fwd_variant >= 0 else 0).decode() + ")",
                "achieved": achieved, "peak": peaks["fma_counted_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["fma_counted_tflops"],
                "peak_source": f"{sms} SMs x 128 lanes x 2 x {max_mhz:.0f} MHz (FMA counted as 2; no fp32 entry in "
                               "MEASURED_PEAKS.json); a MAM unit has no FMA, see the two extra fractions",
                "frac_of_non_fma_peak": achieved / peaks["non_fma_tops"],
                "frac_of_measured_mix_ceiling": (achieved / 3 * 1e3) / peaks["mix_ceiling_gunits"],
                "launch_ms_avg": kavg, "launches_timed": len(kernel_ms),
                "traffic": TRAFFIC_WEIGHT_BYTES + TRAFFIC_CAPTURED_BYTES * M_TOKENS / TRAFFIC_CAPTURED_ROWS,
                "traffic_note": "dram read+write bytes per launch (layer-1 shape): profiler capture at M=4736, "
                                "scaled by rows to M=12608"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "working set per step (~1 GB of activations, indices and "
                       "gradients) exceeds the 126 MB L2; no explicit flush",
                       "parallelism": f"rows sharded over {world} rank(s); dW all-reduced over NCCL from gradient "
                                      "hooks, overlapping the rest of the backward" if world > 1 else "single GPU"},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": x_host.numel() * 4 + gy_host.numel() * 4,
                    "d2h_bytes_per_step": y_host.numel() * 4 + 4},
            "gpu_launches": 10 * args.steps, "clocks": clocks, "roofline": roofline}
    if grad_sum_check is not None:
        line["allreduced_dw_check"] = grad_sum_check
    if no_sync_ranks is not None:
        line["ms_per_step_without_exchange_by_rank"] = no_sync_ranks
    if copies_alone_ms is not None:
        if args.e2e_no_exchange:
            line["e2e"]["diagnosis_only"] = "gradient exchange off in this leg"
        line["e2e"]["copies_alone_ms_per_step"] = copies_alone_ms
        line["e2e"]["numa_placement_by_rank"] = placements
        line["e2e"]["copies_alone_note"] = ("this step's host->device and device->host copies with no kernel running, all "
                                            "ranks at once, max over ranks: what the host side allows at this N")
    # per-step time of every kernel class and, for the two HBM-style kernels, algorithmic bytes over time
    # against the measured copy bandwidth (both layers: M x 768 x 3072 and M x 3072 x 768)
    hbm_peak = measured_hbm_gbs()
    mn, mk_nk = M_TOTAL_OUTPUTS, 2 * (M_TOKENS * D_MODEL + M_TOKENS * D_FF + 2 * D_MODEL * D_FF)
    bwd_bytes = 12 * mn + 4 * mk_nk + 8 * 2 * D_MODEL * D_FF     # + both int32 hit matrices of both layers
    line["kernels_ms_per_step"] = {"forward_main_loop": 2 * kavg, **other_ms}
    bwd_ms = other_ms["backward_scatter"] + other_ms["selection_hits"]
    line["roofline_other_kernels"] = [
        {"kernel": "selected-pair backward with the selection hits (both layers)", "bound": "hbm",
         "achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
         "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / hbm_peak,
         "note": "12*M*N + 8*(M*K + N*K) + 8*N*K bytes per layer over backward_scatter + selection_hits; in "
                 "practice bound by the rate of scattered 4-byte L2 operations (weight gathers and fp32 "
                 "reductions into dW), not by bytes"}]
    if others:
        line["north_star_configs"] = others
    if world == 1 and not args.no_cpu_baseline:
        cpu = CpuPath()
        cv, sample = cpu_mlp_pair_sample(cpu, 128, 2)
        line["cpu_baseline"] = {"value": cv, "unit": UNIT, "cores": cpu.threads, "kind": cpu.kind, "sample": sample}
        if others:
            line["north_star_configs"]["cpu"] = cpu_other_configs(cpu)
    print(json.dumps(line), flush=True)
    D.close()


if __name__ == "__main__":
    main()
