"""Runs one MAM operation on a given shape a few times: the small, bounded command that `ncu`
captures are taken on.

    python -m mamtorch_b200.profile_case --shape 4096x1024x2048 --op fwd_idx --reps 3

ops: fwd_idx (forward with indices: tiled kernel + index resolver), fwd_val (values only),
bwd (selected-pair backward), selcount, step (forward + backward + selection count of one layer
through the nn module), dense_tf32 (tcgen05 product of the beta term), csr_fwd (forward on a weight
pruned to `--sparsity`, CSR), spmm (the ordinary product c[N,M] = w_csr[N,K] . xT[K,M] behind `cusparsemm`;
with `--compare` also `torch.sparse.mm`, i.e. cuSPARSE, on the same operands), conv (forward + backward of
`MAMConv2d` 3x3, padding 1, on x[B,C,H,W] -> F channels, `--shape BxCxHxWxF`, `--order unfold|taps`: patch rows
or im2col-mode TMA; `--fwd-only` for the forward alone).  Inputs are seeded N(0,1)
activations and N(0,1/K) weights in [N,K] layout.  The last line reports the CUDA-event time per repetition
(the first repetition is not timed).
"""
import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="4096x1024x2048", help="MxKxN")
    ap.add_argument("--op", default="fwd_idx", choices=["fwd_idx", "fwd_val", "bwd", "selcount", "step", "dense_tf32", "csr_fwd", "spmm", "conv"])
    ap.add_argument("--order", default="unfold", choices=["unfold", "taps"], help="conv: reduction order / data path")
    ap.add_argument("--fwd-only", action="store_true", help="conv: forward with indices only")
    ap.add_argument("--sparsity", type=float, default=0.9, help="share of zeroed weights for csr_fwd / spmm")
    ap.add_argument("--compare", action="store_true", help="spmm: time torch.sparse.mm on the same operands too")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--variant", type=int, default=-1, help="tile configuration of the tiled forward (-1 auto)")
    ap.add_argument("--dense-split", type=int, default=1, choices=[0, 1],
                    help="dense_tf32: cut the tiles of the last partial wave into column slices (1, default) or not")
    args = ap.parse_args()
    if args.op == "conv":
        return conv_case(args)
    M, K, N = (int(v) for v in args.shape.lower().split("x"))

    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib
    from mamtorch_b200.nn import functional as MF

    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).to(dev)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(dev)
    gy = torch.randn(M, N, generator=g).to(dev)
    if args.variant >= 0:
        _lib.check(_lib.lib().mam_set_fwd_variant(1, args.variant), "variant")
        _lib.check(_lib.lib().mam_set_fwd_variant(0, args.variant), "variant")
    _lib.check(_lib.lib().mam_set_fwd_variant(4, args.dense_split), "dense split")
    ops = torch.ops.mamtorch_b200
    y, imax, imin = ops.linear_forward(x, w, None, None, 1.0, 0.0, True)
    if args.op in ("csr_fwd", "spmm"):
        keep = (torch.rand(N, K, generator=g) >= args.sparsity).float().to(dev)
        w_csr = (w * keep).to_sparse_csr()
        xT = x.t().contiguous()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rep in range(args.reps + 1):
        if rep == min(1, args.reps):
            e0.record()
        if args.op == "fwd_idx":
            y, imax, imin = ops.linear_forward(x, w, None, None, 1.0, 0.0, True)
        elif args.op == "fwd_val":
            y, = ops.linear_forward(x, w, None, None, 1.0, 0.0, False)
        elif args.op == "bwd":
            ops.linear_backward(x, w, gy, imax, imin, 1.0)
        elif args.op == "selcount":
            MF.selection_hits(imax, imin, K)
        elif args.op == "dense_tf32":
            y = ops.dense_nt(x, w)
        elif args.op == "csr_fwd":
            y, imax, imin = mamtorch.sparse.kernel.v1.mam_linear_csr(x, w_csr)
        elif args.op == "spmm":
            y = mamtorch.sparse.kernel.v1.cusparsemm(w_csr, xT)
        else:
            layer = mamtorch.nn.FullyConnected(K, N, store_args=True).to(dev)
            out = layer(x.clone().requires_grad_())
            out.backward(gy)
            layer.update_selection_count()
    e1.record()
    torch.cuda.synchronize()
    _lib.check(_lib.lib().mam_check_device_flag(), "device wait flag")
    ms = e0.elapsed_time(e1) / max(args.reps, 1)
    extra = ""
    if args.op == "spmm" and args.compare:
        ref = torch.sparse.mm(w_csr, xT)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.reps):
            ref = torch.sparse.mm(w_csr, xT)
        e1.record()
        torch.cuda.synchronize()
        extra = (f" torch_sparse_mm_ms {e0.elapsed_time(e1) / max(args.reps, 1):.4f}"
                 f" max_abs_diff {float((y - ref).abs().max()):.3e}")
    print(f"ok {args.op} {M}x{K}x{N} checksum {float(y.double().sum()):.6e} ms_per_rep {ms:.4f}{extra}")


def conv_case(args):
    import mamtorch_b200 as mamtorch
    from mamtorch_b200 import _lib

    B, C, H, W, Fo = (int(v) for v in args.shape.lower().split("x"))
    dev = torch.device("cuda:0")
    if args.variant >= 0:
        _lib.check(_lib.lib().mam_set_fwd_variant(1, args.variant), "variant")
    g = torch.Generator().manual_seed(0)
    torch.manual_seed(0)
    conv = mamtorch.nn.MAMConv2d(C, Fo, 3, padding=1, bias=False, reduction_order=args.order).to(dev)
    x = torch.randn(B, C, H, W, generator=g).to(dev).requires_grad_(not args.fwd_only)
    gy = torch.randn(B, Fo, H, W, generator=g).to(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
    _lib.check(_lib.lib().mam_check_device_flag(), "device wait flag")
    ms = e0.elapsed_time(e1) / max(args.reps, 1)
    print(f"ok conv {args.shape} order {args.order} {'fwd' if args.fwd_only else 'fwd+bwd'} checksum "
          f"{float(y.double().sum()):.6e} ms_per_rep {ms:.4f} peak_alloc_MB {torch.cuda.max_memory_allocated() / 1e6:.0f}")


if __name__ == "__main__":
    main()
