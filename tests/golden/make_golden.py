"""Generates the known-answer fixtures in this folder by running the UNMODIFIED reference checker
(`test/reference.py` of SSIGPRO/mamtorch) on seeded inputs.  Run where the reference checkout is
available:

    python tests/golden/make_golden.py /path/to/mamtorch

Each case is written as `<name>.npz` holding the inputs (so no test depends on a random-number
generator reproducing them) and the reference outputs: y, argmax, argmin (int64 as the reference
returns them), agrad, bgrad for an upstream gradient, and where marked the result of the module's
selection-count update executed literally as `mamtorch/nn/v4/fullyconnected.py:125-129` writes it.
The reference repository itself ships no golden vectors; these files are the pin.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def cases():
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)
    ri = lambda lo, hi, *s: torch.randint(lo, hi + 1, s, generator=g).float()
    out = {}
    # plain random, ragged sizes (no multiple of any tile)
    out["random_37x70x29"] = dict(a=rn(37, 70), b=rn(70, 29), g=rn(37, 29))
    # small-integer values: many exact ties, +0/-0 products, coincident max/min
    out["ties_int_33x45x65"] = dict(a=ri(-2, 2, 33, 45), b=ri(-2, 2, 45, 65), g=rn(33, 65))
    # ReLU'd activations and pruned weights: zero products dominate, the tie rule picks the index
    a = torch.relu(rn(64, 96))
    b = rn(96, 64) * (torch.rand(96, 64, generator=g) > 0.6)
    out["relu_pruned_64x96x64"] = dict(a=a, b=b, g=rn(64, 64), count=True)
    # every product negative / every product positive / every product zero
    out["all_negative_17x40x23"] = dict(a=rn(17, 40).abs() + 0.1, b=-(rn(40, 23).abs() + 0.1), g=rn(17, 23))
    out["all_positive_17x40x23"] = dict(a=-(rn(17, 40).abs() + 0.1), b=-(rn(40, 23).abs() + 0.1), g=rn(17, 23))
    out["all_zero_9x12x10"] = dict(a=torch.zeros(9, 12), b=rn(12, 10), g=rn(9, 10))
    # degenerate extents
    out["k1_20x1x30"] = dict(a=rn(20, 1), b=rn(1, 30), g=rn(20, 30))
    out["m1n1_1x50x1"] = dict(a=rn(1, 50), b=rn(50, 1), g=rn(1, 1))
    out["k5_65x5x63"] = dict(a=rn(65, 5), b=rn(5, 63), g=rn(65, 63))
    # sizes around one 64/128 tile edge, K a multiple of 4 but not of 32
    out["edge_129x100x127"] = dict(a=rn(129, 100), b=rn(100, 127), g=rn(129, 127))
    out["edge_128x160x128"] = dict(a=rn(128, 160), b=rn(160, 128), g=rn(128, 128), count=True)
    # beta-blended call with bias (kernel v2/v3 op semantics)
    out["blend_40x64x48"] = dict(a=rn(40, 64), b=rn(64, 48), g=rn(40, 48), bias=rn(48), beta=0.37)
    # first benchmark configuration: x[256,512]~N(0,1), W[256,512]~N(0,1/512), bias 0, seed 0
    g0 = torch.Generator().manual_seed(0)
    x = torch.randn(256, 512, generator=g0)
    W = torch.randn(256, 512, generator=g0) * 512 ** -0.5
    gr = torch.randn(256, 256, generator=g0)
    out["config1_256x512x256"] = dict(a=x, b=W.T.contiguous(), g=gr, bias=torch.zeros(256), beta=0.0)
    return out


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MAMTORCH_REFERENCE_DIR")
    if not ref_root:
        raise SystemExit("usage: make_golden.py /path/to/mamtorch   (or set MAMTORCH_REFERENCE_DIR)")
    sys.path.insert(0, os.path.join(ref_root, "test"))
    from reference import fullyconnected_backward_reference, fullyconnected_reference

    for name, c in cases().items():
        a, b, g = c["a"], c["b"], c["g"]
        beta = c.get("beta", 0.0)
        bias = c.get("bias", None)
        y, imax, imin = fullyconnected_reference(a, b, 0.0 if bias is None else bias, beta)
        agrad, bgrad = fullyconnected_backward_reference(a, b, g, imax, imin, beta)
        rec = dict(a=a.numpy(), b=b.numpy(), g=g.numpy(), beta=np.float64(beta),
                   y=y.numpy(), argmax=imax.numpy(), argmin=imin.numpy(),
                   agrad=agrad.numpy(), bgrad=bgrad.numpy())
        if bias is not None:
            rec["bias"] = bias.numpy()
        if c.get("count"):
            # literal transcription of update_selection_count (nn/v4/fullyconnected.py:125-129)
            cnt = torch.zeros((b.shape[1], b.shape[0]), dtype=torch.int32)
            for arg in (imax, imin):
                num_rows, num_cols = arg.shape
                col_indices = torch.arange(num_cols).repeat(num_rows)
                cnt[col_indices, arg.flatten()] += 1
            rec["max_selection_count"] = cnt.numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        print(name, tuple(a.shape), tuple(b.shape), "ties(max==min idx):", int((imax == imin).sum()))


if __name__ == "__main__":
    main()
