"""Child process of test_reference_cuda_gpu.py: runs the reference's OWN compiled CUDA operators
(oracle/_ref/mamtorch_kernel_v4.so, built from the reference's sources by oracle/build_ref_cuda.py) on the
cases stored in an .npz file and writes their results next to it.  It must be a process of its own: the
library defines the operator namespace mamtorch_kernel_v4, which mamtorch_b200's shim defines too.

    python tests/ref_cuda_worker.py <library.so> <cases.npz> <results.npz>
"""
import sys

import numpy as np
import torch


def main():
    so, cases_path, out_path = sys.argv[1:4]
    torch.ops.load_library(so)
    ops = torch.ops.mamtorch_kernel_v4
    dev = torch.device("cuda:0")
    cases = np.load(cases_path)
    out = {}
    n = int(cases["count"])
    for i in range(n):
        a = torch.from_numpy(cases[f"a{i}"]).to(dev)
        b = torch.from_numpy(cases[f"b{i}"]).to(dev)                   # [K, N], the operator's layout
        g = torch.from_numpy(cases[f"g{i}"]).to(dev)
        imax = torch.from_numpy(cases[f"imax{i}"]).to(dev)
        imin = torch.from_numpy(cases[f"imin{i}"]).to(dev)
        out[f"y_fast{i}"] = ops.fullyconnected_fast(a, b).cpu().numpy()
        y_idx, amax, amin = ops.fullyconnected(a, b)                      # approximate by design
        out[f"y_idx{i}"] = y_idx.cpu().numpy()
        out[f"amax{i}"] = amax.cpu().numpy()
        out[f"amin{i}"] = amin.cpu().numpy()
        # the reference's backward driven with the exact indices: they are valid addresses in [0, K)
        da, db = ops.fullyconnected_backward(a, b, g, imax, imin)
        out[f"da{i}"] = da.cpu().numpy()
        out[f"db{i}"] = db.cpu().numpy()
    torch.cuda.synchronize()
    np.savez(out_path, **out)


if __name__ == "__main__":
    main()
