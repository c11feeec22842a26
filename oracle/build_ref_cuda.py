"""Builds the reference's own CUDA extensions for an on-device comparison.  Test/measurement
infrastructure only: nothing in the product path loads what this makes.

The sources are compiled where they lie in a checkout of the reference (default: the directory
named by MAMTORCH_REFERENCE_DIR); none of them is copied.  Outputs go to oracle/_ref/:

    mamtorch_kernel_v4.so   mamtorch/kernel/v4/csrc/{register_functions.cpp, cuda/*.cu}
                            ops mamtorch_kernel_v4::{fullyconnected, fullyconnected_fast, fullyconnected_backward}

Only the v4 generation (the reference module's default path) is built.  The v1 operators are left
out on purpose: for outputs whose extents are both multiples of 64 their host code returns buffers it
never wrote (mamtorch/kernel/v1/csrc/cuda/fullyconnected.cu:262-288), and indices of that kind must
not reach a backward kernel that uses them as addresses.

The flags follow the reference's setup.py (-O3 for both compilers, setup.py:33-41) with the device
architecture given explicitly (compute_100/sm_100), which is what TORCH_CUDA_ARCH_LIST=10.0 would
select.  The reference's build system itself is not run.  The libraries define the same operator
namespaces as this package's shim, so a process loads either them or `mamtorch_b200`, never both.

    python oracle/build_ref_cuda.py [--reference DIR] [--force]
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
GENERATIONS = ("v4",)


def lib_path(gen: str) -> str:
    return os.path.join(OUT, f"mamtorch_kernel_{gen}.so")


def _flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        inc += ["-I", p]
    defs = ["-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    return inc, defs, tlib


def build_generation(ref: str, gen: str, force: bool = False) -> str:
    csrc = os.path.join(ref, "mamtorch", "kernel", gen, "csrc")
    cpps = sorted(glob.glob(os.path.join(csrc, "*.cpp")))
    cus = sorted(glob.glob(os.path.join(csrc, "cuda", "*.cu")))
    if not cpps or not cus:
        raise FileNotFoundError(f"no sources under {csrc}")
    target = lib_path(gen)
    if not force and os.path.exists(target) and all(
            os.path.getmtime(s) <= os.path.getmtime(target) for s in cpps + cus):
        return target
    inc, defs, tlib = _flags()
    objdir = os.path.join(OUT, "obj_" + gen)
    os.makedirs(objdir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    jobs = []
    for s in cpps:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        jobs.append((o, ["g++", "-O3", "-std=c++17", "-fPIC", "-Wno-deprecated-declarations", *defs, *inc,
                         "-c", s, "-o", o]))
    for s in cus:
        o = os.path.join(objdir, "cuda_" + os.path.basename(s) + ".o")
        jobs.append((o, [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100,code=sm_100",
                         "--compiler-options", "-fPIC", "--expt-relaxed-constexpr", *defs, *inc, "-c", s, "-o", o]))
    # the torch headers make every translation unit take minutes: compile them side by side
    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
        list(pool.map(lambda j: subprocess.check_call(j[1]), jobs))
    objs = [o for o, _ in jobs]
    subprocess.check_call(["g++", "-shared", "-o", target, *objs, "-L", tlib, "-ltorch", "-ltorch_cpu", "-lc10",
                           "-ltorch_cuda", "-lc10_cuda", "-ltorch_python", "-L", "/usr/local/cuda/lib64", "-lcudart",
                           "-Wl,-rpath," + tlib])
    return target


def build(ref: str | None = None, force: bool = False):
    ref = ref or os.environ.get("MAMTORCH_REFERENCE_DIR", "")
    if not ref or not os.path.isdir(os.path.join(ref, "mamtorch", "kernel")):
        return []
    return [build_generation(ref, g, force) for g in GENERATIONS]


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="checkout of the reference (or MAMTORCH_REFERENCE_DIR)")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    built = build(a.reference, a.force)
    if not built:
        sys.exit("no reference checkout given: pass --reference DIR")
    print("\n".join(built))
