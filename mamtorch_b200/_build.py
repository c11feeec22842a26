"""In-tree build of the two native pieces of this package.

  libmam_b200.so  the CUDA kernels behind a plain C ABI (nvcc, sm_100a only)
  _C.so           the PyTorch operator shim (g++), linked against libmam_b200.so

Both land next to this file so they travel with the source tree; nothing is installed into
site-packages and nothing is built lazily at import time on a machine without the sources.
nvcc cross-compiles for sm_100a without a GPU, so `build()` works on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmam_b200.so")
SHIM = os.path.join(HERE, "_C.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "--compiler-options", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels of mamtorch_b200 cannot be built")


def _stale(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources(exts):
    out = [os.path.join(HERE, "..", "include", "mam_b200.h"), os.path.join(HERE, "..", "include", "mam_b200_tuning.h")]
    for f in sorted(os.listdir(CSRC)):
        if f.endswith(exts):
            out.append(os.path.join(CSRC, f))
    return out


def build_lib(force: bool = False, verbose: bool = False) -> str:
    srcs = _sources((".cu", ".cuh"))
    if force or _stale(LIB, srcs):
        cus = [s for s in srcs if s.endswith(".cu")]
        cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", LIB, *cus]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.check_call(cmd, cwd=CSRC)
    return LIB


def build_shim(force: bool = False) -> str:
    src = os.path.join(CSRC, "torch_shim.cpp")
    if force or _stale(SHIM, [src, os.path.join(HERE, "..", "include", "mam_b200.h"), LIB]):
        import torch
        from torch.utils import cpp_extension as ce

        inc = []
        for p in ce.include_paths("cuda"):
            inc += ["-I", p]
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cxx = "g++"
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-o", SHIM, src, *inc,
               "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
               "-L", tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
               "-L", HERE, "-l:libmam_b200.so",
               "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib, "-Wno-deprecated-declarations"]
        subprocess.check_call(cmd, cwd=CSRC)
    return SHIM


def build(force: bool = False) -> None:
    build_lib(force)
    build_shim(force)


if __name__ == "__main__":
    build(force="--force" in sys.argv)
    print(LIB)
    print(SHIM)
