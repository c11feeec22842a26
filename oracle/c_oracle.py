"""ctypes binding of the plain-C oracle (oracle/mam_oracle.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libmam_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "mam_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "_build/libmam_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.mam_oracle_threads.restype = ctypes.c_int
    return _lib


def _p(x):
    return x.ctypes.data_as(ctypes.c_void_p)


def threads() -> int:
    return int(_load().mam_oracle_threads())


def forward(a: np.ndarray, b: np.ndarray, b_is_nk: bool = False, bias=None):
    """a[M,K] f32; b[K,N] (or W[N,K] when b_is_nk) -> y f32, argmax int64, argmin int64."""
    lib = _load()
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = a.shape
    N = b.shape[0] if b_is_nk else b.shape[1]
    assert (b.shape[1] if b_is_nk else b.shape[0]) == K
    y = np.empty((M, N), np.float32)
    imax = np.empty((M, N), np.int64)
    imin = np.empty((M, N), np.int64)
    bp = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        bp = _p(bias)
    lib.mam_oracle_forward(_p(a), _p(b), ctypes.c_int(int(b_is_nk)), bp, _p(y), _p(imax), _p(imin),
                           ctypes.c_int64(M), ctypes.c_int64(K), ctypes.c_int64(N))
    return y, imax, imin


def backward(a, b, g, argmax, argmin, b_is_nk: bool = False):
    lib = _load()
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    g = np.ascontiguousarray(g, dtype=np.float32)
    argmax = np.ascontiguousarray(argmax, dtype=np.int64)
    argmin = np.ascontiguousarray(argmin, dtype=np.int64)
    M, K = a.shape
    N = g.shape[1]
    agrad = np.empty_like(a)
    bgrad = np.empty_like(b)
    lib.mam_oracle_backward(_p(a), _p(b), ctypes.c_int(int(b_is_nk)), _p(g), _p(argmax), _p(argmin),
                            _p(agrad), _p(bgrad), ctypes.c_int64(M), ctypes.c_int64(K), ctypes.c_int64(N))
    return agrad, bgrad
