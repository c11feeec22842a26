"""Test-side helper: calls the C ABI (include/mam_b200.h) directly through ctypes on torch CUDA
tensors, the way a non-PyTorch host would, so the parity tests exercise the boundary itself."""
import ctypes

import torch

from mamtorch_b200 import _lib

KN, NK = _lib.MAM_B_KN, _lib.MAM_B_NK


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def set_variant(with_idx: bool, variant: int):
    _lib.check(_lib.lib().mam_tune_set(int(with_idx), variant), "mam_tune_set")


def forward(a, b, layout=KN, bias=None, dense=None, blend=False, alpha=1.0, beta=0.0, want_idx=True):
    L = _lib.lib()
    M, K = a.shape
    N = b.shape[1] if layout == KN else b.shape[0]
    y = torch.empty((M, N), dtype=torch.float32, device=a.device)
    amax = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_idx else None
    amin = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_idx else None
    wsb = L.mam_fwd_workspace_bytes(M, K, N, layout, int(want_idx))
    ws = torch.empty((max(wsb, 1),), dtype=torch.uint8, device=a.device)
    st = L.mam_fwd_f32(_ptr(a), _ptr(b), layout, _ptr(bias), _ptr(dense), int(blend), alpha, beta,
                       _ptr(y), _ptr(amax), _ptr(amin), M, K, N, _ptr(ws) if wsb else None, wsb, _stream())
    _lib.check(st, "mam_fwd_f32")
    return y, amax, amin


def backward(a, b, g, amax, amin, layout=KN, scale=1.0):
    L = _lib.lib()
    M, K = a.shape
    N = g.shape[1]
    da = torch.empty_like(a)
    db = torch.empty_like(b)
    st = L.mam_bwd_f32(_ptr(a), _ptr(b), layout, _ptr(g), _ptr(amax), _ptr(amin), _ptr(da), _ptr(db),
                       scale, M, K, N, _stream())
    _lib.check(st, "mam_bwd_f32")
    return da, db


def selcount(amax, amin, K):
    L = _lib.lib()
    M, N = amax.shape
    hmax = torch.zeros((N, K), dtype=torch.int32, device=amax.device)
    hmin = torch.zeros((N, K), dtype=torch.int32, device=amax.device)
    _lib.check(L.mam_selcount_i32(_ptr(amax), _ptr(amin), _ptr(hmax), _ptr(hmin), M, K, N, _stream()),
               "mam_selcount_i32")
    return hmax, hmin


def device_flag_ok():
    return _lib.lib().mam_check_device_flag() == 0
