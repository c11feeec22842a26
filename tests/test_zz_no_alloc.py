"""The allocation-free forward (mam_fwd_kn_static_f32) against the ordinary entry point.

Some hosts of this library cannot hand it a workspace: they run where device allocation is
forbidden or own no allocator at all.  For them one entry point keeps its scratch (the
K-contiguous copy of the weight operand) in a fixed buffer inside the library.  This file checks,
through the C ABI, that it returns exactly what mam_fwd_f32 returns -- on two calls in a row with
different operands, because the buffer is shared and keeps the previous call's contents -- and
that a problem too large for the buffer is refused with its own status code.  The file name sorts
last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

import capi
from mamtorch_b200 import _lib

pytestmark = pytest.mark.gpu


def _static_forward(a, b, want_idx=True):
    M, K = a.shape
    N = b.shape[1]
    y = torch.empty((M, N), dtype=torch.float32, device=a.device)
    imax = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_idx else None
    imin = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_idx else None
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    st = _lib.lib().mam_fwd_kn_static_f32(p(a), p(b), p(y), p(imax), p(imin), M, K, N,
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return st, y, imax, imin


def test_static_scratch_forward_matches_workspace_forward_twice(cuda):
    g = torch.Generator().manual_seed(42)
    shapes = [(300, 512, 260), (129, 96, 1000)]  # second call uses a differently shaped slice of the buffer
    for M, K, N in shapes:
        a = torch.randn(M, K, generator=g).to(cuda)
        b = (torch.randn(K, N, generator=g) * K ** -0.5).to(cuda)
        y_ref, imax_ref, imin_ref = capi.forward(a, b, capi.KN)
        st, y, imax, imin = _static_forward(a, b)
        assert st == 0, _lib.status_str(st)
        torch.cuda.synchronize()
        assert torch.equal(y, y_ref) and torch.equal(imax, imax_ref) and torch.equal(imin, imin_ref)
        st, yv, _, _ = _static_forward(a, b, want_idx=False)
        assert st == 0 and torch.equal(yv, y_ref)
    assert capi.device_flag_ok()


def test_static_scratch_limit_is_enforced(cuda):
    K, N = 2048, 1025  # K*N*4 just over the 8 MiB buffer
    a = torch.zeros((4, K), device=cuda)
    b = torch.zeros((K, N), device=cuda)
    st, _, _, _ = _static_forward(a, b)
    assert st == 7 and "static" in _lib.status_str(st)
