"""Backward and selection-count parity on the GPU through the C ABI."""
import numpy as np
import pytest
import torch

import capi
from conftest import assert_grad_close, golden_names, load_golden
from oracle import c_oracle, mam_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout", [capi.KN, capi.NK])
@pytest.mark.parametrize("name", [n for n in golden_names() if not n.startswith("blend")])
def test_golden_backward(name, layout, cuda):
    g = load_golden(name)
    a = torch.from_numpy(g["a"]).to(cuda)
    b = torch.from_numpy(np.ascontiguousarray(g["b"].T) if layout == capi.NK else g["b"]).to(cuda)
    grad = torch.from_numpy(g["g"]).to(cuda)
    imax = torch.from_numpy(g["argmax"]).to(torch.int32).to(cuda)
    imin = torch.from_numpy(g["argmin"]).to(torch.int32).to(cuda)
    da, db = capi.backward(a, b, grad, imax, imin, layout)
    db = db.T if layout == capi.NK else db
    assert_grad_close(da.cpu().numpy(), g["agrad"])
    assert_grad_close(db.cpu().numpy(), g["bgrad"])


def test_blend_scale(cuda):
    g = load_golden("blend_40x64x48")
    beta = float(g["beta"])
    a, b, grad = (torch.from_numpy(g[k]).to(cuda) for k in ("a", "b", "g"))
    imax = torch.from_numpy(g["argmax"]).to(torch.int32).to(cuda)
    imin = torch.from_numpy(g["argmin"]).to(torch.int32).to(cuda)
    da, db = capi.backward(a, b, grad, imax, imin, capi.KN, scale=1 - beta)
    da = da + beta * (grad @ b.T)
    db = db + beta * (a.T @ grad)
    assert_grad_close(da.cpu().numpy(), g["agrad"])
    assert_grad_close(db.cpu().numpy(), g["bgrad"])


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("shape", [(700, 768, 520), (33, 3000, 40), (2048, 64, 96), (300, 5, 257), (67, 1, 70)])
def test_random_backward_against_c_oracle(shape, mode, cuda):
    """mode 0 = the library's own choice; 1 = single kernel, the rows of da shared by a CTA (shared-memory
    atomics), dW by L2 reductions; 2 = two kernels (row-owned da, column-owned dW); 3 / 4 = one row of da per
    warp, lanes that name the same k merged by match + shuffle (3 also parks the row of a in shared memory).
    The shapes with K = 5 and K = 1 put many lanes of a warp on the same k."""
    M, K, N = shape
    gen = torch.Generator().manual_seed(M + K + N)
    a = torch.randn(M, K, generator=gen)
    w = torch.randn(N, K, generator=gen) * K ** -0.5
    grad = torch.randn(M, N, generator=gen)
    _, imax, imin = c_oracle.forward(a.numpy(), w.numpy(), b_is_nk=True)
    # a few coincident selections: the pair must then be counted twice
    imin[0, :] = imax[0, :]
    da_ref, dw_ref = c_oracle.backward(a.numpy(), w.numpy(), grad.numpy(), imax, imin, b_is_nk=True)
    from mamtorch_b200 import _lib
    _lib.check(_lib.lib().mam_tune_set(3, mode), "backward form")
    try:
        da, dw = capi.backward(a.to(cuda), w.to(cuda), grad.to(cuda),
                               torch.from_numpy(imax).to(torch.int32).to(cuda),
                               torch.from_numpy(imin).to(torch.int32).to(cuda), capi.NK)
        dak, dbk = capi.backward(a.to(cuda), w.T.contiguous().to(cuda), grad.to(cuda),
                                 torch.from_numpy(imax).to(torch.int32).to(cuda),
                                 torch.from_numpy(imin).to(torch.int32).to(cuda), capi.KN)
    finally:
        _lib.lib().mam_tune_set(3, 0)
    assert_grad_close(da.cpu().numpy(), da_ref)
    assert_grad_close(dw.cpu().numpy(), dw_ref)
    assert_grad_close(dak.cpu().numpy(), da_ref)
    assert_grad_close(dbk.T.cpu().numpy(), dw_ref)


def test_backward_counts_hits_on_the_way(cuda):
    import ctypes
    from mamtorch_b200 import _lib

    M, K, N = 3000, 768, 200
    gen = torch.Generator().manual_seed(9)
    a = torch.randn(M, K, generator=gen).to(cuda)
    w = (torch.randn(N, K, generator=gen) * K ** -0.5).to(cuda)
    grad = torch.randn(M, N, generator=gen).to(cuda)
    _, imax, imin = capi.forward(a, w, capi.NK)
    da_ref, dw_ref = capi.backward(a, w, grad, imax, imin, capi.NK)
    hmax_ref, hmin_ref = capi.selcount(imax, imin, K)
    da, dw = torch.empty_like(a), torch.empty_like(w)
    hmax = torch.zeros((N, K), dtype=torch.int32, device=cuda)
    hmin = torch.zeros((N, K), dtype=torch.int32, device=cuda)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    for _ in range(2):  # counts accumulate, gradients are overwritten
        st = _lib.lib().mam_bwd_count_f32(p(a), p(w), capi.NK, p(grad), p(imax), p(imin), p(da), p(dw), p(hmax), p(hmin),
                                          1.0, M, K, N, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        _lib.check(st, "mam_bwd_count_f32")
    assert torch.equal(hmax, 2 * hmax_ref) and torch.equal(hmin, 2 * hmin_ref)
    assert_grad_close(da.cpu().numpy(), da_ref.cpu().numpy())
    assert_grad_close(dw.cpu().numpy(), dw_ref.cpu().numpy())


@pytest.mark.parametrize("layout", [capi.NK, capi.KN])
@pytest.mark.parametrize("shape", [(3000, 768, 200), (1500, 3072, 96), (257, 40, 515), (64, 5, 33)])
def test_backward_with_hits_riding_on_the_dw_reductions(shape, layout, cuda):
    """mam_bwd_count_ws_f32 with scratch for the 16-byte {dW, max hits, min hits} records: one sweep, the same
    gradients (to rounding) and exactly the same hits as the gradient kernel followed by mam_selcount_i32 -- in
    both weight layouts, with both gradient kernels (K = 768 takes the row-per-warp form), hits accumulated
    into the caller's matrices over two calls."""
    import ctypes

    from mamtorch_b200 import _lib

    M, K, N = shape
    L = _lib.lib()
    gen = torch.Generator().manual_seed(M + K)
    a = torch.randn(M, K, generator=gen).to(cuda)
    w = (torch.randn(N, K, generator=gen) * K ** -0.5).to(cuda)
    grad = torch.randn(M, N, generator=gen).to(cuda)
    _, imax, imin = capi.forward(a, w, capi.NK)
    imin[0, :] = imax[0, :]          # coincident selections count for both sides
    b = w if layout == capi.NK else w.T.contiguous()
    da_ref, db_ref = capi.backward(a, b, grad, imax, imin, layout)
    hmax_ref, hmin_ref = capi.selcount(imax, imin, K)
    assert L.mam_bwd_count_workspace_bytes(1 << 24, K, N) == 0            # counts would no longer be exact
    assert L.mam_bwd_count_workspace_bytes(M, K, 1 << 22) == 0 or K < 4   # records beyond L2: second sweep advised
    need = ((K * N * 16 + 255) // 256) * 256
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    da, db = torch.empty_like(a), torch.empty_like(b)
    hmax = torch.zeros((N, K), dtype=torch.int32, device=cuda)
    hmin = torch.zeros((N, K), dtype=torch.int32, device=cuda)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        st = L.mam_bwd_count_ws_f32(p(a), p(b), layout, p(grad), p(imax), p(imin), p(da), 0, p(db), p(hmax), p(hmin),
                                    1.0, M, K, N, p(ws), need, stream)
        _lib.check(st, "mam_bwd_count_ws_f32")
    assert capi.device_flag_ok()
    assert torch.equal(hmax, 2 * hmax_ref) and torch.equal(hmin, 2 * hmin_ref)
    assert_grad_close(da.cpu().numpy(), da_ref.cpu().numpy())
    assert_grad_close(db.cpu().numpy(), db_ref.cpu().numpy())
    # scratch too small or misaligned is refused before anything is launched
    assert L.mam_bwd_count_ws_f32(p(a), p(b), layout, p(grad), p(imax), p(imin), p(da), 0, p(db), p(hmax), p(hmin),
                                  1.0, M, K, N, p(ws), need - 256, stream) == 3


@pytest.mark.parametrize("name", ["relu_pruned_64x96x64", "edge_128x160x128"])
def test_selection_count_golden(name, cuda):
    g = load_golden(name)
    imax = torch.from_numpy(g["argmax"]).to(torch.int32).to(cuda)
    imin = torch.from_numpy(g["argmin"]).to(torch.int32).to(cuda)
    K = g["a"].shape[1]
    hmax, hmin = capi.selcount(imax, imin, K)
    rmax, rmin = mam_oracle.selection_hits(torch.from_numpy(g["argmax"]), torch.from_numpy(g["argmin"]), K)
    assert torch.equal(hmax.cpu(), rmax) and torch.equal(hmin.cpu(), rmin)
    ind = (hmax > 0).int() + (hmin > 0).int()
    assert np.array_equal(ind.cpu().numpy(), g["max_selection_count"])


def test_selection_count_large(cuda):
    M, K, N = 5000, 3072, 300
    gen = torch.Generator().manual_seed(2)
    imax = torch.randint(0, K, (M, N), generator=gen, dtype=torch.int32)
    imin = torch.randint(0, K, (M, N), generator=gen, dtype=torch.int32)
    hmax, hmin = capi.selcount(imax.to(cuda), imin.to(cuda), K)
    rmax, rmin = mam_oracle.selection_hits(imax, imin, K)
    assert torch.equal(hmax.cpu(), rmax) and torch.equal(hmin.cpu(), rmin)
