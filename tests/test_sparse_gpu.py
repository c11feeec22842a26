"""Pruned-weight (CSR) kernels against the dense oracle on the zero-filled weight, and the
cusparsemm operator against a dense product (the check of the reference's test/test_sparse.py:33-44)."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close
from oracle import c_oracle

pytestmark = pytest.mark.gpu


def _pruned(N, K, keep, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * K ** -0.5
    mask = (torch.rand(N, K, generator=g) >= 1 - keep).float()   # Bernoulli keep, as test/test_sparse.py:13-16
    return w, mask, g


# Shapes with fewer than 32 rows run the lane-per-entry kernel, the others the tiled kernels (rows of a
# on the lanes): ragged last stage (K % 64 != 0), ragged row/column tiles, nothing stored, everything
# stored (runs of 128 entry pairs per warp and stage, i.e. several staging batches), one stage only.
@pytest.mark.parametrize("shape,keep", [((70, 96, 45), 0.1), ((33, 257, 64), 0.5), ((9, 40, 20), 0.0),
                                        ((16, 64, 31), 1.0), ((300, 1024, 130), 0.1), ((5, 4096, 37), 0.02),
                                        ((64, 200, 70), 1.0), ((40, 130, 9), 0.0), ((129, 36, 65), 0.3),
                                        ((32, 64, 4), 0.5), ((260, 708, 131), 0.05)])
def test_csr_forward_equals_dense_on_zero_filled_weight(shape, keep, cuda):
    import mamtorch_b200 as mamtorch

    M, K, N = shape
    w, mask, g = _pruned(N, K, keep, M + K + N)
    x = torch.randn(M, K, generator=g)
    if keep == 0.1:
        x = torch.relu(x)                # zero activations: explicit zero products tie with pruned ones
        w[3] = -w[3].abs()               # a row whose stored products are all <= 0 against x >= 0
    wz = w * mask
    y_ref, imax_ref, imin_ref = c_oracle.forward(x.numpy(), wz.numpy(), b_is_nk=True)
    w_csr = mamtorch.sparse.kernel.v1.prune_to_csr(w.to(cuda), mask.to(cuda))
    y, imax, imin = mamtorch.sparse.kernel.v1.mam_linear_csr(x.to(cuda), w_csr)
    assert torch.equal(imax.cpu().long(), torch.from_numpy(imax_ref))
    assert torch.equal(imin.cpu().long(), torch.from_numpy(imin_ref))
    assert torch.equal(y.cpu(), torch.from_numpy(y_ref))
    yv, _, _ = mamtorch.sparse.kernel.v1.mam_linear_csr(x.to(cuda), w_csr, need_indices=False)
    assert torch.equal(yv, y)


@pytest.mark.parametrize("shape,keep", [((96, 512, 200), 0.1), ((45, 100, 33), 0.6), ((2048, 1024, 256), 0.1)])
def test_tiled_and_lane_per_entry_kernels_agree(shape, keep, cuda):
    """The two CSR forward entry points of the C ABI must give identical bits: with a workspace the
    tiled kernels run, without one the lane-per-entry kernel."""
    import ctypes

    from mamtorch_b200 import _lib

    L = _lib.lib()
    M, K, N = shape
    w, mask, g = _pruned(N, K, keep, 3 * M + K + N)
    x = torch.randn(M, K, generator=g).to(cuda)
    w_csr = (w * mask).to(cuda).to_sparse_csr()
    crow, col, val = w_csr.crow_indices().contiguous(), w_csr.col_indices().contiguous(), w_csr.values().contiguous()
    bias = torch.randn(N, generator=g).to(cuda)
    nnz = val.numel()
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    wsb = L.mam_csr_fwd_workspace_bytes(M, K, N, nnz)
    assert wsb > 0
    ws = torch.empty(wsb, dtype=torch.uint8, device=cuda)
    out = []
    for use_ws in (True, False):
        y = torch.empty(M, N, device=cuda)
        i1 = torch.empty(M, N, dtype=torch.int32, device=cuda)
        i2 = torch.empty_like(i1)
        _lib.check(L.mam_csr_fwd_ws_f32(p(x), p(crow), p(col), p(val), nnz, p(bias), p(y), p(i1), p(i2), M, K, N,
                                        p(ws) if use_ws else None, wsb if use_ws else 0, st), "mam_csr_fwd_ws_f32")
        yv = torch.empty(M, N, device=cuda)
        _lib.check(L.mam_csr_fwd_ws_f32(p(x), p(crow), p(col), p(val), nnz, p(bias), p(yv), None, None, M, K, N,
                                        p(ws) if use_ws else None, wsb if use_ws else 0, st), "mam_csr_fwd_ws_f32")
        assert torch.equal(y, yv)
        out.append((y, i1, i2))
    assert L.mam_check_device_flag() == 0
    for a, b in zip(*out):
        assert torch.equal(a, b)
    # a workspace that is too small or misaligned is refused, nothing is launched
    assert L.mam_csr_fwd_ws_f32(p(x), p(crow), p(col), p(val), nnz, None, p(out[0][0]), None, None, M, K, N,
                                p(ws), wsb - 1, st) == 3
    assert L.mam_csr_fwd_ws_f32(p(x), p(crow), p(col), p(val), nnz, None, p(out[0][0]), None, None, M, K, N,
                                ctypes.c_void_p(ws.data_ptr() + 8), wsb, st) == 3


def test_csr_layer_backward_gives_dense_weight_gradient(cuda):
    import mamtorch_b200 as mamtorch

    M, K, N = 64, 128, 48
    w, mask, g = _pruned(N, K, 0.1, 7)
    x = torch.randn(M, K, generator=g)
    gy = torch.randn(M, N, generator=g)
    bias = torch.randn(N, generator=g)
    wz = (w * mask)
    y_ref, imax_ref, imin_ref = c_oracle.forward(x.numpy(), wz.numpy(), b_is_nk=True, bias=bias.numpy())
    da_ref, dw_ref = c_oracle.backward(x.numpy(), wz.numpy(), gy.numpy(), imax_ref, imin_ref, b_is_nk=True)
    xd = x.to(cuda).requires_grad_()
    wd = wz.to(cuda).requires_grad_()
    bd = bias.to(cuda).requires_grad_()
    y, _, _ = mamtorch.sparse.kernel.v1.mam_linear_csr(xd, wd.detach().to_sparse_csr(), bd, dense_weight=wd)
    assert torch.equal(y.detach().cpu(), torch.from_numpy(y_ref))
    y.backward(gy.to(cuda))
    assert_grad_close(xd.grad.cpu().numpy(), da_ref)
    assert_grad_close(wd.grad.cpu().numpy(), dw_ref)   # dense: selected pruned positions get gradient too
    assert (wd.grad.cpu()[mask == 0] != 0).any()
    assert_grad_close(bd.grad.cpu().numpy(), gy.sum(0).numpy())


@pytest.mark.parametrize("layout", ["csr", "coo"])
def test_cusparsemm_matches_dense_product(layout, cuda):
    import mamtorch_b200 as mamtorch

    g = torch.Generator().manual_seed(0)
    N, K, Mc = 130, 257, 200
    a = torch.randn(N, K, generator=g) * (torch.rand(N, K, generator=g) > 0.9)
    b = torch.randn(K, Mc, generator=g)
    a_sp = a.to(cuda).to_sparse_csr() if layout == "csr" else a.to(cuda).to_sparse()
    c = mamtorch.sparse.kernel.v1.cusparsemm(a_sp, b.to(cuda))
    ref = a.double() @ b.double()
    np.testing.assert_allclose(c.cpu().numpy(), ref.numpy(), rtol=1e-5, atol=1e-5)


def test_sharded_pruned_layer_shape_equals_dense_kernels(cuda):
    """One rank's share of the large sharded configuration (M=65536 rows over 8 ranks = 8192, K=N=4096,
    90 % of W pruned): the CSR kernel must reproduce, bit for bit, what the dense kernels give on the
    zero-filled weight (which the oracle-pinned tests cover at small sizes)."""
    import mamtorch_b200 as mamtorch

    M, K, N = 8192, 4096, 4096
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).to(cuda)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda)
    mask = (torch.rand(N, K, generator=g) >= 0.9).float().to(cuda)
    wz = w * mask
    y, imax, imin = mamtorch.sparse.kernel.v1.mam_linear_csr(x, wz.to_sparse_csr())
    yd, imaxd, imind = torch.ops.mamtorch_b200.linear_forward(x, wz, None, None, 1.0, 0.0, True)
    assert torch.equal(y, yd) and torch.equal(imax, imaxd) and torch.equal(imin, imind)


def test_magnitude_pruned_layer_equals_dense_layer_on_zeroed_weight(cuda):
    """Layer-wise magnitude pruning as the reference does it (zero where |w| <= quantile(|w|, p),
    examples/vitb16_imagenet1k/pruning_utils.py:105-116), then the CSR layer against the dense MAM layer
    holding the zeroed weight: identical bits forward, gradients to rounding."""
    import mamtorch_b200 as mamtorch

    torch.manual_seed(21)
    dense = mamtorch.nn.FullyConnected(96, 70, store_args=True).to(cuda)
    p = 0.8
    pruned = mamtorch.sparse.PrunedFullyConnected.from_dense(dense, fraction=p)
    with torch.no_grad():   # what the reference's LMP does to the dense layer
        thr = torch.quantile(dense.weight.flatten().abs(), p)
        dense.weight[dense.weight.abs() <= thr] = 0
    assert abs(pruned.sparsity() - p) < 0.01
    assert torch.equal(pruned.weight.detach() * pruned.keep_mask, dense.weight.detach())
    g = torch.Generator().manual_seed(22)
    x = torch.relu(torch.randn(3, 41, 96, generator=g)).to(cuda)
    gy = torch.randn(3, 41, 70, generator=g).to(cuda)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, yb = pruned(xa), dense(xb)
    assert torch.equal(ya, yb)
    assert torch.equal(pruned.argmax, dense.argmax) and torch.equal(pruned.argmin, dense.argmin)
    ya.backward(gy)
    yb.backward(gy)
    assert_grad_close(xa.grad.cpu().numpy(), xb.grad.cpu().numpy())
    # the dense layer's gradient reaches pruned positions too; the pruned layer's is masked by the chain rule
    assert_grad_close(pruned.weight.grad.cpu().numpy(), (dense.weight.grad * pruned.keep_mask).cpu().numpy())
    assert_grad_close(pruned.bias.grad.cpu().numpy(), dense.bias.grad.cpu().numpy())
    # the CSR form is cached until the weight changes
    csr = pruned._weight_csr()
    assert pruned._weight_csr() is csr
    with torch.no_grad():
        pruned.weight.mul_(2.0)
    assert pruned._weight_csr() is not csr
    # one threshold for several layers (global magnitude pruning)
    other = torch.randn(50, 96, generator=g).to(cuda)
    thr_g = mamtorch.sparse.global_magnitude_threshold([pruned.weight, other], 0.5)
    both = torch.cat([pruned.weight.detach().abs().flatten(), other.abs().flatten()]).sort().values
    assert torch.equal(thr_g, both[int(0.5 * both.numel())])      # the reference's rule: sorted[int(p * n)]


def test_pruned_layer_inference_keeps_the_regrouped_weight_between_calls(cuda):
    """Inference calls on an unchanged weight reuse the scratch buffer's regrouped entries (only the activations
    are prepared again); results must not depend on that, whatever the row counts in between, and a changed
    weight or mask must be picked up."""
    import mamtorch_b200 as mamtorch

    torch.manual_seed(31)
    K, N = 320, 150
    dense = mamtorch.nn.FullyConnected(K, N, store_args=True).to(cuda)
    pruned = mamtorch.sparse.PrunedFullyConnected.from_dense(dense, fraction=0.85).eval()

    def reference(x):
        w = (pruned.weight.detach() * pruned.keep_mask)
        return torch.ops.mamtorch_b200.linear_forward(x, w, pruned.bias.detach(), None, 1.0, 0.0, True)

    g = torch.Generator().manual_seed(32)
    seen_ready = []
    for rows in (200, 200, 64, 500, 33, 8, 200):     # same, smaller, larger (scratch regrown), below 32 rows
        x = torch.relu(torch.randn(rows, K, generator=g)).to(cuda)
        with torch.no_grad():
            y = pruned(x)
        seen_ready.append(pruned._ws_key == ("values", pruned._csr_key))
        yr, imax, imin = reference(x)
        assert torch.equal(y, yr) and torch.equal(pruned.argmax, imax) and torch.equal(pruned.argmin, imin)
    assert all(seen_ready)
    ws_before = pruned._ws
    with torch.no_grad():
        pruned.weight.mul_(-1.5)                      # new weight: the kept entries are stale
        x = torch.randn(200, K, generator=g).to(cuda)
        y = pruned(x)
        yr, imax, imin = reference(x)
    assert torch.equal(y, yr) and torch.equal(pruned.argmax, imax) and torch.equal(pruned.argmin, imin)
    assert pruned._ws is ws_before                    # same buffer, rebuilt in place
    pruned.prune_(fraction=0.5)                       # new mask
    with torch.no_grad():
        y = pruned(x)
        yr, imax, imin = reference(x)
    assert torch.equal(y, yr) and torch.equal(pruned.argmax, imax)
    # through the C ABI: entries_ready on a workspace written by the plain call
    import ctypes

    import capi
    from mamtorch_b200 import _lib

    L = _lib.lib()
    csr = pruned._weight_csr()
    crow, col, val = csr.crow_indices().contiguous(), csr.col_indices().contiguous(), csr.values().contiguous()
    nnz = val.numel()
    need = L.mam_csr_fwd_workspace_bytes(300, K, N, nnz)
    ent = L.mam_csr_fwd_entries_bytes(K, N, nnz)
    assert 0 < ent < need and L.mam_csr_fwd_workspace_bytes(64, K, N, nnz) < need
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    outs = []
    for rows, ready in ((300, 0), (300, 1), (100, 1)):
        xx = torch.randn(rows, K, generator=torch.Generator().manual_seed(rows)).to(cuda)
        yy = torch.empty(rows, N, device=cuda)
        ia = torch.empty(rows, N, dtype=torch.int32, device=cuda)
        ib = torch.empty_like(ia)
        _lib.check(L.mam_csr_fwd_ws_ex_f32(p(xx), p(crow), p(col), p(val), nnz, None, p(yy), p(ia), p(ib), rows, K, N,
                                           p(ws), need, ready, capi._stream()), "mam_csr_fwd_ws_ex_f32")
        w = pruned.weight.detach() * pruned.keep_mask
        yr, imax, imin = torch.ops.mamtorch_b200.linear_forward(xx, w, None, None, 1.0, 0.0, True)
        assert torch.equal(yy, yr) and torch.equal(ia, imax) and torch.equal(ib, imin)


@pytest.mark.parametrize("shape,keep", [((130, 257, 200), 0.1), ((64, 64, 64), 1.0), ((1000, 700, 132), 0.02),
                                        ((33, 4100, 68), 0.3), ((256, 128, 1024), 0.0), ((9, 40, 20), 0.5)])
def test_tiled_spmm_matches_fp64_product_and_the_row_kernel(shape, keep, cuda):
    """cusparsemm's product through both C-ABI entry points: the tiled kernel (workspace given; it does not
    apply to the last shape, Mc < 64, where the call falls back) and the thread-per-output kernel."""
    import ctypes

    from mamtorch_b200 import _lib

    L = _lib.lib()
    N, K, Mc = shape
    g = torch.Generator().manual_seed(N + K + Mc)
    a = torch.randn(N, K, generator=g) * (torch.rand(N, K, generator=g) < keep)
    if keep == 0.1:
        a[5] = 0                                     # an empty row
        a[7] = torch.randn(K, generator=g)           # a full row: several staging batches in one stage
    b = torch.randn(K, Mc, generator=g).to(cuda)
    acsr = a.to(cuda).to_sparse_csr()
    crow, col, val = acsr.crow_indices().contiguous(), acsr.col_indices().contiguous(), acsr.values().contiguous()
    nnz = val.numel()
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    colp, valp = (col, val) if nnz else (crow, b)
    # the size query applies a work threshold (small or very sparse products are left to the row kernel);
    # the kernel itself is exercised here by handing it the workspace of a large dense-ish problem
    assert L.mam_spmm_csr_workspace_bytes(N, K, Mc, nnz) == 0
    big = L.mam_spmm_csr_workspace_bytes(4096, 4096, 4096, 4096 * 410)
    assert big > 0 and L.mam_spmm_csr_workspace_bytes(4096, 4096, 4096, 4096 * 40) == 0
    wsb = big
    ws = torch.empty(wsb, dtype=torch.uint8, device=cuda)
    c_t = torch.full((N, Mc), float("nan"), device=cuda)
    c_r = torch.full((N, Mc), float("nan"), device=cuda)
    _lib.check(L.mam_spmm_csr_ws_f32(p(crow), p(colp), p(valp), nnz, p(b), p(c_t), N, K, Mc, p(ws), wsb, st),
               "mam_spmm_csr_ws_f32")
    _lib.check(L.mam_spmm_csr_f32(p(crow), p(colp), p(valp), p(b), p(c_r), N, K, Mc, st), "mam_spmm_csr_f32")
    assert L.mam_check_device_flag() == 0
    ref = a.double() @ b.cpu().double()
    np.testing.assert_allclose(c_t.cpu().numpy(), ref.numpy(), rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(c_r.cpu().numpy(), ref.numpy(), rtol=1e-5, atol=1e-4)
