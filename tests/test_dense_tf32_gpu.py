"""tcgen05 TF32 product (the dense beta term) against an fp64 product: 1e-3 relative, the
tolerance the blended-training configuration states for this term."""
import ctypes

import numpy as np
import pytest
import torch

from mamtorch_b200 import _lib

pytestmark = pytest.mark.gpu

TF32_RTOL = 1e-3


def _dense(a, w, out=None, c_acc=1.0, c_out=0.0):
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = _lib.lib().mam_dense_tf32(p(a), p(w), p(out), c_acc, c_out, M, K, N,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "mam_dense_tf32")
    return out


def _close(got, ref):
    scale = float(ref.abs().max())
    np.testing.assert_allclose(got.cpu().double().numpy(), ref.cpu().numpy(), rtol=TF32_RTOL, atol=TF32_RTOL * scale)


@pytest.mark.parametrize("shape", [(128, 32, 128), (128, 256, 128), (256, 64, 384), (300, 100, 200),
                                   (1, 8, 1), (129, 36, 257), (1000, 768, 520), (4096, 4096, 512)])
def test_tf32_product_matches_fp64(shape, cuda):
    M, K, N = shape
    g = torch.Generator().manual_seed(M + K + N)
    a = torch.randn(M, K, generator=g).to(cuda)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda)
    out = _dense(a, w)
    torch.cuda.synchronize()
    assert _lib.lib().mam_check_device_flag() == 0
    _close(out, a.double() @ w.double().T)


def test_tf32_product_exact_on_small_integers(cuda):
    """Integers up to 2^10 are exact in TF32, sums stay exact in fp32: the result must be exact,
    which pins the operand layout (any mis-addressed row or k-slice shows up as a wrong integer)."""
    g = torch.Generator().manual_seed(1)
    M, K, N = 256, 160, 384
    a = torch.randint(-8, 9, (M, K), generator=g).float().to(cuda)
    w = torch.randint(-8, 9, (N, K), generator=g).float().to(cuda)
    out = _dense(a, w)
    assert torch.equal(out, a @ w.T)


@pytest.mark.parametrize("shape", [(1280, 96, 1280),    # 50 tiles: last wave cut in two
                                   (1000, 512, 700),    # 24 tiles: cut in four
                                   (4096, 256, 2560),   # 320 tiles = two whole waves + 24 tiles cut in four
                                   (3000, 64, 5000),    # 480 tiles, ragged edges, 36 tiles cut in four
                                   (2432, 128, 4096)])  # 304 tiles: two waves + 8 tiles cut in four
def test_tf32_tail_slices_give_the_same_bits_as_whole_tiles(shape, cuda):
    """Cutting the tiles of the last partial wave into column slices changes which SM computes an output, not
    how: every output still sums its K products in the same order, so the two forms agree bit for bit."""
    M, K, N = shape
    L = _lib.lib()
    g = torch.Generator().manual_seed(M + K + N)
    a = torch.randint(-8, 9, (M, K), generator=g).float().to(cuda)
    w = torch.randint(-8, 9, (N, K), generator=g).float().to(cuda)
    try:
        _lib.check(L.mam_tune_set(4, 0), "selector")
        whole = _dense(a, w)
        _lib.check(L.mam_tune_set(4, 1), "selector")
        sliced = _dense(a, w)
    finally:
        L.mam_tune_set(4, 1)
    torch.cuda.synchronize()
    assert L.mam_check_device_flag() == 0
    assert torch.equal(sliced, whole)
    assert torch.equal(sliced, a @ w.T)      # small integers: exact in TF32, pins rows, columns and k-slices
    ar = torch.randn(M, K, generator=g).to(cuda)
    wr = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda)
    base = torch.randn(M, N, generator=g).to(cuda)
    _close(_dense(ar, wr, out=base.clone(), c_acc=0.5, c_out=2.0), 2.0 * base.double() + 0.5 * (ar.double() @ wr.double().T))


def test_tf32_product_accumulates_into_output(cuda):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(200, 64, generator=g).to(cuda)
    w = torch.randn(130, 64, generator=g).to(cuda)
    base = torch.randn(200, 130, generator=g).to(cuda)
    out = _dense(a, w, out=base.clone(), c_acc=0.25, c_out=0.5)
    _close(out, 0.5 * base.double() + 0.25 * (a.double() @ w.double().T))


def test_unsupported_shapes_are_reported(cuda):
    a = torch.zeros(4, 6, device=cuda)
    w = torch.zeros(5, 6, device=cuda)
    out = torch.zeros(4, 5, device=cuda)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    assert _lib.lib().mam_dense_tf32(p(a), p(w), p(out), 1.0, 0.0, 4, 6, 5, None) == 2


@pytest.mark.parametrize("shape", [(1, 1), (33, 65), (4096, 768), (257, 1000), (5, 70001)])
def test_transpose2d_matches_torch(shape, cuda):
    """The transpose the dense term's gradient products use: bit-identical to torch's strided copy."""
    a = torch.randn(*shape, device=cuda)
    out = torch.ops.mamtorch_b200.transpose2d(a)
    assert out.is_contiguous() and torch.equal(out, a.t().contiguous())
    assert torch.equal(torch.ops.mamtorch_b200.transpose2d(a.t()), a.contiguous())   # strided input
