"""Parity at the benchmark's own sizes, where the CPU oracle cannot cover a whole problem in seconds:

  * forward: size-independent properties over every output plus sampled rows against the C oracle;
  * backward: dX of sampled rows against the C oracle (a row of dX depends on that row alone), dW against a
    float64 accumulate-scatter formed on the GPU from the same indices (torch `index_put_`, not this library);
  * selection hits: against `torch.bincount` over all outputs.

Tolerance for gradients: 1e-5 relative (conftest.assert_grad_close); values and indices bit-exact.
"""
import numpy as np
import pytest
import torch

import capi
from conftest import assert_grad_close
from oracle import c_oracle

pytestmark = pytest.mark.gpu


def _inputs(M, K, N, seed, cuda, x_std=1.0, w_std=None):
    g = torch.Generator(device=cuda).manual_seed(seed)
    a = torch.randn(M, K, generator=g, device=cuda) * x_std
    w = torch.randn(N, K, generator=g, device=cuda) * (K ** -0.5 if w_std is None else w_std)
    gy = torch.randn(M, N, generator=g, device=cuda)
    return a, w, gy


def _dw_fp64(a, gy, imax, imin, N, K):
    """dW[n,k] = sum over rows of gy[m,n] * a[m,k] for k in (argmax, argmin)[m,n], accumulated in float64."""
    M = a.size(0)
    dw = torch.zeros(N * K, dtype=torch.float64, device=a.device)
    cols = torch.arange(N, device=a.device)[None, :]
    step = 2048
    for m0 in range(0, M, step):
        sl = slice(m0, min(M, m0 + step))
        for idx in (imax[sl].long(), imin[sl].long()):
            contrib = gy[sl].double() * torch.gather(a[sl], 1, idx).double()
            dw.index_put_(((cols * K + idx).reshape(-1),), contrib.reshape(-1), accumulate=True)
    return dw.view(N, K)


@pytest.mark.parametrize("shape", [(12608, 768, 3072), (12608, 3072, 768), (4096, 4096, 4096)],
                         ids=["vit_layer1", "vit_layer2", "blend_4096"])
def test_full_size_forward_backward_and_hits(shape, cuda):
    M, K, N = shape
    std = 4096 ** -0.25 if shape[0] == 4096 else None
    a, w, gy = _inputs(M, K, N, 11 + K, cuda, x_std=1.0 if std is None else std, w_std=std)
    y, imax, imin = capi.forward(a, w, capi.NK)
    yv, _, _ = capi.forward(a, w, capi.NK, want_idx=False)
    assert capi.device_flag_ok()
    # forward: properties that hold at any size
    assert torch.equal(y, yv)
    assert int(imax.min()) >= 0 and int(imax.max()) < K and int(imin.min()) >= 0 and int(imin.max()) < K
    cols = torch.arange(N, device=cuda)[None, :].expand(M, N)
    pmax = torch.gather(a, 1, imax.long()) * w[cols, imax.long()]
    pmin = torch.gather(a, 1, imin.long()) * w[cols, imin.long()]
    assert torch.equal(y, pmax + pmin)
    del pmax, pmin, yv
    # forward + dX on sampled rows against the C oracle
    gs = torch.Generator().manual_seed(5)
    sample = torch.randperm(M, generator=gs)[:24].sort().values.to(cuda)
    a_s, w_c = a[sample].cpu().numpy(), w.cpu().numpy()
    y_ref, imax_ref, imin_ref = c_oracle.forward(a_s, w_c, b_is_nk=True)
    assert torch.equal(y[sample].cpu(), torch.from_numpy(y_ref))
    assert torch.equal(imax[sample].cpu().long(), torch.from_numpy(imax_ref))
    assert torch.equal(imin[sample].cpu().long(), torch.from_numpy(imin_ref))
    da, dw = capi.backward(a, w, gy, imax, imin, capi.NK)
    assert capi.device_flag_ok()
    da_ref, _ = c_oracle.backward(a_s, w_c, gy[sample].cpu().numpy(), imax_ref, imin_ref, b_is_nk=True)
    assert_grad_close(da[sample].cpu().numpy(), da_ref)
    # dW over all rows against the float64 scatter
    dw_ref = _dw_fp64(a, gy, imax, imin, N, K)
    scale = float(dw_ref.abs().max())
    err = float((dw.double() - dw_ref).abs().max())
    assert err <= 1e-5 * scale, f"dW differs from the float64 scatter: {err} vs scale {scale}"
    # selection hits over all outputs
    hmax, hmin = capi.selcount(imax, imin, K)
    want_max = torch.bincount((cols * K + imax.long()).reshape(-1), minlength=N * K).view(N, K)
    want_min = torch.bincount((cols * K + imin.long()).reshape(-1), minlength=N * K).view(N, K)
    assert torch.equal(hmax.long(), want_max) and torch.equal(hmin.long(), want_min)


def test_full_size_backward_with_hits_counted_on_the_way(cuda):
    """The backward entry point that also counts the hits, at the headline layer's size."""
    import ctypes

    from mamtorch_b200 import _lib

    M, K, N = 12608, 768, 3072
    a, w, gy = _inputs(M, K, N, 3, cuda)
    _, imax, imin = capi.forward(a, w, capi.NK)
    da0, dw0 = capi.backward(a, w, gy, imax, imin, capi.NK)
    da, dw = torch.empty_like(a), torch.empty_like(w)
    hmax = torch.zeros((N, K), dtype=torch.int32, device=cuda)
    hmin = torch.zeros((N, K), dtype=torch.int32, device=cuda)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = _lib.lib().mam_bwd_count_f32(p(a), p(w), capi.NK, p(gy), p(imax), p(imin), p(da), p(dw), p(hmax), p(hmin),
                                      1.0, M, K, N, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "mam_bwd_count_f32")
    assert capi.device_flag_ok()
    assert_grad_close(da.cpu().numpy(), da0.cpu().numpy())
    assert_grad_close(dw.cpu().numpy(), dw0.cpu().numpy())
    want_max, want_min = capi.selcount(imax, imin, K)
    assert torch.equal(hmax, want_max) and torch.equal(hmin, want_min)


def test_full_size_conv_backward(cuda):
    """MAM conv2d at the benchmark's size ([128,64,56,56], 3x3 64 -> 128, padding 1): the module's backward
    against the patch-row formulation -- dX of sampled images folded from the C oracle's row gradients, dW
    against the float64 scatter over all output pixels."""
    import mamtorch_b200 as mamtorch

    B, C, H, W, Fo = 128, 64, 56, 56, 128
    g = torch.Generator(device=cuda).manual_seed(21)
    torch.manual_seed(0)
    conv = mamtorch.nn.MAMConv2d(C, Fo, 3, padding=1, bias=False).to(cuda)
    with torch.no_grad():
        conv.weight.copy_(torch.randn(Fo, C, 3, 3, generator=g, device=cuda) * (C * 9) ** -0.5)
    x = torch.randn(B, C, H, W, generator=g, device=cuda).requires_grad_()
    gy = torch.randn(B, Fo, H, W, generator=g, device=cuda)
    y = conv(x)
    y.backward(gy)
    torch.cuda.synchronize()
    assert capi.device_flag_ok()
    K = C * 9
    w2d = conv.weight.detach().reshape(Fo, K)
    imax = conv.argmax.permute(0, 2, 3, 1).reshape(-1, Fo)
    imin = conv.argmin.permute(0, 2, 3, 1).reshape(-1, Fo)
    g2d = gy.permute(0, 2, 3, 1).reshape(-1, Fo)
    # dW: float64 scatter, patch rows formed image block by image block
    dw = torch.zeros(Fo * K, dtype=torch.float64, device=cuda)
    cols = torch.arange(Fo, device=cuda)[None, :]
    per = H * W
    for b0 in range(0, B, 8):
        rows = torch.nn.functional.unfold(x.detach()[b0:b0 + 8], 3, padding=1).transpose(1, 2).reshape(-1, K)
        sl = slice(b0 * per, (b0 + 8) * per)
        for idx in (imax[sl].long(), imin[sl].long()):
            contrib = g2d[sl].double() * torch.gather(rows, 1, idx).double()
            dw.index_put_(((cols * K + idx).reshape(-1),), contrib.reshape(-1), accumulate=True)
    dw = dw.view(Fo, K)
    scale = float(dw.abs().max())
    assert float((conv.weight.grad.reshape(Fo, K).double() - dw).abs().max()) <= 1e-5 * scale
    # dX of two images: row gradients from the C oracle, folded back with F.fold
    for b in (0, 77):
        rows = torch.nn.functional.unfold(x.detach()[b:b + 1], 3, padding=1).transpose(1, 2).reshape(-1, K)
        sl = slice(b * per, (b + 1) * per)
        y_ref, imax_ref, imin_ref = c_oracle.forward(rows.cpu().numpy(), w2d.cpu().numpy(), b_is_nk=True)
        assert torch.equal(y[b].permute(1, 2, 0).reshape(-1, Fo).cpu(), torch.from_numpy(y_ref))
        assert torch.equal(imax[sl].cpu().long(), torch.from_numpy(imax_ref))
        da_ref, _ = c_oracle.backward(rows.cpu().numpy(), w2d.cpu().numpy(), g2d[sl].cpu().numpy(), imax_ref, imin_ref,
                                      b_is_nk=True)
        dx_ref = torch.nn.functional.fold(torch.from_numpy(da_ref).T.unsqueeze(0).double(), (H, W), 3, padding=1)[0]
        assert_grad_close(x.grad[b].cpu().numpy(), dx_ref.numpy())


def test_nan_products_are_ignored(cuda):
    """The library's stated NaN rule: fp32 max/min return the operand that is a number, so a NaN product never
    becomes the maximum or minimum and never receives an index -- unlike torch.max / torch.min, which propagate
    NaN.  Rows without NaN are unaffected; a row whose products are ALL NaN yields index 0 (clamped) and an
    unspecified value."""
    M, K, N = 128, 96, 64
    g = torch.Generator().manual_seed(8)
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g)
    a[5, 17] = float("nan")
    a[9, 0] = float("nan")
    w[3, 40] = float("nan")
    y, imax, imin = capi.forward(a.to(cuda), w.to(cuda), capi.NK)
    yv, _, _ = capi.forward(a.to(cuda), w.to(cuda), capi.NK, want_idx=False)
    assert capi.device_flag_ok()
    # what the rule means: the same problem with every NaN product taken out of the running
    p = a[:, None, :] * w[None, :, :]                 # [M,N,K]
    nan = torch.isnan(p)
    pmax = torch.where(nan, torch.full_like(p, -float("inf")), p)
    pmin = torch.where(nan, torch.full_like(p, float("inf")), p)
    vmax, imax_ref = pmax.max(-1)
    vmin, imin_ref = pmin.min(-1)
    assert torch.equal(y.cpu(), vmax + vmin) and torch.equal(yv.cpu(), vmax + vmin)
    assert torch.equal(imax.cpu().long(), imax_ref) and torch.equal(imin.cpu().long(), imin_ref)
    assert not torch.isnan(y).any()
    picked_nan = torch.gather(nan, 2, imax.cpu().long()[..., None]) | torch.gather(nan, 2, imin.cpu().long()[..., None])
    assert not picked_nan.any()
