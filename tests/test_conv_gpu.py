"""Patch (im2col) and fold (col2im) kernels of the MAM convolution and the transposed row-gradient
layout of the backward, through the C ABI, against torch's unfold / fold on the same inputs; then
the strided, padded module against the oracle's selected-product gradient."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import assert_grad_close
from mamtorch_b200 import _lib
from oracle import mam_oracle

import capi

pytestmark = pytest.mark.gpu

GEOMS = [  # B, C, H, W, kH, kW, sh, sw, ph, pw
    (2, 3, 7, 9, 3, 3, 1, 1, 1, 1),
    (1, 5, 8, 8, 3, 2, 2, 1, 0, 1),
    (3, 4, 11, 6, 1, 1, 1, 1, 0, 0),
    (2, 2, 10, 13, 5, 3, 2, 3, 2, 1),
    (1, 1, 4, 4, 4, 4, 1, 1, 0, 0),
    (4, 64, 14, 14, 3, 3, 1, 1, 1, 1),
]


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("geom", GEOMS)
def test_im2col_and_col2im_match_unfold_and_fold(geom, cuda):
    B, C, H, W, kH, kW, sh, sw, ph, pw = geom
    L = _lib.lib()
    g = torch.Generator().manual_seed(sum(geom))
    x = torch.randn(B, C, H, W, generator=g).to(cuda)
    Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
    M, K = B * Ho * Wo, C * kH * kW
    rows = torch.empty(M, K, device=cuda)
    _lib.check(L.mam_im2col_f32(_p(x), _p(rows), B, C, H, W, kH, kW, sh, sw, ph, pw, capi._stream()), "mam_im2col_f32")
    ref = torch.nn.functional.unfold(x, (kH, kW), padding=(ph, pw), stride=(sh, sw)).transpose(1, 2).reshape(M, K)
    assert torch.equal(rows, ref)
    # fold: the adjoint of unfold, fed with the transposed layout [K, M]
    cols = torch.randn(M, K, generator=g).to(cuda)
    dx = torch.empty(B, C, H, W, device=cuda)
    cols_t = cols.t().contiguous()
    _lib.check(L.mam_col2im_f32(_p(cols_t), _p(dx), B, C, H, W, kH, kW, sh, sw, ph, pw, capi._stream()), "mam_col2im_f32")
    want = torch.nn.functional.fold(cols.view(B, Ho * Wo, K).transpose(1, 2), (H, W), (kH, kW), padding=(ph, pw),
                                    stride=(sh, sw))
    assert_grad_close(dx.cpu().numpy(), want.cpu().numpy())


@pytest.mark.parametrize("shape", [(37, 20, 11), (256, 576, 128), (1000, 64, 7)])
def test_backward_transposed_row_gradients(shape, cuda):
    """MAM_DA_KM must hold exactly the transpose of what MAM_DA_MK holds for da (each CTA sums its own
    rows in the same order either way); dW goes through atomics in both and agrees to rounding."""
    M, K, N = shape
    L = _lib.lib()
    g = torch.Generator().manual_seed(M + K + N)
    a = torch.randn(M, K, generator=g).to(cuda)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda)
    gy = torch.randn(M, N, generator=g).to(cuda)
    _, imax, imin = capi.forward(a, w, capi.NK)
    da, dw = capi.backward(a, w, gy, imax, imin, capi.NK)
    da_t = torch.empty(K, M, device=cuda)
    dw2 = torch.empty_like(w)
    _lib.check(L.mam_bwd_count_ex_f32(_p(a), _p(w), capi.NK, _p(gy), _p(imax), _p(imin), _p(da_t), 1, _p(dw2), None, None,
                                      1.0, M, K, N, capi._stream()), "mam_bwd_count_ex_f32")
    assert_grad_close(da_t.t().cpu().numpy(), da.cpu().numpy())
    assert_grad_close(dw2.cpu().numpy(), dw.cpu().numpy())
    assert L.mam_bwd_count_ex_f32(_p(a), _p(w), capi.NK, _p(gy), _p(imax), _p(imin), _p(da_t), 2, _p(dw2), None, None,
                                  1.0, M, K, N, capi._stream()) == 1


@pytest.mark.parametrize("geom", [GEOMS[0], GEOMS[1], GEOMS[3], GEOMS[5]])
def test_conv_backward_from_the_input_equals_backward_on_patch_rows(geom, cuda):
    """mam_conv_bwd_f32 reads the selected activations from x; mam_bwd_count_ex_f32 reads them from the patch
    rows: same row gradients (same summation order per CTA), dW to rounding (atomics)."""
    B, C, H, W, kH, kW, sh, sw, ph, pw = geom
    L = _lib.lib()
    g = torch.Generator().manual_seed(7 + sum(geom))
    x = torch.randn(B, C, H, W, generator=g).to(cuda)
    Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
    M, K, N = B * Ho * Wo, C * kH * kW, 9
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda)
    gy = torch.randn(M, N, generator=g).to(cuda)
    rows = torch.empty(M, K, device=cuda)
    _lib.check(L.mam_im2col_f32(_p(x), _p(rows), B, C, H, W, kH, kW, sh, sw, ph, pw, capi._stream()), "mam_im2col_f32")
    _, imax, imin = capi.forward(rows, w, capi.NK)
    ct_a, dw_a = torch.empty(K, M, device=cuda), torch.empty_like(w)
    ct_b, dw_b = torch.empty(K, M, device=cuda), torch.empty_like(w)
    _lib.check(L.mam_bwd_count_ex_f32(_p(rows), _p(w), capi.NK, _p(gy), _p(imax), _p(imin), _p(ct_a), 1, _p(dw_a), None,
                                      None, 0.5, M, K, N, capi._stream()), "mam_bwd_count_ex_f32")
    _lib.check(L.mam_conv_bwd_f32(_p(x), _p(w), _p(gy), _p(imax), _p(imin), _p(ct_b), _p(dw_b), 0.5, B, C, H, W, kH, kW,
                                  sh, sw, ph, pw, N, capi._stream()), "mam_conv_bwd_f32")
    assert_grad_close(ct_b.cpu().numpy(), ct_a.cpu().numpy())
    assert_grad_close(dw_b.cpu().numpy(), dw_a.cpu().numpy())


def test_strided_padded_conv_module_gradients(cuda):
    import mamtorch_b200 as mamtorch

    torch.manual_seed(11)
    conv = mamtorch.nn.MAMConv2d(6, 5, (3, 2), stride=(2, 1), padding=(1, 0)).to(cuda)
    x = torch.randn(3, 6, 9, 7, generator=torch.Generator().manual_seed(12)).to(cuda).requires_grad_()
    y = conv(x)
    y_ref, imax_ref, imin_ref = mam_oracle.mam_conv2d_forward(x.detach().cpu(), conv.weight.detach().cpu(),
                                                              conv.bias.detach().cpu(), stride=(2, 1), padding=(1, 0))
    assert torch.equal(y.detach().cpu(), y_ref)
    assert torch.equal(conv.argmax.cpu().long(), imax_ref) and torch.equal(conv.argmin.cpu().long(), imin_ref)
    gy = torch.randn(y.shape, generator=torch.Generator().manual_seed(13)).to(cuda)
    y.backward(gy)
    xw = x.detach().cpu().requires_grad_()
    ww = conv.weight.detach().cpu().requires_grad_()
    rows = mam_oracle.conv2d_as_rows(xw, (3, 2), stride=(2, 1), padding=(1, 0))
    wf = ww.reshape(5, -1)
    im = imax_ref.permute(0, 2, 3, 1).reshape(-1, 5)
    imn = imin_ref.permute(0, 2, 3, 1).reshape(-1, 5)
    r = torch.arange(rows.shape[0])[:, None].expand_as(im)
    c = torch.arange(5)[None, :].expand_as(im)
    out = rows[r, im] * wf[c, im] + rows[r, imn] * wf[c, imn]
    (out * gy.cpu().permute(0, 2, 3, 1).reshape(-1, 5)).sum().backward()
    assert_grad_close(x.grad.cpu().numpy(), xw.grad.numpy())
    assert_grad_close(conv.weight.grad.cpu().numpy(), ww.grad.numpy())
    assert_grad_close(conv.bias.grad.cpu().numpy(), gy.sum((0, 2, 3)).cpu().numpy())
