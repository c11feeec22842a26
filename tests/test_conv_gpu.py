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


DIRECT_GEOMS = GEOMS + [
    (2, 8, 12, 16, 3, 3, 1, 1, 1, 1),      # W % 4 == 0: the tile goes out four floats per reduction
    (2, 4, 13, 12, 3, 3, 2, 2, 1, 1),      # stride 2, several tiles of output rows per image
    (1, 3, 40, 8, 5, 1, 1, 1, 2, 0),       # more output rows than one tile holds, tall kernel
    (3, 2, 6, 5, 2, 2, 1, 1, 3, 3),        # padding wider than the kernel: whole patches in the padding
]


@pytest.mark.parametrize("geom", DIRECT_GEOMS)
def test_one_kernel_conv_backward_equals_row_gradients_plus_fold(geom, cuda):
    """mam_conv_bwd_direct_f32 sums dx per tile of output rows in shared memory and adds the tiles into dx;
    mam_conv_bwd_f32 + mam_col2im_f32 go through the transposed row gradients.  Same sums in another order:
    dx and dW agree to rounding.  A few outputs get the same index on both sides (counted twice) and one row of
    outputs gets indices outside [0, K), which both forms skip."""
    B, C, H, W, kH, kW, sh, sw, ph, pw = geom
    L = _lib.lib()
    assert L.mam_conv_bwd_direct_applies(B, C, H, W, kH, kW, sh, sw, ph, pw) == 1
    g = torch.Generator().manual_seed(3 + sum(geom))
    x = torch.randn(B, C, H, W, generator=g).to(cuda)
    Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
    M, K, N = B * Ho * Wo, C * kH * kW, 37
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda)
    gy = torch.randn(M, N, generator=g).to(cuda)
    rows = torch.empty(M, K, device=cuda)
    _lib.check(L.mam_im2col_f32(_p(x), _p(rows), B, C, H, W, kH, kW, sh, sw, ph, pw, capi._stream()), "mam_im2col_f32")
    _, imax, imin = capi.forward(rows, w, capi.NK)
    imin[0, :] = imax[0, :]
    imax[M - 1, :] = K + 5
    imin[M - 1, :] = -1
    ct, dw_a = torch.empty(K, M, device=cuda), torch.empty_like(w)
    dx_a = torch.empty_like(x)
    _lib.check(L.mam_conv_bwd_f32(_p(x), _p(w), _p(gy), _p(imax), _p(imin), _p(ct), _p(dw_a), 0.5, B, C, H, W, kH, kW,
                                  sh, sw, ph, pw, N, capi._stream()), "mam_conv_bwd_f32")
    _lib.check(L.mam_col2im_f32(_p(ct), _p(dx_a), B, C, H, W, kH, kW, sh, sw, ph, pw, capi._stream()), "mam_col2im_f32")
    for _ in range(2):   # twice: the call zero-fills what it accumulates into
        dx_b, dw_b = torch.full_like(x, 7.0), torch.full_like(w, 7.0)
        _lib.check(L.mam_conv_bwd_direct_f32(_p(x), _p(w), _p(gy), _p(imax), _p(imin), _p(dx_b), _p(dw_b), 0.5, B, C, H,
                                             W, kH, kW, sh, sw, ph, pw, N, capi._stream()), "mam_conv_bwd_direct_f32")
        assert_grad_close(dx_b.cpu().numpy(), dx_a.cpu().numpy())
        assert_grad_close(dw_b.cpu().numpy(), dw_a.cpu().numpy())


def test_one_kernel_conv_backward_declines_what_does_not_fit(cuda):
    L = _lib.lib()
    # 4096 channels x 3 input rows x 64 columns of fp32 = 3 MiB: no tile of dx fits a CTA's shared memory
    assert L.mam_conv_bwd_direct_applies(1, 4096, 64, 64, 3, 3, 1, 1, 1, 1) == 0
    assert L.mam_conv_bwd_direct_applies(128, 64, 56, 56, 3, 3, 1, 1, 1, 1) == 1
    t = torch.zeros(16, device=cuda)
    i = torch.zeros(16, dtype=torch.int32, device=cuda)
    st = L.mam_conv_bwd_direct_f32(_p(t), _p(t), _p(t), _p(i), _p(i), _p(t), _p(t), 1.0, 1, 4096, 64, 64, 3, 3, 1, 1, 1,
                                   1, 8, capi._stream())
    assert st == 2   # MAM_ERR_UNSUPPORTED


@pytest.mark.parametrize("form", ["auto", "fold"])
def test_strided_padded_conv_module_gradients(form, cuda):
    import mamtorch_b200 as mamtorch
    from mamtorch_b200.nn.conv import set_conv_backward_form

    set_conv_backward_form(form)
    try:
        _strided_padded_conv_module_gradients(mamtorch, cuda)
    finally:
        set_conv_backward_form("auto")


def _strided_padded_conv_module_gradients(mamtorch, cuda):
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


# ---------------------------------------------------------------- forward without patch rows (im2col-mode TMA)
IMPLICIT_GEOMS = [  # B, C, H, W, kH, kW, sh, sw, ph, pw, N   (C % 32 == 0, input >= 128 KiB)
    (4, 64, 14, 14, 3, 3, 1, 1, 1, 1, 128),
    (2, 32, 33, 37, 3, 3, 2, 2, 1, 1, 70),
    (3, 96, 20, 17, 5, 3, 1, 2, 2, 0, 33),
    (2, 32, 40, 40, 1, 1, 1, 1, 0, 0, 130),
    (1, 32, 64, 48, 2, 4, 3, 1, 0, 3, 17),
    (5, 32, 19, 23, 3, 3, 1, 1, 2, 2, 64),     # padding larger than "same"
]


def _tap_order_oracle(x, w, geom, relu=False):
    """The oracle on patch rows whose columns are in the order (kw, kh, c) -- channels fastest, then kh, then
    kw -- with indices mapped back to the numbering of weight.view(N, -1)."""
    from mamtorch_b200.nn.conv import tap_order_permutation

    B, C, H, W, kH, kW, sh, sw, ph, pw, N = geom
    rows = mam_oracle.conv2d_as_rows(x.cpu(), (kH, kW), stride=(sh, sw), padding=(ph, pw))
    perm = tap_order_permutation(C, kH, kW)
    y, imax, imin = mam_oracle.mam_forward(rows[:, perm], w.cpu().reshape(N, -1)[:, perm].T.contiguous())
    return y, perm[imax], perm[imin]


@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("geom", IMPLICIT_GEOMS)
def test_implicit_conv_forward_matches_the_oracle_in_tap_order(geom, relu, cuda):
    B, C, H, W, kH, kW, sh, sw, ph, pw, N = geom
    L = _lib.lib()
    assert L.mam_conv_fwd_applies(B, C, H, W, kH, kW, sh, sw, ph, pw) == 1
    g = torch.Generator().manual_seed(sum(geom))
    x = torch.randn(B, C, H, W, generator=g)
    if relu:
        x = torch.relu(x)           # half of the activations exactly zero: extremes tie at zero all the time
    w = torch.randn(N, C, kH, kW, generator=g) * (C * kH * kW) ** -0.5
    if relu:
        w = w.abs()                 # every product >= 0, so every minimum is a tie among the zeros
    Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
    M = B * Ho * Wo
    x_nhwc = x.permute(0, 2, 3, 1).contiguous().to(cuda)
    w_taps = w.permute(0, 3, 2, 1).reshape(N, -1).contiguous().to(cuda)
    y = torch.empty(M, N, device=cuda)
    imax = torch.empty(M, N, dtype=torch.int32, device=cuda)
    imin = torch.empty_like(imax)
    _lib.check(L.mam_conv_fwd_f32(_p(x_nhwc), _p(w_taps), None, None, 0, 1.0, 0.0, _p(y), _p(imax), _p(imin), B, C, H, W,
                                  kH, kW, sh, sw, ph, pw, N, capi._stream()), "mam_conv_fwd_f32")
    torch.cuda.synchronize()
    _lib.check(L.mam_check_device_flag(), "device wait flag")
    y_ref, imax_ref, imin_ref = _tap_order_oracle(x, w, geom)
    assert torch.equal(y.cpu(), y_ref)
    assert torch.equal(imax.cpu().long(), imax_ref) and torch.equal(imin.cpu().long(), imin_ref)
    # values only: same kernel family without tracking
    y2 = torch.empty_like(y)
    _lib.check(L.mam_conv_fwd_f32(_p(x_nhwc), _p(w_taps), None, None, 0, 1.0, 0.0, _p(y2), None, None, B, C, H, W,
                                  kH, kW, sh, sw, ph, pw, N, capi._stream()), "mam_conv_fwd_f32")
    assert torch.equal(y2, y)


def test_implicit_conv_forward_rejects_what_the_copy_engine_cannot_express(cuda):
    L = _lib.lib()
    assert L.mam_conv_fwd_applies(4, 48, 14, 14, 3, 3, 1, 1, 1, 1) == 0        # channels not a multiple of 32
    assert L.mam_conv_fwd_applies(1, 32, 8, 8, 3, 3, 1, 1, 1, 1) == 0          # input below 128 KiB
    assert L.mam_conv_fwd_applies(4, 64, 14, 14, 3, 3, 9, 1, 1, 1) == 0        # stride beyond the traversal field
    assert L.mam_conv_fwd_applies(4, 64, 14, 14, 3, 3, 1, 1, 1, 1) == 1
    x = torch.zeros(4, 14, 14, 48, device=cuda)
    w = torch.zeros(8, 9 * 48, device=cuda)
    y = torch.empty(4 * 14 * 14, 8, device=cuda)
    assert L.mam_conv_fwd_f32(_p(x), _p(w), None, None, 0, 1.0, 0.0, _p(y), None, None, 4, 48, 14, 14, 3, 3, 1, 1, 1, 1,
                              8, capi._stream()) == 2
    assert L.mam_conv_fwd_f32(None, _p(w), None, None, 0, 1.0, 0.0, _p(y), None, None, 4, 64, 14, 14, 3, 3, 1, 1, 1, 1,
                              8, capi._stream()) == 1


@pytest.mark.parametrize("channels", [64, 5])      # 64: im2col-mode TMA; 5: same order through permuted patch rows
def test_conv_module_in_tap_order_matches_the_patch_row_module(channels, cuda):
    import mamtorch_b200 as mamtorch

    torch.manual_seed(21)
    a = mamtorch.nn.MAMConv2d(channels, 24, 3, stride=1, padding=1).to(cuda)
    b = mamtorch.nn.MAMConv2d(channels, 24, 3, stride=1, padding=1, reduction_order="taps").to(cuda)
    b.load_state_dict(a.state_dict())
    x = torch.randn(4, channels, 18, 15, generator=torch.Generator().manual_seed(22)).to(cuda)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, yb = a(xa), b(xb)
    assert torch.equal(ya, yb)
    # continuous random data: no two products are equal, so both orders name the same positions
    assert torch.equal(a.argmax, b.argmax) and torch.equal(a.argmin, b.argmin)
    gy = torch.randn(ya.shape, generator=torch.Generator().manual_seed(23)).to(cuda)
    ya.backward(gy)
    yb.backward(gy)
    assert_grad_close(xb.grad.cpu().numpy(), xa.grad.cpu().numpy())
    assert_grad_close(b.weight.grad.cpu().numpy(), a.weight.grad.cpu().numpy())
    # values-only path (no autograd, no indices asked for)
    with torch.no_grad():
        from mamtorch_b200.nn.conv import mam_conv2d
        y3, _, _ = mam_conv2d(x, b.weight, b.bias, 1, 1, need_indices=False, reduction_order="taps")
    assert torch.equal(y3, yb.detach())
    # ties: ReLU'd input, positive weights -> the two orders must each agree with their own oracle
    xr = torch.relu(x)
    with torch.no_grad():
        w_pos = b.weight.abs()
        y4, imax4, imin4 = mam_conv2d(xr, w_pos, None, 1, 1, reduction_order="taps")
    geom = (4, channels, 18, 15, 3, 3, 1, 1, 1, 1, 24)
    y_ref, imax_ref, imin_ref = _tap_order_oracle(xr, w_pos, geom)
    flat = lambda t: t.permute(0, 2, 3, 1).reshape(-1, 24).cpu()
    assert torch.equal(flat(y4), y_ref)
    assert torch.equal(flat(imax4).long(), imax_ref) and torch.equal(flat(imin4).long(), imin_ref)


@pytest.mark.parametrize("shape", [(3, 64, 14, 9), (2, 5, 7, 33), (1, 96, 1, 1), (4, 32, 56, 56)])
def test_channels_last_copy(shape, cuda):
    B, C, H, W = shape
    x = torch.randn(B, C, H, W, generator=torch.Generator().manual_seed(B * C + H)).to(cuda)
    out = torch.ops.mamtorch_b200.conv_channels_last(x)
    assert out.shape == (B, H, W, C) and out.is_contiguous()
    assert torch.equal(out, x.permute(0, 2, 3, 1))
    # the operator always returns a fresh tensor (its schema says so); an input that already is channels-last
    # in memory gives the same values, and the module uses such an input in place without calling it
    xcl = x.contiguous(memory_format=torch.channels_last)
    copy = torch.ops.mamtorch_b200.conv_channels_last(xcl)
    assert copy.data_ptr() != xcl.data_ptr() and torch.equal(copy, out)
    assert xcl.permute(0, 2, 3, 1).is_contiguous()
    torch.library.opcheck(torch.ops.mamtorch_b200.conv_channels_last, (xcl,))


def test_conv1d_without_patch_rows(cuda):
    """MAMConv1d with reduction_order="taps" and a channel count that is a multiple of 32: a convolution of height
    one through the im2col-mode TMA path (no patch rows), against the oracle in tap order, forward and backward,
    and against the patch-row module where no extreme is tied."""
    import mamtorch_b200 as mamtorch

    B, C, Lx, Fo, k = 12, 64, 700, 40, 5
    assert _lib.lib().mam_conv_fwd_applies(B, C, 1, Lx, 1, k, 1, 1, 0, 2) == 1
    torch.manual_seed(3)
    taps = mamtorch.nn.MAMConv1d(C, Fo, k, padding=2, reduction_order="taps").to(cuda)
    rows = mamtorch.nn.MAMConv1d(C, Fo, k, padding=2).to(cuda)
    rows.load_state_dict(taps.state_dict())
    g = torch.Generator().manual_seed(4)
    x = torch.randn(B, C, Lx, generator=g).to(cuda)
    gy = torch.randn(B, Fo, Lx, generator=g).to(cuda)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, yb = taps(xa), rows(xb)
    torch.cuda.synchronize()
    assert capi.device_flag_ok()
    geom = (B, C, 1, Lx, 1, k, 1, 1, 0, 2, Fo)
    y_ref, imax_ref, imin_ref = _tap_order_oracle(x.cpu().unsqueeze(2), taps.weight.detach().cpu().unsqueeze(2), geom)
    y_ref = y_ref + taps.bias.detach().cpu()
    flat = lambda t: t.permute(0, 2, 1).reshape(-1, Fo)
    assert torch.equal(flat(ya.detach()).cpu(), y_ref)
    assert torch.equal(flat(taps.argmax).cpu().long(), imax_ref) and torch.equal(flat(taps.argmin).cpu().long(), imin_ref)
    assert torch.equal(ya, yb)                                  # values do not depend on the reduction order
    assert torch.equal(taps.argmax, rows.argmax)                # random data: no ties, so neither do the indices
    ya.backward(gy)
    yb.backward(gy)
    assert_grad_close(xa.grad.cpu().numpy(), xb.grad.cpu().numpy())
    assert_grad_close(taps.weight.grad.cpu().numpy(), rows.weight.grad.cpu().numpy())


@pytest.mark.parametrize("geom", [
    (6, 48, 28, 28, 3, 3, 1, 1, 1, 1, 40),     # 48 channels -> padded to 64
    (16, 3, 64, 64, 3, 3, 1, 1, 1, 1, 24),     # an RGB first layer: 3 -> 32
    (4, 33, 20, 31, 3, 2, 2, 1, 1, 0, 17),     # 33 -> 64, one real channel in the second chunk of every tap
    (8, 100, 17, 17, 1, 1, 1, 1, 0, 0, 64),    # 1x1 kernel, 100 -> 128
])
@pytest.mark.parametrize("relu", [False, True])
def test_no_patch_rows_for_channel_counts_that_are_not_multiples_of_32(geom, relu, cuda):
    """reduction_order="taps" with C % 32 != 0: the channels are padded to a multiple of 32 -- zeros in the
    channels-last copy of x, NaN in the weight -- and the padded products (NaN) must never show up in a value or
    an index: everything equals the oracle in tap order on the unpadded problem, forward and backward."""
    from mamtorch_b200.nn.conv import mam_conv2d

    B, C, H, W, kH, kW, sh, sw, ph, pw, N = geom
    assert C % 32 != 0 and _lib.lib().mam_conv_fwd_applies(B, -(-C // 32) * 32, H, W, kH, kW, sh, sw, ph, pw) == 1
    g = torch.Generator().manual_seed(sum(geom))
    x = torch.randn(B, C, H, W, generator=g)
    w = torch.randn(N, C, kH, kW, generator=g) * (C * kH * kW) ** -0.5
    if relu:
        x, w = torch.relu(x), w.abs()      # zero ties everywhere: the first in tap order must win
    y_ref, imax_ref, imin_ref = _tap_order_oracle(x, w, geom)
    xd = x.to(cuda).requires_grad_()
    wd = w.to(cuda).requires_grad_()
    y, imax, imin = mam_conv2d(xd, wd, None, (sh, sw), (ph, pw), reduction_order="taps")
    torch.cuda.synchronize()
    assert capi.device_flag_ok()
    flat = lambda t: t.permute(0, 2, 3, 1).reshape(-1, N)
    assert not torch.isnan(y).any()
    assert torch.equal(flat(y.detach()).cpu(), y_ref)
    assert torch.equal(flat(imax).cpu().long(), imax_ref) and torch.equal(flat(imin).cpu().long(), imin_ref)
    yv, _, _ = mam_conv2d(x.to(cuda), w.to(cuda), None, (sh, sw), (ph, pw), need_indices=False, reduction_order="taps")
    assert torch.equal(yv, y.detach())
    # backward against the patch-row module path on the same indices (no ties in the random case)
    gy = torch.randn(y.shape, generator=g).to(cuda)
    y.backward(gy)
    xr = x.to(cuda).requires_grad_()
    wr = w.to(cuda).requires_grad_()
    yr, imax_r, _ = mam_conv2d(xr, wr, None, (sh, sw), (ph, pw))
    assert torch.equal(yr, y)
    if not relu:
        assert torch.equal(imax_r, imax)
        yr.backward(gy)
        assert_grad_close(xd.grad.cpu().numpy(), xr.grad.cpu().numpy())
        assert_grad_close(wd.grad.cpu().numpy(), wr.grad.cpu().numpy())
