"""MAM convolutions as patch rows (im2col) + the fully-connected kernels.

The reference carries convolution only as never-compiled text backups
(`mamtorch/nn/backup/mamconv2d.txt:20-177`, `mamconv1d.txt`, kernels in
`mamtorch/kernel/backup/mamconv2d_forward.txt`).  These modules keep those constructor signatures
and attributes (weight [F,C,kH,kW], bias, beta schedule, argmax/argmin, selection counts) but:

  * integer `padding` is the usual symmetric convolution padding (the backup pads p//2 on the
    left and p-p//2 on the right, `mamconv2d.txt:133-139`);
  * the reduction index is k = (c*kH + kh)*kW + kw, the order of `weight.view(F, -1)` and of
    F.unfold, not the backup's k = c + C*(kh + kH*kw) (`mamconv2d_forward.txt:128`);
    `to_legacy_index` converts.

Each output pixel is one row of a GEMM-shaped MAM problem: M = B*Ho*Wo, K = C*kH*kW, N = F.

`reduction_order` chooses which of several EQUAL products an index names, and with it the data path:

  "unfold" (default)  the lowest k in the numbering above: patch rows are written once by
                      `conv_im2col` and the fully-connected kernels run on them;
  "taps"              the first in the backup's own reduction order (channels fastest, then kh, then
                      kw).  No patch rows exist: the kernels fetch 32-channel chunks of them from the
                      channels-last input by im2col-mode TMA (`conv_forward_implicit`).  A channel count
                      that is not a multiple of 32 is padded up to one (zero channels in the copy of x, NaN
                      channels in the weight: a NaN product never becomes an extreme), at Cp / C of the
                      arithmetic; only where the copy engine cannot express the geometry at all is the same
                      order produced through permuted patch rows.

Values are identical in both; indices are always NUMBERED k = (c*kH + kh)*kW + kw and differ between
the two orders only where a maximum or minimum is attained more than once (zero products of padding
or of ReLU'd inputs).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import functional as MF

_ops = torch.ops.mamtorch_b200

__all__ = ["MAMConv1d", "MAMConv2d", "mam_conv2d", "tap_order_permutation", "to_legacy_index",
           "set_conv_backward_form"]


# "auto": the one-kernel backward where its tile of dx fits shared memory, else transposed row gradients +
# fold; "fold": always the latter (kept for cross-checks and timing comparisons).
_backward_form = "auto"


def set_conv_backward_form(form: str) -> None:
    global _backward_form
    if form not in ("auto", "fold"):
        raise ValueError("form must be 'auto' or 'fold'")
    _backward_form = form


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


class _MamConv2d(torch.autograd.Function):
    """MAM convolution on patch rows: one im2col pass, the fully-connected kernels, and for the input
    gradient the backward's transposed row gradients folded by a gather kernel (no atomics).  The
    patch rows live only during the forward: the backward reads the two selected activations per
    output from the input itself."""

    @staticmethod
    def forward(ctx, x, weight, bias, dense, alpha, beta, stride, padding, taps=False):
        B, C, H, W = x.shape
        Fo, _, kH, kW = weight.shape
        (sh, sw), (ph, pw) = stride, padding
        Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
        w2d = weight.reshape(Fo, -1).contiguous()
        dflat = None
        if dense is not None:
            dflat = dense.permute(0, 2, 3, 1).reshape(B * Ho * Wo, Fo).contiguous()
        y, amax, amin = _forward_rows(x, weight, w2d, bias, dflat, alpha, beta, (kH, kW, sh, sw, ph, pw), taps, True)
        ctx.save_for_backward(x, w2d, amax, amin)
        ctx.geom = (B, C, H, W, Fo, kH, kW, sh, sw, ph, pw, Ho, Wo)
        ctx.alpha, ctx.beta = alpha, beta
        ctx.has_bias, ctx.has_dense = bias is not None, dense is not None
        img = lambda t: t.view(B, Ho, Wo, Fo).permute(0, 3, 1, 2)
        amax, amin = img(amax), img(amin)
        ctx.mark_non_differentiable(amax, amin)
        ctx.set_materialize_grads(False)   # no zero-filled index "gradients" before every backward call
        return img(y), amax, amin

    @staticmethod
    def backward(ctx, gy, _g1, _g2):
        if gy is None:
            return (None,) * 9
        x, w2d, amax, amin = ctx.saved_tensors
        B, C, H, W, Fo, kH, kW, sh, sw, ph, pw, Ho, Wo = ctx.geom
        g_rows = gy.permute(0, 2, 3, 1)
        if not g_rows.is_contiguous() and gy.is_cuda and gy.dtype == torch.float32:
            g_rows = _ops.conv_channels_last(gy)   # the library's batched transpose: ~3x torch's strided copy
        g2d = g_rows.reshape(B * Ho * Wo, Fo).contiguous()
        dx = dw = dbias = ddense = None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            if (_backward_form != "fold" and Fo * C * kH * kW < 2 ** 31
                    and _ops.conv_direct_applies(B, C, H, W, kH, kW, sh, sw, ph, pw)):
                # one kernel: dx summed in shared memory per tile of output rows, no row gradients in memory
                dx, dw2d = _ops.conv_backward_direct(x, w2d, g2d, amax, amin, ctx.alpha, kH, kW, sh, sw, ph, pw)
            else:
                cols_t, dw2d = _ops.conv_backward(x, w2d, g2d, amax, amin, ctx.alpha, kH, kW, sh, sw, ph, pw)
                if ctx.needs_input_grad[0]:
                    dx = _ops.conv_col2im(cols_t, B, C, H, W, kH, kW, sh, sw, ph, pw)
            dw = dw2d.view(Fo, C, kH, kW)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            dbias = g2d.sum(0)
        if ctx.has_dense and ctx.needs_input_grad[3]:
            ddense = gy * ctx.beta
        return dx, dw, dbias, ddense, None, None, None, None, None


def tap_order_permutation(in_channels, kH, kW, device=None):
    """perm[k'] = k: position k' = (kw*kH + kh)*C + c of the backup's reduction order -> the index
    k = (c*kH + kh)*kW + kw of `weight.view(F, -1)`."""
    return torch.arange(in_channels * kH * kW, device=device).view(in_channels, kH, kW).permute(2, 1, 0).reshape(-1)


def _forward_rows(x, weight, w2d, bias, dflat, alpha, beta, geom, taps, need_indices):
    """The row-form forward: [y[M,F]] or [y, argmax, argmin] with indices numbered like weight.view(F, -1)."""
    kH, kW, sh, sw, ph, pw = geom
    B, C, H, W = x.shape
    Fo = weight.size(0)
    if not taps:
        rows = _ops.conv_im2col(x, kH, kW, sh, sw, ph, pw)                    # [B*Ho*Wo, C*kH*kW]
        return _ops.linear_forward(rows, w2d, bias, dflat, alpha, beta, need_indices)
    w_taps = weight.permute(0, 3, 2, 1).reshape(Fo, -1).contiguous()          # [F, (kw, kh, c)]
    if _ops.conv_implicit_applies(B, C, H, W, kH, kW, sh, sw, ph, pw):
        x_nhwc = x.permute(0, 2, 3, 1)                                        # as it is if x is channels_last
        if not x_nhwc.is_contiguous():
            x_nhwc = _ops.conv_channels_last(x)                               # else one permuting copy
        if x_nhwc.data_ptr() % 16 == 0:
            return _ops.conv_forward_implicit(x_nhwc, w_taps, bias, dflat, alpha, beta, kH, kW, sh, sw, ph, pw,
                                              need_indices)
    Cp = -(-C // 32) * 32
    if Cp != C and _ops.conv_implicit_applies(B, Cp, H, W, kH, kW, sh, sw, ph, pw):
        # A channel count that is not a multiple of 32: the copy engine wants whole 32-channel chunks, so the
        # channels-last copy of x is padded with zero channels and the weight with NaN channels.  A padded
        # product is 0 * NaN = NaN, and fp32 max / min return the operand that is a number: the padded channels
        # never reach a maximum, a minimum or an index (the indices' numbering (c*kH + kh)*kW + kw does not
        # involve the channel count).  Costs Cp / C of the arithmetic, and still no patch rows.
        x_nhwc = x.new_zeros((B, H, W, Cp))
        x_nhwc[..., :C] = x.permute(0, 2, 3, 1)
        w_pad = weight.new_full((Fo, kW, kH, Cp), float("nan"))
        w_pad[..., :C] = weight.permute(0, 3, 2, 1)
        return _ops.conv_forward_implicit(x_nhwc, w_pad.reshape(Fo, -1), bias, dflat, alpha, beta, kH, kW, sh, sw, ph,
                                          pw, need_indices)
    # same reduction order through explicit patch rows with permuted columns
    perm = tap_order_permutation(C, kH, kW, x.device)
    rows = _ops.conv_im2col(x, kH, kW, sh, sw, ph, pw).index_select(1, perm)
    out = _ops.linear_forward(rows, w_taps, bias, dflat, alpha, beta, need_indices)
    if need_indices:
        perm32 = perm.to(torch.int32)
        out = [out[0], perm32[out[1].long()], perm32[out[2].long()]]
    return out


def mam_conv2d(x, weight, bias=None, stride=1, padding=0, dense=None, alpha=1.0, beta=0.0, need_indices=True,
               reduction_order="unfold"):
    """x[B,C,H,W], weight[F,C,kH,kW] -> (y[B,F,Ho,Wo], argmax, argmin) with indices into C*kH*kW."""
    if reduction_order not in ("unfold", "taps"):
        raise ValueError("reduction_order must be 'unfold' or 'taps'")
    taps = reduction_order == "taps"
    stride, padding = _pair(stride), _pair(padding)
    wants_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (x, weight, bias, dense))
    if need_indices or wants_grad:
        y, amax, amin = _MamConv2d.apply(x, weight, bias, dense, float(alpha), float(beta), stride, padding, taps)
        return (y, amax, amin) if need_indices else (y, None, None)
    B, C, H, W = x.shape
    Fo, _, kH, kW = weight.shape
    (sh, sw), (ph, pw) = stride, padding
    Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
    dflat = None if dense is None else dense.permute(0, 2, 3, 1).reshape(B * Ho * Wo, Fo).contiguous()
    y, = _forward_rows(x, weight, weight.reshape(Fo, -1).contiguous(), bias, dflat, float(alpha), float(beta),
                       (kH, kW, sh, sw, ph, pw), taps, False)
    return y.view(B, Ho, Wo, Fo).permute(0, 3, 1, 2), None, None


def to_legacy_index(idx, in_channels, kH, kW):
    """(c*kH + kh)*kW + kw  ->  c + C*(kh + kH*kw), the order of the reference's backup kernels."""
    kw = idx % kW
    kh = (idx // kW) % kH
    c = idx // (kW * kH)
    return c + in_channels * (kh + kH * kw)


class _ConvBase(torch.nn.Module):
    def _init_common(self, bias, beta, beta_decay, beta_epochs, out_channels):
        self.beta_decay, self.beta_epochs = beta_decay, beta_epochs
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        self.beta = 1.0 if beta else 0.0
        self.max_selection_count = self.min_selection_count = None
        self.argmax = self.argmin = None
        self.reset_parameters()

    def reset_parameters(self):
        torch.nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in = self.weight[0].numel()
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            torch.nn.init.uniform_(self.bias, -bound, bound)

    def adjust_beta(self, epoch):
        if self.beta_epochs <= 0:
            raise Exception("Invalid value for beta_epochs. Please use a positive integer.")
        t = epoch / self.beta_epochs
        if epoch >= self.beta_epochs:
            self.beta = 0
        elif self.beta_decay == "linear":
            self.beta = 1 - t
        elif self.beta_decay == "descending-parabola":
            self.beta = 1 - t ** 2
        elif self.beta_decay == "ascending-parabola":
            self.beta = 1 + t ** 2 - 2 * t

    def reset_selection_count(self):
        self.max_selection_count = torch.zeros(self.weight.shape, dtype=torch.int32, device=self.weight.device)
        self.min_selection_count = torch.zeros_like(self.max_selection_count)

    def update_selection_count(self):
        """Adds the number of output pixels that selected each weight: max hits into
        max_selection_count, min hits into min_selection_count (`mamconv2d.txt:90-114` keeps the
        two apart, unlike the fully-connected module)."""
        if self.argmax is None or self.argmin is None:
            raise Exception("No argmax or argmin values have been evaluated yet.")
        if self.max_selection_count is None:
            self.reset_selection_count()
        Fo = self.weight.size(0)
        K = self.weight[0].numel()
        flat = lambda t: t.movedim(1, -1).reshape(-1, Fo).contiguous()
        hmax, hmin = MF.selection_hits(flat(self.argmax), flat(self.argmin), K)
        self.max_selection_count += (hmax > 0).view_as(self.max_selection_count).to(torch.int32)
        self.min_selection_count += (hmin > 0).view_as(self.min_selection_count).to(torch.int32)


class MAMConv2d(_ConvBase):
    def __init__(self, in_channels, out_channels, kernel_size, bias=True, stride=1, padding=0,
                 padding_mode="zeros", beta=False, beta_decay="linear", beta_epochs=1, reduction_order="unfold"):
        super().__init__()
        if reduction_order not in ("unfold", "taps"):
            raise ValueError("reduction_order must be 'unfold' or 'taps'")
        self.reduction_order = reduction_order
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.padding_mode = kernel_size, stride, padding, padding_mode
        kH, kW = _pair(kernel_size)
        self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels, kH, kW))
        self.hstride, self.wstride = _pair(stride)
        self._init_common(bias, beta, beta_decay, beta_epochs, out_channels)

    def _padding(self):
        kH, kW = self.weight.shape[2:]
        if self.padding == "same":
            if (self.hstride, self.wstride) != (1, 1):
                raise Exception("Cannot apply 'same' padding with stride > 1.")
            if kH % 2 == 0 or kW % 2 == 0:
                raise Exception("'same' padding needs odd kernel sizes here.")
            return (kH // 2, kW // 2)
        if self.padding == "valid":
            return (0, 0)
        return _pair(self.padding)

    def forward(self, input):
        ph, pw = self._padding()
        x = input
        if self.padding_mode != "zeros" and (ph or pw):
            x = F.pad(x, (pw, pw, ph, ph), mode=self.padding_mode)
            ph = pw = 0
        dense = None
        blend = self.beta >= 10e-5
        if blend:
            dense = F.conv2d(x, self.weight, stride=(self.hstride, self.wstride), padding=(ph, pw))
        y, self.argmax, self.argmin = mam_conv2d(x, self.weight, self.bias, (self.hstride, self.wstride), (ph, pw),
                                                 dense, 1 - self.beta if blend else 1.0,
                                                 self.beta if blend else 0.0, reduction_order=self.reduction_order)
        return y


class MAMConv1d(_ConvBase):
    """1-D form (`mamtorch/nn/backup/mamconv1d.txt`): a 2-D convolution with a height of one."""

    def __init__(self, in_channels, out_channels, kernel_size, bias=True, stride=1, padding=0,
                 padding_mode="zeros", beta=False, beta_decay="linear", beta_epochs=1, reduction_order="unfold"):
        super().__init__()
        if reduction_order not in ("unfold", "taps"):
            raise ValueError("reduction_order must be 'unfold' or 'taps'")
        self.reduction_order = reduction_order
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.padding_mode = kernel_size, stride, padding, padding_mode
        self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels, kernel_size))
        self._init_common(bias, beta, beta_decay, beta_epochs, out_channels)

    def forward(self, input):
        k = self.weight.size(2)
        if self.padding == "same":
            if self.stride != 1 or k % 2 == 0:
                raise Exception("'same' padding needs stride 1 and an odd kernel size.")
            p = k // 2
        elif self.padding == "valid":
            p = 0
        else:
            p = int(self.padding)
        x = input
        if self.padding_mode != "zeros" and p:
            x = F.pad(x, (p, p), mode=self.padding_mode)
            p = 0
        blend = self.beta >= 10e-5
        dense = F.conv1d(x, self.weight, stride=self.stride, padding=p).unsqueeze(2) if blend else None
        y, amax, amin = mam_conv2d(x.unsqueeze(2), self.weight.unsqueeze(2), self.bias, (1, self.stride), (0, p),
                                   dense, 1 - self.beta if blend else 1.0, self.beta if blend else 0.0,
                                   reduction_order=self.reduction_order)
        self.argmax, self.argmin = amax.squeeze(2), amin.squeeze(2)
        return y.squeeze(2)

    def update_selection_count(self):
        am, an = self.argmax, self.argmin
        self.argmax, self.argmin = am.unsqueeze(2), an.unsqueeze(2)
        try:
            super().update_selection_count()
        finally:
            self.argmax, self.argmin = am, an
