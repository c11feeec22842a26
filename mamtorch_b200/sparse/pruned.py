"""From a magnitude-pruned weight straight to the CSR kernels.

The reference prunes a fine-tuned ViT by zeroing dense weights in place -- per layer, every weight whose
magnitude is at or below the p-quantile of that layer's magnitudes
(`examples/vitb16_imagenet1k/pruning_utils.py:105-116`, `LMP`), or with one threshold for all layers
(`:137-160`, `GMP`) -- and then keeps running the dense kernels on the zeros.  Here the same masks are
formed on the device and the layer runs on the stored weights only:

  * `magnitude_threshold`, `magnitude_keep_mask`  the quantile threshold (torch.quantile's linear interpolation,
                                                  as `LMP` uses it) and the keep mask of one weight;
  * `global_magnitude_threshold`                  one threshold over several weights: the element at position
                                                  int(p * n) of the sorted magnitudes, `GMP`'s own rule (`:147-151`);
  * `PrunedFullyConnected`                        a MAM layer that keeps a dense parameter plus its mask and
                                                  evaluates through CSR.  The forward sees `weight * keep_mask`,
                                                  so the chain rule hands pruned positions a zero gradient: they
                                                  stay where they are (and stay pruned) under any optimiser.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor, nn

from .kernel.v1 import mam_linear_csr

__all__ = ["magnitude_threshold", "global_magnitude_threshold", "magnitude_keep_mask", "PrunedFullyConnected"]

_QUANTILE_MAX = 1 << 24   # torch.quantile refuses larger inputs


def _quantile(values: Tensor, p: float) -> Tensor:
    """torch.quantile's default (linear) interpolation, also for inputs beyond its size limit."""
    if values.numel() <= _QUANTILE_MAX:
        return torch.quantile(values, p)
    s = values.sort().values
    pos = p * (s.numel() - 1)
    lo, hi = int(math.floor(pos)), int(math.ceil(pos))
    return s[lo] + (s[hi] - s[lo]) * (pos - lo)


def magnitude_threshold(weight: Tensor, fraction: float) -> Tensor:
    """The `fraction`-quantile of |weight| (a 0-d tensor on the weight's device)."""
    if not 0.0 <= fraction <= 1.0:
        raise ValueError("fraction must be in [0, 1]")
    return _quantile(weight.detach().abs().flatten().float(), fraction)


def global_magnitude_threshold(weights, fraction: float) -> Tensor:
    """One threshold for several weights together (global magnitude pruning): the magnitude at position
    int(fraction * n) of the n sorted magnitudes, clamped to the last one -- the reference's rule
    (`examples/vitb16_imagenet1k/pruning_utils.py:147-151`), not an interpolated quantile."""
    if not 0.0 <= fraction <= 1.0:
        raise ValueError("fraction must be in [0, 1]")
    flat = torch.cat([w.detach().abs().flatten().float() for w in weights])
    s = flat.sort().values
    return s[max(0, min(int(fraction * s.numel()), s.numel() - 1))]


def magnitude_keep_mask(weight: Tensor, threshold) -> Tensor:
    """1.0 where |weight| > threshold, 0.0 elsewhere: the reference zeroes `abs() <= threshold`."""
    return (weight.detach().abs() > threshold).to(weight.dtype)


class _MamLinearCsrKept(torch.autograd.Function):
    """CSR forward on a scratch buffer that keeps the regrouped sparsity pattern between calls; backward through
    the selected pairs into the dense (zero-filled) weight."""

    @staticmethod
    def forward(ctx, x, crow, col, val, dense_weight, bias, ws, ready):
        y, argmax, argmin = torch.ops.mamtorch_b200.csr_linear_forward_ws(x, crow, col, val, bias, True, ws, ready)
        ctx.save_for_backward(x, dense_weight, argmax, argmin)
        ctx.has_bias = bias is not None
        ctx.mark_non_differentiable(argmax, argmin)
        ctx.set_materialize_grads(False)   # no zero-filled index "gradients" before every backward call
        return y, argmax, argmin

    @staticmethod
    def backward(ctx, gy, _a, _b):
        if gy is None:
            return (None,) * 8
        x, w, argmax, argmin = ctx.saved_tensors
        gy = gy.contiguous()
        dx, dw = torch.ops.mamtorch_b200.linear_backward(x, w, gy, argmax, argmin, 1.0)
        dbias = gy.sum(0) if ctx.has_bias and ctx.needs_input_grad[5] else None
        return dx, None, None, None, dw, dbias, None, None


class PrunedFullyConnected(nn.Module):
    """MAM fully-connected layer on a pruned weight.

    `weight` stays a dense [out, in] parameter and `keep_mask` a buffer; the forward runs the CSR kernels
    on `weight * keep_mask` and is bit-identical to `mamtorch.nn.FullyConnected` holding that zeroed
    weight.  The CSR form is rebuilt only when the parameter or the mask has changed."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        kw = {"device": device, "dtype": dtype}
        self.weight = nn.Parameter(torch.empty(out_features, in_features, **kw))
        self.bias = nn.Parameter(torch.empty(out_features, **kw)) if bias else None
        self.register_buffer("keep_mask", torch.ones(out_features, in_features, **kw))
        self.argmax = self.argmin = None
        self._csr = None
        self._csr_key = None
        self._ws = None          # scratch of the tiled kernels, kept between inference calls
        self._ws_key = None      # the CSR build whose regrouped entries the scratch holds
        self._ws_pattern = None  # the mask whose regrouped pattern the scratch holds (training steps)
        self._pattern_key = None
        self._pattern_val = None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(in_features) if in_features > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    @classmethod
    def from_dense(cls, layer: nn.Module, fraction: float | None = None, threshold=None) -> "PrunedFullyConnected":
        """From any module with `weight` [out, in] and optional `bias` (nn.Linear, FullyConnected): prune
        the `fraction` of smallest magnitudes of this layer, or everything at or below `threshold`."""
        w = layer.weight
        new = cls(w.size(1), w.size(0), bias=getattr(layer, "bias", None) is not None, device=w.device, dtype=w.dtype)
        with torch.no_grad():
            new.weight.copy_(w)
            if new.bias is not None:
                new.bias.copy_(layer.bias)
        if fraction is not None or threshold is not None:
            new.prune_(fraction=fraction, threshold=threshold)
        return new

    @torch.no_grad()
    def prune_(self, fraction: float | None = None, threshold=None) -> "PrunedFullyConnected":
        if (fraction is None) == (threshold is None):
            raise ValueError("give exactly one of fraction and threshold")
        if threshold is None:
            threshold = magnitude_threshold(self.weight, fraction)
        self.keep_mask.copy_(magnitude_keep_mask(self.weight, threshold))
        self._csr = None
        self._ws_key = self._ws_pattern = self._pattern_key = None
        return self

    def sparsity(self) -> float:
        return 1.0 - float(self.keep_mask.mean())

    def _weight_csr(self) -> Tensor:
        key = (self.weight._version, self.keep_mask._version, self.weight.data_ptr(), self.keep_mask.data_ptr())
        if self._csr is None or self._csr_key != key:
            self._csr = (self.weight.detach() * self.keep_mask).to_sparse_csr()
            self._csr_key = key
        return self._csr

    def _scratch(self, x: Tensor, nnz: int):
        """(scratch buffer large enough for this call or None where the tiled kernels do not apply, was it kept)."""
        M, K = x.shape
        need, _ = torch.ops.mamtorch_b200.csr_workspace_bytes(M, K, self.out_features, nnz)
        if need == 0:
            return None, False
        kept = self._ws is not None and self._ws.numel() >= need and self._ws.device == x.device
        if not kept:
            self._ws = torch.empty(need, dtype=torch.uint8, device=x.device)
            self._ws_key = self._ws_pattern = None
        return self._ws, kept

    def _forward_kept_scratch(self, x: Tensor, csr: Tensor):
        """Inference on a weight that has not changed since the last call: the regrouped entries the tiled
        kernels work from are still in the scratch buffer, so only the activations are prepared again."""
        ops = torch.ops.mamtorch_b200
        crow, col, val = csr.crow_indices(), csr.col_indices(), csr.values()
        if x.size(0) == 0 or val.numel() == 0:
            return None
        ws, kept = self._scratch(x, val.numel())
        if ws is None:
            return None                      # the tiled kernels do not apply (few rows): no scratch involved
        ready = 1 if (kept and self._ws_key == ("values", self._csr_key)) else 0
        out = ops.csr_linear_forward_ws(x.contiguous(), crow.contiguous(), col.contiguous(), val.contiguous(),
                                        self.bias, True, ws, ready)
        self._ws_key = ("values", self._csr_key)
        self._ws_pattern = None
        return out

    def _pattern(self):
        """CSR pattern of the mask -- crow, col and the flat positions of the kept weights -- rebuilt only when
        the mask changes; a training step then gathers the kept values with one index_select."""
        key = (self.keep_mask._version, self.keep_mask.data_ptr())
        if self._pattern_key != key:
            csr = self.keep_mask.to_sparse_csr()
            crow, col = csr.crow_indices().contiguous(), csr.col_indices().contiguous()
            rows = torch.repeat_interleave(torch.arange(self.out_features, device=col.device), crow.diff())
            self._pattern_val = (crow, col, rows * self.in_features + col)
            self._pattern_key = key
        return self._pattern_val

    def _forward_training(self, x: Tensor):
        """Forward + gradient on a weight whose values move every step while its mask stays: the sparsity
        pattern (and the segment offsets regrouped from it in the scratch buffer) is kept across steps and
        only the stored values are gathered and regrouped again."""
        crow, col, flat = self._pattern()
        dense = self.weight * self.keep_mask
        if x.size(0) == 0 or flat.numel() == 0:
            return None, dense
        val = dense.detach().reshape(-1).index_select(0, flat)
        ws, kept = self._scratch(x, flat.numel())
        if ws is None:
            return None, dense
        ready = 2 if (kept and self._ws_pattern == self._pattern_key) else 0
        out = _MamLinearCsrKept.apply(x.contiguous(), crow, col, val, dense, self.bias, ws, ready)
        self._ws_pattern, self._ws_key = self._pattern_key, None
        return out, dense

    def forward(self, input: Tensor) -> Tensor:
        x = input.reshape(-1, input.size(-1))
        wants_grad = torch.is_grad_enabled() and (self.weight.requires_grad or x.requires_grad)
        out = None
        if wants_grad:
            out, dense = self._forward_training(x)
            if out is None:
                out = mam_linear_csr(x, (dense.detach()).to_sparse_csr(), self.bias, dense_weight=dense)
        else:
            csr = self._weight_csr()
            out = self._forward_kept_scratch(x, csr)
            if out is None:
                out = mam_linear_csr(x, csr, self.bias)
        y, self.argmax, self.argmin = out
        return y.view(input.shape[:-1] + (self.out_features,))

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
