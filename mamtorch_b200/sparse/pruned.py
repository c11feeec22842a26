"""From a magnitude-pruned weight straight to the CSR kernels.

The reference prunes a fine-tuned ViT by zeroing dense weights in place -- per layer, every weight whose
magnitude is at or below the p-quantile of that layer's magnitudes
(`examples/vitb16_imagenet1k/pruning_utils.py:105-116`, `LMP`), or with one threshold for all layers
(`:137-160`, `GMP`) -- and then keeps running the dense kernels on the zeros.  Here the same masks are
formed on the device and the layer runs on the stored weights only:

  * `magnitude_threshold`, `magnitude_keep_mask`  the quantile threshold and the keep mask of one weight;
  * `global_magnitude_threshold`                  one threshold over several weights;
  * `PrunedFullyConnected`                        a MAM layer that keeps a dense parameter (so that it trains
                                                  like the reference's zeroed layer: selected pruned positions
                                                  receive gradient) plus its mask, and evaluates through CSR.
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
    """One threshold for several weights together (global magnitude pruning)."""
    flat = torch.cat([w.detach().abs().flatten().float() for w in weights])
    return _quantile(flat, fraction)


def magnitude_keep_mask(weight: Tensor, threshold) -> Tensor:
    """1.0 where |weight| > threshold, 0.0 elsewhere: the reference zeroes `abs() <= threshold`."""
    return (weight.detach().abs() > threshold).to(weight.dtype)


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
        self._ws_key = None
        return self

    def sparsity(self) -> float:
        return 1.0 - float(self.keep_mask.mean())

    def _weight_csr(self) -> Tensor:
        key = (self.weight._version, self.keep_mask._version, self.weight.data_ptr(), self.keep_mask.data_ptr())
        if self._csr is None or self._csr_key != key:
            self._csr = (self.weight.detach() * self.keep_mask).to_sparse_csr()
            self._csr_key = key
        return self._csr

    def _forward_kept_scratch(self, x: Tensor, csr: Tensor):
        """Inference on a weight that has not changed since the last call: the regrouped entries the tiled
        kernels work from are still in the scratch buffer, so only the activations are prepared again."""
        ops = torch.ops.mamtorch_b200
        crow, col, val = csr.crow_indices(), csr.col_indices(), csr.values()
        M, K = x.shape
        if M == 0 or val.numel() == 0:
            return None
        need, _ = ops.csr_workspace_bytes(M, K, self.out_features, val.numel())
        if need == 0:
            return None                      # the tiled kernels do not apply (few rows): no scratch involved
        ready = (self._ws is not None and self._ws_key == self._csr_key and self._ws.numel() >= need
                 and self._ws.device == x.device)
        if not ready and (self._ws is None or self._ws.numel() < need or self._ws.device != x.device):
            self._ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        out = ops.csr_linear_forward_ws(x.contiguous(), crow.contiguous(), col.contiguous(), val.contiguous(),
                                        self.bias, True, self._ws, ready)
        self._ws_key = self._csr_key
        return out

    def forward(self, input: Tensor) -> Tensor:
        x = input.reshape(-1, input.size(-1))
        csr = self._weight_csr()
        wants_grad = torch.is_grad_enabled() and (self.weight.requires_grad or x.requires_grad)
        out = None if wants_grad else self._forward_kept_scratch(x, csr)
        if out is not None:
            y, self.argmax, self.argmin = out
        else:
            dense = self.weight * self.keep_mask if torch.is_grad_enabled() and self.weight.requires_grad else None
            y, self.argmax, self.argmin = mam_linear_csr(x, csr, self.bias, dense_weight=dense)
        return y.view(input.shape[:-1] + (self.out_features,))

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
