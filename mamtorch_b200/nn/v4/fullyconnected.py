"""`mamtorch.nn.FullyConnected` (the reference's exported default,
`mamtorch/nn/v4/fullyconnected.py:11-220`) on the B200 kernels.

Constructor arguments, attribute names, the vanishing-contribution schedule and the selection
count bookkeeping follow the reference so that user code and state dicts carry over.  What
differs is underneath: the weight is used as stored (no per-call transposes), the blend
`alpha*mam + beta*linear` and the bias add run in the kernel epilogue, both kernel choices of the
reference (`compute_exact` True/False) map to the one exact kernel, and the selection count is
formed on the device instead of through [M*N]-sized index tensors.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Module, Parameter

from .. import functional as MF

__all__ = ["FullyConnected"]


class FullyConnected(Module):
    __name__ = "FullyConnected"
    __constants__ = ["in_features", "out_features"]

    def __init__(self, in_features: int, out_features: int, bias: bool = True, splits: int = 1,
                 relu_in: bool = False, vcon_steps: int = 0, vcon_type: str = "linear",
                 vcon_eps: float = 1e-3, vcon_expand: bool = False, wdrop_rate: float = 0,
                 drop_rate: float = 0, compute_exact=False, train_mam_only=False, store_args=False,
                 device=None, dtype=None, **ignored) -> None:
        # `ignored` swallows stale keyword arguments such as the `beta_zero_gain` the reference's own
        # ViT example still passes (examples/vitb16_imagenet1k/utils.py:73).
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.splits, self.relu_in = splits, relu_in
        self.vcon_type, self.vcon_steps = vcon_type, vcon_steps
        self.vcon_eps, self.vcon_expand = vcon_eps, vcon_expand
        self.wdrop_rate, self.drop_rate = wdrop_rate, drop_rate
        self.compute_exact, self.train_mam_only, self.store_args = compute_exact, train_mam_only, store_args

        kw = {"device": device, "dtype": dtype}
        self.weight = Parameter(torch.empty(out_features, in_features, **kw))
        if bias:
            self.bias = Parameter(torch.empty(out_features, **kw))
        else:
            self.register_parameter("bias", None)
        if splits > 1:
            self.in_subfeatures = math.ceil(in_features / splits)
            self.in_subfeatures_last = in_features - self.in_subfeatures * (splits - 1)

        self.beta, self.alpha = (1.0, 0.0) if vcon_steps > 0 else (0.0, 1.0)
        self.max_selection_count = None
        self.min_selection_count = None
        self.argmax = None
        self.argmin = None
        self._hit_sink = MF.HitSink() if store_args else None
        self.reset_parameters()

    # -- initialisation: the same distributions as torch.nn.Linear, as in the reference (:76-84)
    def reset_parameters(self) -> None:
        torch.nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in = self.in_features
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            torch.nn.init.uniform_(self.bias, -bound, bound)

    # -- vanishing contribution: beta decays from 1 to 0, alpha = 1 - beta (reference :86-105)
    def vcon_step(self) -> None:
        if self.vcon_steps < 0:
            raise Exception("Invalid value for vcon_steps. Please use 0 or a positive integer.")
        if self.vcon_steps == 0:
            return
        if self.vcon_type == "linear":
            self.beta -= 1 / self.vcon_steps
        elif self.vcon_type == "exponential":
            self.beta *= math.exp(math.log(self.vcon_eps) / self.vcon_steps)
        else:
            raise Exception(f"vcon_type '{self.vcon_type}' is not supported.")
        if self.beta <= self.vcon_eps:
            self.beta = 0
        self.alpha = 1.0 - self.beta
        if self.vcon_expand:
            self.alpha *= self.in_features / (2 * self.splits)

    # -- selection counts (reference :107-131)
    def _require_store_args(self, what: str) -> None:
        if not self.store_args:
            raise Exception("MAM layer has not been set to store max and min arguments "
                            f"(store_args is False). Do not use {what}()")

    def reset_selection_count(self) -> None:
        self._require_store_args("reset_selection_count")
        self.max_selection_count = torch.zeros(self.weight.shape, dtype=torch.int32, device=self.weight.device)
        self.min_selection_count = torch.zeros_like(self.max_selection_count)

    def update_selection_count(self) -> None:
        self._require_store_args("update_selection_count")
        if self.argmax is None or self.argmin is None:
            raise Exception("No argmax or argmin values have been evaluated yet.")
        if self.max_selection_count is None or self.min_selection_count is None:
            self.reset_selection_count()
        # Both updates land in max_selection_count and each distinct (n,k) counts once per call:
        # that is what the reference's two `t[idx] += 1` statements do (:125-129).
        # if a backward pass already ran on these indices it counted the hits on its way
        hits = self._hit_sink.take(self.argmax) if self._hit_sink is not None else None
        MF.selection_count_update_(self.max_selection_count, self.argmax, self.argmin, hits)
        MF.poll_device_flag()     # raises if a kernel of an earlier call gave up a bounded wait

    def selection_hits(self):
        """True per-weight hit counts (hit_max, hit_min) of the last stored forward: an extension,
        the reference only keeps the 0/1-per-call form above."""
        self._require_store_args("selection_hits")
        if self.argmax is None or self.argmin is None:
            raise Exception("No argmax or argmin values have been evaluated yet.")
        return MF.selection_hits(self.argmax, self.argmin, self.in_features)

    # -- forward (reference :133-208)
    def forward(self, input: Tensor) -> Tensor:
        if input.is_cuda:
            MF.poll_device_flag()     # raises if a kernel of an earlier call gave up a bounded wait
        if self.relu_in:
            input = F.relu(input)
        x = input.reshape(-1, input.size(-1))
        w = self.weight
        if self.training and self.wdrop_rate != 0:
            if not 0 < self.wdrop_rate < 1:
                raise Exception("wdrop_rate must be between 0 and 1.")
            # one kernel pass, the mask formed again from its seed in the backward (no stored mask, no temporaries)
            w = MF.weight_drop(w, self.wdrop_rate)

        dense = None
        if self.beta > 0:
            dense = MF.dense_linear(x, self.weight.detach() if self.train_mam_only else self.weight)
        need_idx = self.training or (self.store_args and self.splits <= 1)

        if self.beta >= 1:
            # pure MAC phase of the schedule: the MAM term is multiplied by alpha = 0 in the
            # reference too (it substitutes zeros, :160-161)
            y = self.beta * dense
            if self.bias is not None:
                y = y + self.bias
            if self.store_args and self.splits <= 1:
                # the reference runs the MAM kernel on this path whatever beta is and keeps its indices
                # (:178-186), so that update_selection_count() works from the first step of the schedule
                with torch.no_grad():
                    _, self.argmax, self.argmin = MF.mam_linear(x.detach(), w.detach(), need_indices=True)
        elif self.splits > 1:
            # K is cut into slices; every slice contributes its own max+min (reference :164-176)
            y = None
            if not self.training and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad)):
                # inference: all slices in one launch (needs slice widths that are multiples of 32)
                fused = torch.ops.mamtorch_b200.linear_forward_splits(
                    x.contiguous(), w.contiguous(), self.bias, dense, float(self.alpha) if dense is not None else 1.0,
                    float(self.beta) if dense is not None else 0.0, self.in_subfeatures)
                if fused.numel() == x.size(0) * self.out_features and fused.dim() == 2:
                    y = fused.view(input.shape[:-1] + (self.out_features,))
                    if self.drop_rate > 0:
                        y = F.dropout(y, self.drop_rate, self.training)
                    return y
            elif self.in_subfeatures * (self.splits - 1) < self.in_features:
                # training: all slices in one launch of the index-producing forward, one backward pass over all
                # of them (same restrictions on the slice width)
                y = MF.mam_linear_splits(x, w, self.in_subfeatures, self.bias, dense,
                                         self.alpha if dense is not None else 1.0,
                                         self.beta if dense is not None else 0.0)
                if y is not None:
                    y = y.view(input.shape[:-1] + (self.out_features,))
                    if self.drop_rate > 0:
                        y = F.dropout(y, self.drop_rate, self.training)
                    return y
            bounds = [(i * self.in_subfeatures, self.in_subfeatures) for i in range(self.splits - 1)]
            bounds.append((self.in_features - self.in_subfeatures_last, self.in_subfeatures_last))
            for start, width in bounds:
                part, _, _ = MF.mam_linear(x.narrow(-1, start, width), w.narrow(-1, start, width),
                                           need_indices=self.training)
                y = part if y is None else y + part
            if dense is not None:
                y = self.alpha * y + self.beta * dense
            if self.bias is not None:
                y = y + self.bias
        else:
            # output dropout rides in the kernel epilogue (training only; F.dropout is the identity otherwise)
            fused_drop = self.drop_rate if (self.training and 0 < self.drop_rate < 1) else 0.0
            y, argmax, argmin = MF.mam_linear(x, w, self.bias, dense, self.alpha, self.beta if dense is not None else 0.0,
                                              need_indices=need_idx,
                                              hit_sink=self._hit_sink if (self.store_args and self.training) else None,
                                              drop_rate=fused_drop)
            if self.store_args:
                self.argmax, self.argmin = argmax, argmin
            if fused_drop > 0:
                return y.view(input.shape[:-1] + (self.out_features,))

        y = y.view(input.shape[:-1] + (self.out_features,))
        if self.drop_rate > 0:
            y = F.dropout(y, self.drop_rate, self.training)
        return y

    def __repr__(self) -> str:
        parts = [f"in_features={self.in_features}", f"out_features={self.out_features}",
                 f"bias={self.bias is not None}"]
        if self.vcon_steps > 0:
            parts.append(f"vcon_steps={self.vcon_steps}, vcon_type={self.vcon_type}")
        if self.splits > 1:
            parts.append(f"splits={self.splits}")
        if self.vcon_expand:
            parts.append("vcon_expand=True")
        if self.relu_in:
            parts.append("relu_in=True")
        return "MAM@FullyConnected(" + ", ".join(parts) + ")"
