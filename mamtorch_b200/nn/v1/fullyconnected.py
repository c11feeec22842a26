"""First-generation module (`mamtorch/nn/v1/fullyconnected.py:8-121`): always stores the indices,
xavier-style initialisation, linear vanishing contribution only."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .. import functional as MF

__all__ = ["FullyConnected"]


class _SelectionCountMixin:
    """Selection-count bookkeeping shared by the first-generation modules
    (`mamtorch/nn/v1/fullyconnected.py:69-87`, `mamtorch/nn/compat.py:62-80`)."""

    def reset_selection_count(self):
        self.max_selection_count = torch.zeros(self.weight.shape, dtype=torch.int32, device=self.weight.device)
        self.min_selection_count = torch.zeros_like(self.max_selection_count)

    def update_selection_count(self):
        if self.argmax is None or self.argmin is None:
            raise Exception("No argmax or argmin values have been evaluated yet.")
        if self.max_selection_count is None or self.min_selection_count is None:
            self.reset_selection_count()
        MF.selection_count_update_(self.max_selection_count, self.argmax, self.argmin)

    def _mam_forward(self, input, beta_floor):
        """(1-beta)*mam + beta*linear + bias with the indices kept on the module."""
        x = input.reshape(-1, input.size(-1))
        blend = self.beta > beta_floor
        dense = MF.dense_linear(x, self.weight) if blend else None
        y, self.argmax, self.argmin = MF.mam_linear(x, self.weight, self.bias, dense,
                                                    1 - self.beta if blend else 1.0,
                                                    self.beta if blend else 0.0)
        return y.view(tuple(input.shape[:-1]) + (self.weight.size(0),))


class FullyConnected(_SelectionCountMixin, torch.nn.Module):
    def __init__(self, in_features, out_features, bias=True, vcon_steps=0, vcon_type="linear",
                 init_mode="uniform", **kwargs):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.use_bias = bias
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features))
        self.vcon_type, self.vcon_steps, self.init_mode = vcon_type, vcon_steps, init_mode
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self.beta = 1.0 if vcon_steps > 0 else 0.0
        self.max_selection_count = self.min_selection_count = None
        self.argmax = self.argmin = None
        self.reset_parameters()

    def reset_parameters(self):
        # fan_in of a MAM neuron is taken as 2: only two products reach the output (reference :37-48)
        if self.init_mode == "uniform":
            bound = math.sqrt(6 / (2 + self.out_features))
            torch.nn.init.uniform_(self.weight, -bound, bound)
        elif self.init_mode == "normal":
            torch.nn.init.normal_(self.weight, std=math.sqrt(2 / (2 + self.out_features)))
        if self.bias is not None:
            torch.nn.init.zeros_(self.bias)

    def vcon_step(self):
        if self.vcon_steps < 0:
            raise Exception("Invalid value for vcon_steps. Please use 0 or a positive integer.")
        if self.vcon_steps == 0:
            return
        if self.vcon_type != "linear":
            raise Exception(f"Vanishing contribution type '{self.vcon_type}' is not supported")
        self.beta -= 1 / self.vcon_steps
        if self.beta <= 1e-8:
            self.beta = 0

    def forward(self, input):
        return self._mam_forward(input, 0.0)

    def __repr__(self):
        return (f"MAM@FullyConnected(in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.use_bias}, vcon_steps={self.vcon_steps}, vcon_type={self.vcon_type})")
