"""`mamtorch.MAMDense`, the deprecated first API (`mamtorch/nn/compat.py:8-112`)."""
from __future__ import annotations

import math

import torch

from .v1.fullyconnected import _SelectionCountMixin

__all__ = ["MAMDense"]


class MAMDense(_SelectionCountMixin, torch.nn.Module):
    def __init__(self, in_features, out_features, bias=True, beta=False, beta_decay="linear", beta_epochs=1):
        print("Warning: the use of mamtorch.MAMDense is deprecated. Use mamtorch.nn.FullyConnected instead.")
        super().__init__()
        self.input_features, self.state_size = in_features, out_features
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features))
        self.beta_decay, self.beta_epochs = beta_decay, beta_epochs
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self.beta = 1.0 if beta else 0.0
        self.max_selection_count = self.min_selection_count = None
        self.argmax = self.argmin = None
        self.reset_parameters()

    def reset_parameters(self):
        torch.nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.input_features) if self.input_features > 0 else 0
            torch.nn.init.uniform_(self.bias, -bound, bound)

    def adjust_beta(self, epoch):
        """beta as a function of the epoch (reference :44-60)."""
        if self.beta_epochs < 0:
            raise Exception("Invalid value for beta_epochs. Please use a positive integer.")
        t = epoch / self.beta_epochs if self.beta_epochs else 1.0
        if epoch >= self.beta_epochs:
            self.beta = 0
        elif self.beta_decay == "linear":
            self.beta = 1 - t
        elif self.beta_decay == "descending-parabola":
            self.beta = 1 - t ** 2
        elif self.beta_decay == "ascending-parabola":
            self.beta = 1 + t ** 2 - 2 * t

    def forward(self, input):
        return self._mam_forward(input, 10e-5)
