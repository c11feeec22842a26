"""Kernel v3 (`mamtorch/kernel/v3/fullyconnected.py`, `fullyconnected_fast.py`)."""
from torch import Tensor
import torch

from .._register import register_blended

__all__ = ["fullyconnected", "fullyconnected_fast"]

register_blended("mamtorch_kernel_v3", with_fast=True, with_dense=False)


def fullyconnected(a: Tensor, b: Tensor, bias: Tensor, beta: float) -> list[Tensor]:
    return torch.ops.mamtorch_kernel_v3.fullyconnected.default(a, b, bias, beta)


def fullyconnected_fast(a: Tensor, b: Tensor, bias: Tensor, beta: float) -> Tensor:
    return torch.ops.mamtorch_kernel_v3.fullyconnected_fast.default(a, b, bias, beta)
