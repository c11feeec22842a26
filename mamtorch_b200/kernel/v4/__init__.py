"""Kernel v4 (`mamtorch/kernel/v4/fullyconnected.py`, `fullyconnected_fast.py`).

In the reference `fullyconnected` is an approximation (k packed into the low mantissa bits of each
product, `mamtorch/kernel/v4/csrc/cuda/fullyconnected_kernel.cu:130-137`); here the same operator
name is served by the exact kernel, so values and indices always agree with the checker."""
from torch import Tensor
import torch

from .._register import register_plain

__all__ = ["fullyconnected", "fullyconnected_fast"]

register_plain("mamtorch_kernel_v4", with_fast=True)


def fullyconnected(a: Tensor, b: Tensor) -> list[Tensor]:
    return torch.ops.mamtorch_kernel_v4.fullyconnected.default(a, b)


def fullyconnected_fast(a: Tensor, b: Tensor) -> Tensor:
    """Values only (no indices): the inference form."""
    return torch.ops.mamtorch_kernel_v4.fullyconnected_fast.default(a, b)
