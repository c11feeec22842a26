"""Kernel v2 (`mamtorch/kernel/v2/fullyconnected.py`, `dense.py`): bias and beta blend in the op."""
from torch import Tensor
import torch

from .._register import register_blended

__all__ = ["fullyconnected", "dense"]

register_blended("mamtorch_kernel_v2", with_fast=False, with_dense=True)


def fullyconnected(a: Tensor, b: Tensor, bias: Tensor, beta: float) -> list[Tensor]:
    """C = (1-beta)*(max+min) + beta*(a@b) + bias, with argmax/argmin of the MAM term."""
    return torch.ops.mamtorch_kernel_v2.fullyconnected.default(a, b, bias, beta)


def dense(a: Tensor, b: Tensor) -> Tensor:
    return torch.ops.mamtorch_kernel_v2.dense.default(a, b)
