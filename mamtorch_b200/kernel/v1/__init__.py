"""Kernel v1: exact MAM forward with indices (`mamtorch/kernel/v1/fullyconnected.py`)."""
from torch import Tensor
import torch

from .._register import register_plain

__all__ = ["fullyconnected"]

register_plain("mamtorch_kernel_v1", with_fast=False)


def fullyconnected(a: Tensor, b: Tensor) -> list[Tensor]:
    """[C, argmax, argmin] for a[M,K], b[K,N]; C = max_k(a*b) + min_k(a*b), indices int32."""
    return torch.ops.mamtorch_kernel_v1.fullyconnected.default(a, b)
