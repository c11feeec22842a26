"""Sparse side of the package (`mamtorch/sparse/kernel/v1/cusparsemm.py`).

`cusparsemm(a_sparse, b)` keeps the reference's name, schema and dispatch (COO and CSR layouts)
but runs this library's CSR kernel instead of cuSPARSE.  `mam_linear_csr` is new: the MAM layer
on a pruned weight stored as CSR, equal to the dense layer on the weight with zeros at the
positions that are not stored.
"""
from __future__ import annotations

import torch
from torch import Tensor

__all__ = ["cusparsemm", "mam_linear_csr", "prune_to_csr", "fullyconnected_csr", "fullyconnected_csr_backward"]


def cusparsemm(a: Tensor, b: Tensor) -> Tensor:
    """a: sparse [N,K] (COO or CSR), b: dense [K,M] -> dense [N,M] = a @ b."""
    return torch.ops.mamtorch_kernel_sparsev1.cusparsemm.default(a, b)


@torch.library.register_fake("mamtorch_kernel_sparsev1::cusparsemm")
def _(a, b):
    torch._check(a.size(1) == b.size(0))
    torch._check(b.dtype == torch.float)
    return b.new_empty((a.size(0), b.size(1)))


@torch.library.register_fake("mamtorch_b200::csr_linear_forward")
def _(x, crow, col, val, bias, want_idx):
    shape = (x.size(0), crow.size(0) - 1)
    out = [x.new_empty(shape)]
    if want_idx:
        out += [x.new_empty(shape, dtype=torch.int), x.new_empty(shape, dtype=torch.int)]
    return out


@torch.library.register_fake("mamtorch_kernel_sparsev1::fullyconnected_csr")
def _(a, crow, col, val, bias):
    shape = (a.size(0), crow.size(0) - 1)
    return [a.new_empty(shape), a.new_empty(shape, dtype=torch.int), a.new_empty(shape, dtype=torch.int)]


@torch.library.register_fake("mamtorch_kernel_sparsev1::fullyconnected_csr_backward")
def _(a, w_dense, grad, argmax, argmin):
    return [torch.empty_like(a), torch.empty_like(w_dense)]


def fullyconnected_csr(a: Tensor, w_csr: Tensor, bias: Tensor | None = None):
    """[y, argmax, argmin] of the MAM layer on a pruned weight: a[M,K], w_csr sparse-CSR [N,K].  Operator
    `mamtorch_kernel_sparsev1::fullyconnected_csr`, beside the reference's `cusparsemm`."""
    return torch.ops.mamtorch_kernel_sparsev1.fullyconnected_csr.default(
        a, w_csr.crow_indices(), w_csr.col_indices(), w_csr.values(), bias)


def fullyconnected_csr_backward(a: Tensor, w_dense: Tensor, grad: Tensor, argmax: Tensor, argmin: Tensor):
    """[a_grad, w_grad (dense, like w_dense[N,K])] through the selected pairs; `w_dense` is the weight with
    zeros at the pruned positions."""
    return torch.ops.mamtorch_kernel_sparsev1.fullyconnected_csr_backward.default(a, w_dense, grad, argmax, argmin)


def prune_to_csr(weight: Tensor, keep_mask: Tensor) -> Tensor:
    """CSR form of `weight * keep_mask` ([out,in]); positions with keep_mask == 0 are not stored."""
    return (weight * keep_mask).to_sparse_csr()


class _MamLinearCsr(torch.autograd.Function):
    """Forward on the stored weights only; backward through the selected pairs into a DENSE weight
    gradient: a pruned position that was selected (its zero product was the extreme) receives
    gradient, exactly as it does when the dense kernels run on zeroed weights."""

    @staticmethod
    def forward(ctx, x, crow, col, val, dense_weight, bias):
        y, argmax, argmin = torch.ops.mamtorch_b200.csr_linear_forward(x, crow, col, val, bias, True)
        ctx.save_for_backward(x, dense_weight, argmax, argmin)
        ctx.has_bias = bias is not None
        ctx.mark_non_differentiable(argmax, argmin)
        ctx.set_materialize_grads(False)   # no zero-filled index "gradients" before every backward call
        return y, argmax, argmin

    @staticmethod
    def backward(ctx, gy, _a, _b):
        if gy is None:
            return (None,) * 6
        x, w, argmax, argmin = ctx.saved_tensors
        gy = gy.contiguous()
        dx, dw = torch.ops.mamtorch_b200.linear_backward(x, w, gy, argmax, argmin, 1.0)
        dbias = gy.sum(0) if ctx.has_bias and ctx.needs_input_grad[5] else None
        return dx, None, None, None, dw, dbias


def mam_linear_csr(x: Tensor, w_csr: Tensor, bias: Tensor | None = None, dense_weight: Tensor | None = None,
                   need_indices: bool = True):
    """x[M,K], w_csr sparse-CSR [N,K] -> (y, argmax, argmin).

    Pass `dense_weight` (the [N,K] weight with zeros at pruned positions, e.g. the module's
    parameter times its mask) to make the call differentiable; without it the call is
    inference-only."""
    x = x.contiguous()
    crow, col, val = w_csr.crow_indices(), w_csr.col_indices(), w_csr.values()
    if dense_weight is not None and need_indices:
        return _MamLinearCsr.apply(x, crow, col, val, dense_weight.contiguous(), bias)
    out = torch.ops.mamtorch_b200.csr_linear_forward(x, crow, col, val, bias, need_indices)
    return (out[0], out[1], out[2]) if need_indices else (out[0], None, None)
