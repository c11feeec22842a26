"""Fake (meta) kernels and autograd formulas for the MAM operators, shared by every kernel
version.  The C++ shim only registers CUDA implementations; shape inference for tracing and the
backward rule are attached here from Python, as the reference does in
`mamtorch/kernel/v4/fullyconnected.py:12-64` and `mamtorch/kernel/v3/fullyconnected.py:12-75`.
"""
from __future__ import annotations

import torch


def _check_pair(a, b):
    torch._check(a.dim() == 2 and b.dim() == 2)
    torch._check(a.size(1) == b.size(0))
    torch._check(a.dtype == torch.float and b.dtype == torch.float)
    torch._check(a.device == b.device)
    torch._check(a.is_contiguous() and b.is_contiguous())


def _out_triplet(a, b):
    shape = (a.size(0), b.size(1))
    return [a.new_empty(shape), a.new_empty(shape, dtype=torch.int), a.new_empty(shape, dtype=torch.int)]


def _check_backward(a, b, grad, argmax, argmin):
    _check_pair(a, b)
    torch._check(grad.size(0) == a.size(0) and grad.size(1) == b.size(1))
    torch._check(grad.shape == argmax.shape and grad.shape == argmin.shape)
    torch._check(grad.dtype == torch.float)
    torch._check(argmax.dtype == torch.int and argmin.dtype == torch.int)
    for t in (grad, argmax, argmin):
        torch._check(t.device == a.device)
        torch._check(t.is_contiguous())


def register_plain(ns: str, with_fast: bool) -> None:
    """fullyconnected(a,b), fullyconnected_backward(...), optionally fullyconnected_fast(a,b)."""
    ops = getattr(torch.ops, ns)

    @torch.library.register_fake(f"{ns}::fullyconnected")
    def _(a, b):
        _check_pair(a, b)
        return _out_triplet(a, b)

    @torch.library.register_fake(f"{ns}::fullyconnected_backward")
    def _(a, b, grad, argmax, argmin):
        _check_backward(a, b, grad, argmax, argmin)
        return [torch.empty_like(a), torch.empty_like(b)]

    def setup(ctx, inputs, output):
        a, b = inputs
        need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        ctx.save_for_backward(a if need else None, b if need else None, output[1], output[2])

    def backward(ctx, grads):
        a, b, argmax, argmin = ctx.saved_tensors
        if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]):
            return None, None
        da, db = ops.fullyconnected_backward.default(a, b, grads[0].contiguous(), argmax, argmin)
        return da, db

    torch.library.register_autograd(f"{ns}::fullyconnected", backward, setup_context=setup)

    if with_fast:
        @torch.library.register_fake(f"{ns}::fullyconnected_fast")
        def _(a, b):
            _check_pair(a, b)
            return a.new_empty((a.size(0), b.size(1)))

        # The values-only operator is meant for inference; like the reference
        # (mamtorch/kernel/v4/fullyconnected_fast.py:22-28) its registered gradient is the dense one.
        def setup_fast(ctx, inputs, output):
            a, b = inputs
            need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
            ctx.save_for_backward(a if need else None, b if need else None)

        def backward_fast(ctx, grad):
            a, b = ctx.saved_tensors
            if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]):
                return None, None
            return grad @ b.T, a.T @ grad

        torch.library.register_autograd(f"{ns}::fullyconnected_fast", backward_fast, setup_context=setup_fast)


def register_blended(ns: str, with_fast: bool, with_dense: bool) -> None:
    """The (a, b, bias, beta) operator family of kernel versions 2 and 3."""
    ops = getattr(torch.ops, ns)

    def check_bias(a, b, bias):
        _check_pair(a, b)
        torch._check(bias.dim() == 1 and bias.size(0) == b.size(1))
        torch._check(bias.dtype == torch.float and bias.device == a.device and bias.is_contiguous())

    @torch.library.register_fake(f"{ns}::fullyconnected")
    def _(a, b, bias, beta):
        check_bias(a, b, bias)
        return _out_triplet(a, b)

    @torch.library.register_fake(f"{ns}::fullyconnected_backward")
    def _(a, b, grad, argmax, argmin, beta):
        _check_backward(a, b, grad, argmax, argmin)
        return [torch.empty_like(a), torch.empty_like(b)]

    def setup(ctx, inputs, output):
        a, b, _bias, beta = inputs
        need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        ctx.beta = beta
        ctx.save_for_backward(a if need else None, b if need else None, output[1], output[2])

    def backward(ctx, grads):
        a, b, argmax, argmin = ctx.saved_tensors
        g = grads[0].contiguous()
        da = db = dbias = None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            da, db = ops.fullyconnected_backward.default(a, b, g, argmax, argmin, ctx.beta)
        if ctx.needs_input_grad[2]:
            # the reference hands back the [M,N] upstream gradient here
            # (mamtorch/kernel/v3/fullyconnected.py:34-35), which autograd rejects for a [N] bias;
            # the gradient of a broadcast add is the column sum.
            dbias = g.sum(0)
        return da, db, dbias, None

    torch.library.register_autograd(f"{ns}::fullyconnected", backward, setup_context=setup)

    if with_fast:
        @torch.library.register_fake(f"{ns}::fullyconnected_fast")
        def _(a, b, bias, beta):
            check_bias(a, b, bias)
            return a.new_empty((a.size(0), b.size(1)))

        # like the reference (mamtorch/kernel/v3/fullyconnected_fast.py:26-52) the values-only operator
        # carries the dense gradients: grad @ b.T, a.T @ grad, and the column sum for the bias
        def setup_fast(ctx, inputs, output):
            a, b, _bias, _beta = inputs
            need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
            ctx.save_for_backward(a if need else None, b if need else None)

        def backward_fast(ctx, grad):
            a, b = ctx.saved_tensors
            da = grad @ b.T if ctx.needs_input_grad[0] else None
            db = a.T @ grad if ctx.needs_input_grad[1] else None
            dbias = grad.sum(0) if ctx.needs_input_grad[2] else None
            return da, db, dbias, None

        torch.library.register_autograd(f"{ns}::fullyconnected_fast", backward_fast, setup_context=setup_fast)

    if with_dense:
        @torch.library.register_fake(f"{ns}::dense")
        def _(a, b):
            _check_pair(a, b)
            return a.new_empty((a.size(0), b.size(1)))
