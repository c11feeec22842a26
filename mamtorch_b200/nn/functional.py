"""Differentiable MAM primitives on the weight as a module stores it (W[out,in], K-contiguous).

`mam_linear` is what the modules call.  It hands W to the kernels in place -- the reference
transposes it into a fresh [K,N] copy on every forward (`mamtorch/nn/v4/fullyconnected.py:141`) and
its host code transposes the activations again (`mamtorch/kernel/v4/csrc/cuda/fullyconnected.cu:66`)
-- and folds the alpha/beta blend and the bias add into the kernel epilogue.
"""
from __future__ import annotations

import torch
from torch import Tensor

_ops = torch.ops.mamtorch_b200


@torch.library.register_fake("mamtorch_b200::linear_forward")
def _(x, weight, bias, dense, alpha, beta, want_idx):
    torch._check(x.dim() == 2 and weight.dim() == 2 and x.size(1) == weight.size(1))
    shape = (x.size(0), weight.size(0))
    out = [x.new_empty(shape)]
    if want_idx:
        out += [x.new_empty(shape, dtype=torch.int), x.new_empty(shape, dtype=torch.int)]
    return out


@torch.library.register_fake("mamtorch_b200::linear_forward_drop")
def _(x, weight, bias, dense, alpha, beta, want_idx, drop_rate, drop_seed):
    torch._check(x.dim() == 2 and weight.dim() == 2 and x.size(1) == weight.size(1))
    shape = (x.size(0), weight.size(0))
    out = [x.new_empty(shape)]
    if want_idx:
        out += [x.new_empty(shape, dtype=torch.int), x.new_empty(shape, dtype=torch.int)]
    return out


@torch.library.register_fake("mamtorch_b200::drop_apply")
def _(t, rate, scale, seed):
    return torch.empty_like(t, memory_format=torch.contiguous_format)


@torch.library.register_fake("mamtorch_b200::linear_backward")
def _(x, weight, grad, argmax, argmin, scale):
    return [torch.empty_like(x), torch.empty_like(weight)]


@torch.library.register_fake("mamtorch_b200::linear_backward_km")
def _(x, weight, grad, argmax, argmin, scale):
    return [x.new_empty((x.size(1), x.size(0))), torch.empty_like(weight)]


@torch.library.register_fake("mamtorch_b200::conv_backward")
def _(x, weight, grad, argmax, argmin, scale, kH, kW, sh, sw, ph, pw):
    return [x.new_empty((weight.size(1), grad.size(0))), torch.empty_like(weight)]


@torch.library.register_fake("mamtorch_b200::conv_im2col")
def _(x, kH, kW, sh, sw, ph, pw):
    B, C, H, W = x.shape
    Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
    return x.new_empty((B * Ho * Wo, C * kH * kW))


@torch.library.register_fake("mamtorch_b200::csr_linear_forward_ws")
def _(x, crow, col, val, bias, want_idx, workspace, entries_ready):
    y = x.new_empty((x.size(0), crow.numel() - 1))
    if not want_idx:
        return [y]
    return [y, y.new_empty(y.shape, dtype=torch.int32), y.new_empty(y.shape, dtype=torch.int32)]


@torch.library.register_fake("mamtorch_b200::linear_forward_splits_idx")
def _(x, weight, bias, dense, alpha, beta, split_width):
    M, K, N = x.size(0), x.size(1), weight.size(0)
    S = (K + split_width - 1) // split_width
    return [x.new_empty((M, N)), x.new_empty((S, M, N), dtype=torch.int), x.new_empty((S, M, N), dtype=torch.int)]


@torch.library.register_fake("mamtorch_b200::linear_backward_splits")
def _(x, weight, grad, argmax, argmin, scale):
    return [torch.empty_like(x), torch.empty_like(weight)]


@torch.library.register_fake("mamtorch_b200::linear_forward_splits")
def _(x, weight, bias, dense, alpha, beta, split_width):
    return x.new_empty((x.size(0), weight.size(0)))


@torch.library.register_fake("mamtorch_b200::check_device_flag")
def _():
    return None


@torch.library.register_fake("mamtorch_b200::poll_device_flag")
def _():
    return None


@torch.library.register_fake("mamtorch_b200::conv_channels_last")
def _(x):
    B, C, H, W = x.shape
    return x.new_empty((B, H, W, C))


@torch.library.register_fake("mamtorch_b200::transpose2d")
def _(a):
    return a.new_empty((a.shape[1], a.shape[0]))


@torch.library.register_fake("mamtorch_b200::conv_forward_implicit")
def _(x_nhwc, w_taps, bias, dense, alpha, beta, kH, kW, sh, sw, ph, pw, need_indices):
    B, H, W, C = x_nhwc.shape
    Ho, Wo = (H + 2 * ph - kH) // sh + 1, (W + 2 * pw - kW) // sw + 1
    y = x_nhwc.new_empty((B * Ho * Wo, w_taps.size(0)))
    if not need_indices:
        return [y]
    return [y, y.new_empty(y.shape, dtype=torch.int32), y.new_empty(y.shape, dtype=torch.int32)]


@torch.library.register_fake("mamtorch_b200::conv_backward_direct")
def _(x, weight, grad, argmax, argmin, scale, kH, kW, sh, sw, ph, pw):
    return [torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(weight)]


@torch.library.register_fake("mamtorch_b200::conv_col2im")
def _(cols_t, B, C, H, W, kH, kW, sh, sw, ph, pw):
    return cols_t.new_empty((B, C, H, W))


@torch.library.register_fake("mamtorch_b200::linear_backward_count")
def _(x, weight, grad, argmax, argmin, scale):
    shape = (weight.size(0), weight.size(1))
    return [torch.empty_like(x), torch.empty_like(weight), argmax.new_empty(shape), argmax.new_empty(shape)]


class HitSink:
    """Receives the selection hits a backward pass counted on its way, tagged with the index
    tensor they belong to, so that a later `update_selection_count()` need not sweep the indices
    again."""

    def __init__(self):
        self.argmax = None
        self.hits = None

    def take(self, argmax):
        """The hits recorded for exactly this index tensor, or None."""
        if self.hits is not None and self.argmax is argmax:
            hits, self.hits, self.argmax = self.hits, None, None
            return hits
        return None


@torch.library.register_fake("mamtorch_b200::selection_hits")
def _(argmax, argmin, K):
    shape = (argmax.size(1), K)
    return [argmax.new_empty(shape), argmax.new_empty(shape)]


@torch.library.register_fake("mamtorch_b200::dense_nt")
def _(a, w):
    torch._check(a.dim() == 2 and w.dim() == 2 and a.size(1) == w.size(1))
    return a.new_empty((a.size(0), w.size(0)))


def set_dense_backend(name: str) -> None:
    """Backend of the dense (sum-of-products) beta term: "tf32" = this library's tcgen05 kernel
    (TF32 inputs, fp32 accumulation, 1e-3 relative to fp32), "fp32" = torch/cuBLAS in full fp32, what
    the reference's `F.linear` / `at::linalg_matmul` compute, "auto" (the default) = "tf32" only while
    `torch.backends.cuda.matmul.allow_tf32` is on, as for torch's own matrix products."""
    if name not in ("tf32", "fp32", "auto"):
        raise ValueError("dense backend must be 'tf32', 'fp32' or 'auto'")
    _ops.set_dense_backend({"tf32": 1, "fp32": 0, "auto": -1}[name])


def get_dense_backend() -> str:
    return {1: "tf32", 0: "fp32", -1: "auto"}[int(_ops.get_dense_backend())]


def check_device_flag() -> None:
    """Waits for the device and raises RuntimeError if a kernel of this library gave up a bounded wait since
    the last check (its outputs are then invalid).  The modules call the non-waiting `poll_device_flag` on
    every forward and in `update_selection_count`, which reports such a time-out one call late at most;
    code that drives `torch.ops.mamtorch_kernel_v*` directly should call this where it synchronises anyway
    (end of an epoch, before a checkpoint)."""
    _ops.check_device_flag()


def poll_device_flag() -> None:
    """The same check without waiting for the device: raises if an EARLIER poll's copy of the flag shows a
    time-out, then queues the next fetch on the current stream."""
    _ops.poll_device_flag()


class _DenseLinear(torch.autograd.Function):
    """x[M,K] . W[N,K]^T on the tensor cores, with the two gradient products on them as well."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return _ops.dense_nt(x, weight)

    @staticmethod
    def backward(ctx, g):
        x, weight = ctx.saved_tensors
        g = g.contiguous()
        dx = dw = None
        tr = _ops.transpose2d if g.is_cuda and g.dtype == torch.float32 else (lambda t: t.t().contiguous())
        if ctx.needs_input_grad[0]:
            dx = _ops.dense_nt(g, tr(weight))          # [M,N] . [K,N]^T
        if ctx.needs_input_grad[1]:
            dw = _ops.dense_nt(tr(g), tr(x))           # [N,M] . [K,M]^T
        return dx, dw


def dense_linear(x: Tensor, weight: Tensor) -> Tensor:
    """The MAC term of a blended layer: x @ weight.T (no bias)."""
    return _DenseLinear.apply(x.contiguous(), weight.contiguous())


def fresh_drop_seed() -> int:
    """A seed for the library's counter-based drop masks, drawn from torch's CPU generator: reproducible
    under torch.manual_seed and without a device synchronisation."""
    return int(torch.randint(0, 2 ** 62, (1,)).item())


class _WeightDrop(torch.autograd.Function):
    """weight * mask with mask ~ Bernoulli(1 - rate) per element, unscaled, as the reference module's weight
    drop (`mamtorch/nn/v4/fullyconnected.py:143-148`): one kernel pass forward and one backward, the mask formed
    again from its seed instead of being stored."""

    @staticmethod
    def forward(ctx, weight, rate, seed):
        ctx.rate, ctx.seed = rate, seed
        return _ops.drop_apply(weight, rate, 1.0, seed)

    @staticmethod
    def backward(ctx, g):
        return _ops.drop_apply(g, ctx.rate, 1.0, ctx.seed), None, None


def weight_drop(weight: Tensor, rate: float, seed: int | None = None) -> Tensor:
    return _WeightDrop.apply(weight, float(rate), fresh_drop_seed() if seed is None else int(seed))


class _MamLinear(torch.autograd.Function):
    """y = drop(alpha*(max_k x*w + min_k x*w) + beta*dense + bias), gradient through the selected pairs.  The
    output dropout (drop_rate > 0) happens in the forward kernel's epilogue; its mask is formed again from
    (drop_seed, element index) for the backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, dense, alpha, beta, hit_sink=None, drop_rate=0.0, drop_seed=0):
        if drop_rate > 0:
            y, argmax, argmin = _ops.linear_forward_drop(x, weight, bias, dense, alpha, beta, True, drop_rate, drop_seed)
        else:
            y, argmax, argmin = _ops.linear_forward(x, weight, bias, dense, alpha, beta, True)
        ctx.save_for_backward(x, weight, argmax, argmin)
        ctx.alpha, ctx.beta, ctx.hit_sink = alpha, beta, hit_sink
        ctx.drop_rate, ctx.drop_seed = drop_rate, drop_seed
        ctx.has_bias, ctx.has_dense = bias is not None, dense is not None
        ctx.mark_non_differentiable(argmax, argmin)
        # the index outputs get no gradient: without this, autograd fills two [M,N] int32 zero tensors for them
        # before every backward call
        ctx.set_materialize_grads(False)
        return y, argmax, argmin

    @staticmethod
    def backward(ctx, gy, _g1, _g2):
        if gy is None:
            return (None,) * 9
        x, weight, argmax, argmin = ctx.saved_tensors
        gy = gy.contiguous()
        if ctx.drop_rate > 0:
            gy = _ops.drop_apply(gy, ctx.drop_rate, 1.0 / (1.0 - ctx.drop_rate), ctx.drop_seed)
        dx = dw = dbias = ddense = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            dbias = gy.sum(0)     # first: the layer above has only just written gy, much of it is still in L2
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            if ctx.hit_sink is not None:
                dx, dw, hmax, hmin = _ops.linear_backward_count(x, weight, gy, argmax, argmin, ctx.alpha)
                ctx.hit_sink.argmax, ctx.hit_sink.hits = argmax, (hmax, hmin)
            else:
                dx, dw = _ops.linear_backward(x, weight, gy, argmax, argmin, ctx.alpha)
        if ctx.has_dense and ctx.needs_input_grad[3]:
            ddense = gy * ctx.beta
        return dx, dw, dbias, ddense, None, None, None, None, None


def mam_linear(x: Tensor, weight: Tensor, bias: Tensor | None = None, dense: Tensor | None = None,
               alpha: float = 1.0, beta: float = 0.0, need_indices: bool = True, hit_sink: "HitSink | None" = None,
               drop_rate: float = 0.0, drop_seed: int | None = None):
    """x[M,K], weight[N,K] -> (y[M,N], argmax, argmin) or (y, None, None).

    With `need_indices=False` the values-only kernel runs (no autograd: use it for inference).
    `drop_rate > 0` applies output dropout in the kernel epilogue (a training-time option: it always drops)."""
    x = x.contiguous()
    weight = weight.contiguous()
    drop_rate = float(drop_rate)
    if drop_rate > 0 and drop_seed is None:
        drop_seed = fresh_drop_seed()
    drop_seed = int(drop_seed or 0)
    if not need_indices and torch.is_grad_enabled() and (
            x.requires_grad or weight.requires_grad or (bias is not None and bias.requires_grad)
            or (dense is not None and dense.requires_grad)):
        need_indices = True  # a gradient is wanted: only the index-producing kernel can route it
        y, _, _ = _MamLinear.apply(x, weight, bias, dense, float(alpha), float(beta), None, drop_rate, drop_seed)
        return y, None, None
    if need_indices:
        return _MamLinear.apply(x, weight, bias, dense, float(alpha), float(beta), hit_sink, drop_rate, drop_seed)
    if drop_rate > 0:
        y, = _ops.linear_forward_drop(x, weight, bias, dense, float(alpha), float(beta), False, drop_rate, drop_seed)
    else:
        y, = _ops.linear_forward(x, weight, bias, dense, float(alpha), float(beta), False)
    return y, None, None


class _MamLinearSplits(torch.autograd.Function):
    """The module's `splits` in training: y = alpha * sum over K slices of (max + min of the slice) + beta*dense + bias
    from ONE launch of the index-producing forward (plus one index resolver per slice), every slice keeping its
    own selected pairs; the backward routes the gradient through all of them in one pass."""

    @staticmethod
    def forward(ctx, x, weight, bias, dense, alpha, beta, split_width):
        out = _ops.linear_forward_splits_idx(x, weight, bias, dense, alpha, beta, split_width)
        if len(out) == 0:
            raise _SplitsUnsupported()
        y, argmax, argmin = out
        ctx.save_for_backward(x, weight, argmax, argmin)
        ctx.alpha, ctx.beta = alpha, beta
        ctx.has_bias, ctx.has_dense = bias is not None, dense is not None
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight, argmax, argmin = ctx.saved_tensors
        gy = gy.contiguous()
        dx = dw = dbias = ddense = None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            dx, dw = _ops.linear_backward_splits(x, weight, gy, argmax, argmin, ctx.alpha)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            dbias = gy.sum(0)
        if ctx.has_dense and ctx.needs_input_grad[3]:
            ddense = gy * ctx.beta
        return dx, dw, dbias, ddense, None, None, None


class _SplitsUnsupported(Exception):
    pass


def mam_linear_splits(x: Tensor, weight: Tensor, split_width: int, bias: Tensor | None = None,
                      dense: Tensor | None = None, alpha: float = 1.0, beta: float = 0.0):
    """Differentiable MAM layer with K cut into slices of `split_width` columns, all slices in one launch.
    Returns None where that form does not apply (slice width not a multiple of 32, K % 4 != 0, unaligned
    operands): the caller then goes slice by slice."""
    try:
        return _MamLinearSplits.apply(x.contiguous(), weight.contiguous(), bias, dense, float(alpha), float(beta),
                                      int(split_width))
    except _SplitsUnsupported:
        return None


def selection_hits(argmax: Tensor, argmin: Tensor, in_features: int):
    """(hit_max[N,K], hit_min[N,K]): how many rows picked each weight as max / as min."""
    return _ops.selection_hits(argmax.contiguous(), argmin.contiguous(), int(in_features))


def selection_count_update_(count: Tensor, argmax: Tensor, argmin: Tensor, hits=None) -> Tensor:
    """In-place equivalent of one `update_selection_count()` of the reference module
    (`mamtorch/nn/v4/fullyconnected.py:114-131`): +1 for every weight any row selected as max and
    +1 for every weight any row selected as min, both added to the same matrix."""
    hmax, hmin = hits if hits is not None else selection_hits(argmax, argmin, count.size(1))
    return _ops.selection_count_update_(count, hmax, hmin)
