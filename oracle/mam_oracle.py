"""CPU oracle for the Multiply-And-Max/min (MAM) path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch-on-CPU, the algorithm of the reference's own checker
(`test/reference.py` in SSIGPRO/mamtorch).  It exists so that the CUDA path can be compared with
something that does not share a line of code with it.  Only `tests/`, `__graft_entry__.smoke()`
and the CPU-baseline / reference legs of `bench.py` may import it; the product package never
does, and fails loudly when its CUDA library is missing instead of falling back to this.

Pinning: `tests/golden/make_golden.py` ran the unmodified reference functions and stored their
outputs; `tests/test_oracle.py` checks every function here against those stored outputs
(bit-exact for values and indices, 1e-6 relative for the re-associated gradient sums).

Semantics restated (file:line are the reference's):
  * forward, `test/reference.py:3-10`: v[m,k,n] = fl32(a[m,k] * b[k,n]); max and min over k with
    the FIRST occurrence winning ties (torch.max / torch.min on CPU), -0.0 == +0.0;
    y = (a @ b) * beta + (vmax + vmin) * (1 - beta) + bias.  Indices are int64.
  * backward, `test/reference.py:12-25`: each output routes its upstream gradient to the two
    selected products only; a position selected as both max and min is counted twice; blended
    with the dense gradients by beta.
  * selection count, `mamtorch/nn/v4/fullyconnected.py:114-131`: the module adds, per call, one
    for every weight (n,k) that any row selected as max and one for every weight any row
    selected as min, both into `max_selection_count` (a non-accumulating `index_put_`).
"""
from __future__ import annotations

import torch

__all__ = [
    "mam_forward",
    "mam_backward",
    "selection_hits",
    "selection_count_update",
    "conv2d_as_rows",
    "mam_conv2d_forward",
]


def mam_forward(a: torch.Tensor, b: torch.Tensor, bias=0.0, beta: float = 0.0,
                max_chunk_bytes: int = 1 << 29):
    """y, argmax, argmin for a[M,K], b[K,N]  (reference `test/reference.py:3-10`).

    The reference materialises the whole [M,K,N] product tensor; rows are independent, so this
    does the same thing in row chunks that keep the temporary under `max_chunk_bytes`.
    """
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[0]
    a = a.detach().to(torch.float32).cpu()
    b = b.detach().to(torch.float32).cpu()
    M, K = a.shape
    N = b.shape[1]
    rows = max(1, min(M, max_chunk_bytes // max(1, 4 * K * N)))
    s = torch.empty((M, N), dtype=torch.float32)
    amax = torch.empty((M, N), dtype=torch.int64)
    amin = torch.empty((M, N), dtype=torch.int64)
    for r0 in range(0, M, rows):
        v = a[r0:r0 + rows, :, None] * b           # one rounded fp32 multiply per product
        vmax, imax = torch.max(v, dim=-2)           # first occurrence wins ties
        vmin, imin = torch.min(v, dim=-2)
        s[r0:r0 + rows] = vmax + vmin
        amax[r0:r0 + rows] = imax
        amin[r0:r0 + rows] = imin
    if isinstance(bias, torch.Tensor):
        bias = bias.detach().to(torch.float32).cpu()
    y = (a @ b) * beta + s * (1.0 - beta) + bias
    return y, amax, amin


def mam_backward(a, b, cgrad, argmax, argmin, beta: float = 0.0):
    """agrad[M,K], bgrad[K,N]  (reference `test/reference.py:12-25`).

    The reference loops over rows building a [K,N] mask per row; the same sums are formed here
    with two accumulating scatters per operand (the order of the additions differs, the set of
    addends does not).
    """
    a = a.detach().to(torch.float32).cpu()
    b = b.detach().to(torch.float32).cpu()
    g = cgrad.detach().to(torch.float32).cpu()
    argmax = argmax.detach().to(torch.int64).cpu()
    argmin = argmin.detach().to(torch.int64).cpu()
    M, K = a.shape
    N = b.shape[1]
    rows = torch.arange(M)[:, None].expand(M, N)
    cols = torch.arange(N)[None, :].expand(M, N)
    # accumulate in float64 and round once: an order-independent stand-in for the fp32 sums
    agrad = torch.zeros((M, K), dtype=torch.float64)
    bgrad = torch.zeros((K, N), dtype=torch.float64)
    g64 = g.double()
    for idx in (argmax, argmin):
        agrad.index_put_((rows, idx), g64 * b[idx, cols].double(), accumulate=True)
        bgrad.index_put_((idx, cols), g64 * a[rows, idx].double(), accumulate=True)
    agrad = agrad.float()
    bgrad = bgrad.float()
    if beta != 0.0:
        agrad = (g @ b.T) * beta + agrad * (1 - beta)
        bgrad = (a.T @ g) * beta + bgrad * (1 - beta)
    return agrad, bgrad


def selection_hits(argmax, argmin, K: int):
    """True hit counts: cnt_max[n,k] = #rows whose argmax for output n is k (same for min)."""
    argmax = argmax.detach().to(torch.int64).cpu()
    argmin = argmin.detach().to(torch.int64).cpu()
    M, N = argmax.shape
    cols = torch.arange(N)[None, :].expand(M, N)
    one = torch.ones((M, N), dtype=torch.int32)
    cmax = torch.zeros((N, K), dtype=torch.int32).index_put_((cols, argmax), one, accumulate=True)
    cmin = torch.zeros((N, K), dtype=torch.int32).index_put_((cols, argmin), one, accumulate=True)
    return cmax, cmin


def selection_count_update(max_selection_count, argmax, argmin):
    """What one `update_selection_count()` call adds (`mamtorch/nn/v4/fullyconnected.py:114-131`).

    `t[idx] += 1` with duplicate indices writes each distinct position once, and the reference
    applies both the argmax and the argmin update to `max_selection_count`.
    """
    out = max_selection_count.clone()
    M, N = argmax.shape
    cols = torch.arange(N).repeat(M)
    out[cols, argmax.flatten().long().cpu()] += 1
    out[cols, argmin.flatten().long().cpu()] += 1
    return out


def conv2d_as_rows(x, kernel_size, stride=1, padding=0, dilation=1):
    """im2col: x[B,C,H,W] -> rows[B*Ho*Wo, C*kH*kW] with k = (c*kH + kh)*kW + kw (F.unfold order)."""
    cols = torch.nn.functional.unfold(x, kernel_size, dilation=dilation, padding=padding, stride=stride)
    B, CK, L = cols.shape
    return cols.transpose(1, 2).reshape(B * L, CK)


def mam_conv2d_forward(x, w, bias=None, stride=1, padding=0):
    """MAM convolution as im2col + the fully-connected oracle.  The reference only carries
    never-compiled text backups of a conv kernel (`mamtorch/kernel/backup/mamconv2d_forward.txt`),
    so this composition is the conv oracle; its index order is F.unfold's."""
    B, C, H, W = x.shape
    F_, _, kH, kW = w.shape
    rows = conv2d_as_rows(x.cpu(), (kH, kW), stride=stride, padding=padding)
    y, imax, imin = mam_forward(rows, w.reshape(F_, -1).T.contiguous().cpu(),
                                bias=0.0 if bias is None else bias.cpu())
    pair = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v, v)
    (sh, sw), (ph, pw) = pair(stride), pair(padding)
    Ho = (H + 2 * ph - kH) // sh + 1
    Wo = (W + 2 * pw - kW) // sw + 1
    to_img = lambda t: t.reshape(B, Ho, Wo, F_).permute(0, 3, 1, 2).contiguous()
    return to_img(y), to_img(imax), to_img(imin)
