"""The checks of the reference's own test script (`test/test.py:9-180` of SSIGPRO/mamtorch) run against
this package THROUGH the reference's import name: `import mamtorch`, `torch.ops.mamtorch_kernel_v1..v4`,
`torch.library.opcheck` on every operator the script opchecks, and the script's functionality checks (result,
argmax and argmin errors against `fullyconnected_reference`; gradient errors against
`fullyconnected_backward_reference`) -- asserted here instead of printed.  Shapes are drawn like the
script's (`random.randint(10, 1000)` per extent) from a fixed seed.  The oracle restates the script's
`test/reference.py`; values and indices must be bit-exact where beta = 0 and within 1e-5 relative where
the dense term takes part (full fp32 by default), gradients within 1e-5.
"""
import random

import pytest
import torch

from conftest import assert_grad_close
from oracle import mam_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def case(cuda):
    import mamtorch  # noqa: F401  (the alias package: resolves to mamtorch_b200)

    rnd = random.Random(7)
    n, m, l = (rnd.randint(10, 1000) for _ in range(3))
    g = torch.Generator().manual_seed(7)
    a = torch.randn(n, m, generator=g)
    b = torch.randn(m, l, generator=g)
    c = torch.randn(n, l, generator=g)
    bias = torch.randn(l, generator=g)
    beta = rnd.uniform(0, 1)
    return {k: (v.to(cuda) if isinstance(v, torch.Tensor) else v)
            for k, v in dict(a=a, b=b, c=c, bias=bias, beta=beta).items()}


def _close(got, want, rtol=1e-5):
    scale = float(want.abs().max())
    assert float((got.cpu().double() - want.double()).abs().max()) <= rtol * scale


def test_import_name_resolves_to_this_package(cuda):
    import mamtorch
    import mamtorch_b200

    assert mamtorch is mamtorch_b200
    assert mamtorch.kernel.v4.fullyconnected is mamtorch_b200.kernel.v4.fullyconnected
    assert mamtorch.nn.FullyConnected is mamtorch_b200.nn.FullyConnected
    assert hasattr(mamtorch, "MAMDense") and hasattr(mamtorch.sparse.kernel.v1, "cusparsemm")


@pytest.mark.parametrize("ns", ["mamtorch_kernel_v1", "mamtorch_kernel_v4"])
def test_plain_generations(ns, case):
    ops = getattr(torch.ops, ns)
    a, b, c = case["a"], case["b"], case["c"]
    torch.library.opcheck(ops.fullyconnected, (a, b))
    res, argmax, argmin = ops.fullyconnected(a, b)
    res_ref, argmax_ref, argmin_ref = mam_oracle.mam_forward(a.cpu(), b.cpu())
    assert torch.equal(res.cpu(), res_ref)
    assert torch.equal(argmax.cpu().long(), argmax_ref) and torch.equal(argmin.cpu().long(), argmin_ref)
    assert argmax.dtype == torch.int32 and 0 <= int(argmax.min()) and int(argmax.max()) < a.size(1)
    if ns.endswith("v4"):
        torch.library.opcheck(ops.fullyconnected_fast, (a, b))
        assert torch.equal(ops.fullyconnected_fast(a, b).cpu(), res_ref)
    da, db = ops.fullyconnected_backward(a, b, c, argmax, argmin)
    da_ref, db_ref = mam_oracle.mam_backward(a.cpu(), b.cpu(), c.cpu(), argmax_ref, argmin_ref)
    assert_grad_close(da.cpu().numpy(), da_ref.numpy())
    assert_grad_close(db.cpu().numpy(), db_ref.numpy())


@pytest.mark.parametrize("ns", ["mamtorch_kernel_v2", "mamtorch_kernel_v3"])
def test_blended_generations(ns, case):
    ops = getattr(torch.ops, ns)
    a, b, c, bias, beta = case["a"], case["b"], case["c"], case["bias"], case["beta"]
    torch.library.opcheck(ops.fullyconnected, (a, b, bias, beta))
    res, argmax, argmin = ops.fullyconnected(a, b, bias, beta)
    res_ref, argmax_ref, argmin_ref = mam_oracle.mam_forward(a.cpu(), b.cpu(), bias.cpu(), beta)
    _close(res, res_ref)
    assert torch.equal(argmax.cpu().long(), argmax_ref) and torch.equal(argmin.cpu().long(), argmin_ref)
    if ns.endswith("v2"):
        _close(ops.dense(a, b), a.cpu() @ b.cpu())
    else:
        torch.library.opcheck(ops.fullyconnected_fast, (a, b, bias, beta))
        _close(ops.fullyconnected_fast(a, b, bias, beta), res_ref)
        # the values-only operator carries the dense gradients (mamtorch/kernel/v3/fullyconnected_fast.py:26-52)
        a2, b2, bias2 = (t.detach().clone().requires_grad_() for t in (a, b, bias))
        ops.fullyconnected_fast(a2, b2, bias2, beta).backward(c)
        _close(a2.grad, c.cpu() @ b.cpu().T, 1e-4)
        _close(b2.grad, a.cpu().T @ c.cpu(), 1e-4)
        _close(bias2.grad, c.cpu().sum(0), 1e-4)
    da, db = ops.fullyconnected_backward(a, b, c, argmax, argmin, beta)
    da_ref, db_ref = mam_oracle.mam_backward(a.cpu(), b.cpu(), c.cpu(), argmax_ref, argmin_ref, beta)
    assert_grad_close(da.cpu().numpy(), da_ref.numpy())
    assert_grad_close(db.cpu().numpy(), db_ref.numpy())


def test_sparse_namespace_carries_the_csr_mam_pair(case, cuda):
    """`mamtorch_kernel_sparsev1` holds the reference's `cusparsemm` and, beside it, the MAM layer on a CSR
    weight with its backward; both equal the dense operators on the zero-filled weight."""
    import mamtorch

    a, c = case["a"], case["c"]
    g = torch.Generator().manual_seed(3)
    w = torch.randn(c.size(1), a.size(1), generator=g)
    w = (w * (torch.rand(w.shape, generator=g) >= 0.8).float()).to(cuda)       # [N,K], 80 % zeros
    w_csr = w.to_sparse_csr()
    y, argmax, argmin = mamtorch.sparse.kernel.v1.fullyconnected_csr(a, w_csr)
    y0, argmax0, argmin0 = torch.ops.mamtorch_kernel_v4.fullyconnected(a, w.T.contiguous())
    assert torch.equal(y, y0) and torch.equal(argmax, argmax0) and torch.equal(argmin, argmin0)
    da, dw = mamtorch.sparse.kernel.v1.fullyconnected_csr_backward(a, w, c, argmax, argmin)
    da0, db0 = torch.ops.mamtorch_kernel_v4.fullyconnected_backward(a, w.T.contiguous(), c, argmax0, argmin0)
    assert_grad_close(da.cpu().numpy(), da0.cpu().numpy())
    assert_grad_close(dw.cpu().numpy(), db0.T.cpu().numpy())
    crow, col, val = (t.clone() for t in (w_csr.crow_indices(), w_csr.col_indices(), w_csr.values()))
    torch.library.opcheck(torch.ops.mamtorch_kernel_sparsev1.fullyconnected_csr, (a, crow, col, val, None))
