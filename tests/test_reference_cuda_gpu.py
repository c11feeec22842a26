"""Parity against the reference's own CUDA kernels on the same GPU and the same seeded inputs.

The reference's v4 operators are compiled from its sources into oracle/_ref/ (oracle/build_ref_cuda.py); a
child process runs them (they define the same operator namespace as this package, so they cannot share a
process with it).  What is comparable bit for bit: the values of `fullyconnected_fast` (exact max + min).  The
reference's index-producing `fullyconnected` overwrites the low 16 mantissa bits of every product with the
index, so its values are only close and its indices can differ where two products agree in their upper bits;
its `fullyconnected_backward`, fed the exact indices, must reproduce the gradients to the tolerance of fp32
atomics (1e-5 relative)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import assert_grad_close

import capi

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "mamtorch_kernel_v4.so")
CASES = [(256, 512, 256), (300, 200, 130), (64, 64, 64), (197, 768, 384), (33, 1000, 65), (1024, 96, 200)]


@pytest.fixture(scope="module")
def both(cuda, tmp_path_factory):
    if not os.path.exists(REF_SO):
        pytest.skip("the reference's CUDA operators were not built (python oracle/build_ref_cuda.py --reference DIR)")
    tmp = tmp_path_factory.mktemp("refcuda")
    cases, ours = {"count": len(CASES)}, []
    for i, (M, K, N) in enumerate(CASES):
        g = torch.Generator().manual_seed(1000 + i)
        a = torch.randn(M, K, generator=g)
        w = torch.randn(N, K, generator=g) * K ** -0.5
        gy = torch.randn(M, N, generator=g)
        b = w.T.contiguous()
        y, imax, imin = capi.forward(a.to(cuda), b.to(cuda), capi.KN)
        da, db = capi.backward(a.to(cuda), b.to(cuda), gy.to(cuda), imax, imin, capi.KN)
        ours.append((y.cpu(), imax.cpu(), imin.cpu(), da.cpu(), db.cpu(), float(a.abs().max() * w.abs().max())))
        cases.update({f"a{i}": a.numpy(), f"b{i}": b.numpy(), f"g{i}": gy.numpy(), f"imax{i}": imax.cpu().numpy(),
                      f"imin{i}": imin.cpu().numpy()})
    cases_path, out_path = str(tmp / "cases.npz"), str(tmp / "results.npz")
    np.savez(cases_path, **cases)
    run = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_cuda_worker.py"), REF_SO, cases_path, out_path],
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    return ours, np.load(out_path)


@pytest.mark.parametrize("i", range(len(CASES)))
def test_values_equal_the_reference_fast_kernel_bit_for_bit(both, i):
    ours, ref = both
    y = ours[i][0].numpy()
    assert np.array_equal(y, ref[f"y_fast{i}"])


@pytest.mark.parametrize("i", range(len(CASES)))
def test_reference_backward_on_the_exact_indices_gives_the_same_gradients(both, i):
    ours, ref = both
    assert_grad_close(ours[i][3].numpy(), ref[f"da{i}"])
    assert_grad_close(ours[i][4].numpy(), ref[f"db{i}"])


@pytest.mark.parametrize("i", range(len(CASES)))
def test_reference_index_kernel_is_close_and_mostly_agrees(both, i):
    """Its packed-index kernel is approximate by design: values within 2^-7 relative of the products involved,
    indices equal wherever the extreme is not contested in the upper 16 bits -- the majority."""
    ours, ref = both
    y, imax, imin = ours[i][0].numpy(), ours[i][1].numpy(), ours[i][2].numpy()
    # each of the two selected products keeps 7 mantissa bits: error below 2^-7 of the largest possible product
    np.testing.assert_allclose(ref[f"y_idx{i}"], y, rtol=0, atol=2 ** -6 * ours[i][5])
    assert (ref[f"amax{i}"] == imax).mean() > 0.7 and (ref[f"amin{i}"] == imin).mean() > 0.7
