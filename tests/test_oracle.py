"""The oracle is only trusted after it reproduces stored outputs of the unmodified reference
checker (tests/golden/*.npz, produced by tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close, golden_names, load_golden
from oracle import c_oracle, mam_oracle


@pytest.mark.parametrize("name", golden_names())
def test_torch_oracle_matches_reference_outputs(name):
    g = load_golden(name)
    a, b = torch.from_numpy(g["a"]), torch.from_numpy(g["b"])
    bias = torch.from_numpy(g["bias"]) if "bias" in g else 0.0
    beta = float(g["beta"])
    y, imax, imin = mam_oracle.mam_forward(a, b, bias, beta)
    assert np.array_equal(imax.numpy(), g["argmax"])
    assert np.array_equal(imin.numpy(), g["argmin"])
    assert np.array_equal(y.numpy(), g["y"])  # same torch ops in the same order: bit-identical
    agrad, bgrad = mam_oracle.mam_backward(a, b, torch.from_numpy(g["g"]), imax, imin, beta)
    assert_grad_close(agrad.numpy(), g["agrad"])
    assert_grad_close(bgrad.numpy(), g["bgrad"])


@pytest.mark.parametrize("name", [n for n in golden_names() if not n.startswith("blend")])
def test_c_oracle_matches_reference_outputs(name):
    g = load_golden(name)
    bias = g.get("bias")
    for nk in (False, True):
        b = np.ascontiguousarray(g["b"].T) if nk else g["b"]
        y, imax, imin = c_oracle.forward(g["a"], b, b_is_nk=nk, bias=bias)
        assert np.array_equal(imax, g["argmax"])
        assert np.array_equal(imin, g["argmin"])
        assert np.array_equal(y, g["y"])
        agrad, bgrad = c_oracle.backward(g["a"], b, g["g"], imax, imin, b_is_nk=nk)
        if nk:
            bgrad = bgrad.T
        assert_grad_close(agrad, g["agrad"])
        assert_grad_close(bgrad, g["bgrad"])


@pytest.mark.parametrize("name", [n for n in golden_names() if "max_selection_count" in load_golden(n)])
def test_selection_count_oracle(name):
    g = load_golden(name)
    imax, imin = torch.from_numpy(g["argmax"]), torch.from_numpy(g["argmin"])
    K = g["a"].shape[1]
    N = g["b"].shape[1]
    cnt = mam_oracle.selection_count_update(torch.zeros((N, K), dtype=torch.int32), imax, imin)
    assert np.array_equal(cnt.numpy(), g["max_selection_count"])
    hmax, hmin = mam_oracle.selection_hits(imax, imin, K)
    assert int(hmax.sum()) == imax.numel() and int(hmin.sum()) == imin.numel()
    assert np.array_equal(((hmax > 0).int() + (hmin > 0).int()).numpy(), g["max_selection_count"])


def test_conv_oracle_agrees_with_direct_loops():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 3, 6, 5, generator=g)
    w = torch.randn(4, 3, 3, 2, generator=g)
    y, imax, imin = mam_oracle.mam_conv2d_forward(x, w, stride=1, padding=1)
    xp = torch.nn.functional.pad(x, (1, 1, 1, 1))
    Ho, Wo = y.shape[2:]
    for b_, f, i, j in [(0, 0, 0, 0), (1, 3, Ho - 1, Wo - 1), (0, 2, 2, 3)]:
        patch = xp[b_, :, i:i + 3, j:j + 2]
        p = (patch * w[f]).reshape(-1)
        assert y[b_, f, i, j] == p.max() + p.min()
        assert imax[b_, f, i, j] == int(p.argmax()) and imin[b_, f, i, j] == int(p.argmin())
