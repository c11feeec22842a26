"""The reference-facing Python surface on the GPU: torch.ops schemas under opcheck, autograd, the
nn modules and the im2col convolution, checked against the oracle."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close, load_golden
from oracle import mam_oracle

pytestmark = pytest.mark.gpu


def _rand(shape, seed, dev, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dev)


@pytest.mark.parametrize("ns", ["mamtorch_kernel_v1", "mamtorch_kernel_v4"])
def test_opcheck_plain_ops(ns, cuda):
    import mamtorch_b200  # noqa: F401

    a = _rand((37, 52), 1, cuda).requires_grad_()
    b = _rand((52, 29), 2, cuda).requires_grad_()
    ops = getattr(torch.ops, ns)
    torch.library.opcheck(ops.fullyconnected, (a, b))
    if ns.endswith("v4"):
        torch.library.opcheck(ops.fullyconnected_fast, (a.detach(), b.detach()))
    c, imax, imin = ops.fullyconnected(a.detach(), b.detach())
    torch.library.opcheck(ops.fullyconnected_backward, (a.detach(), b.detach(), torch.ones_like(c), imax, imin))


@pytest.mark.parametrize("backend", ["fp32", "tf32"])
@pytest.mark.parametrize("ns", ["mamtorch_kernel_v2", "mamtorch_kernel_v3"])
def test_blended_ops_match_reference_formula(ns, backend, cuda):
    """The MAM term (indices) is exact with either backend of the dense term; the blended value is
    held to 1e-5 with the fp32 backend and to 1e-3 (TF32 inputs) with the tensor-core backend."""
    import mamtorch_b200
    from mamtorch_b200.nn import functional as MF

    tol = 1e-5 if backend == "fp32" else 1e-3
    MF.set_dense_backend(backend)
    g = load_golden("blend_40x64x48")
    a, b, bias, grad = (torch.from_numpy(g[k]).to(cuda) for k in ("a", "b", "bias", "g"))
    beta = float(g["beta"])
    ops = getattr(torch.ops, ns)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        c, imax, imin = ops.fullyconnected(a, b, bias, beta)
        da, db = ops.fullyconnected_backward(a, b, grad, imax, imin, beta)
        if ns.endswith("v3"):
            cf = ops.fullyconnected_fast(a, b, bias, beta)
            assert torch.equal(cf, c)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
        MF.set_dense_backend("auto")
    assert np.array_equal(imax.cpu().numpy(), g["argmax"]) and np.array_equal(imin.cpu().numpy(), g["argmin"])
    np.testing.assert_allclose(c.cpu().numpy(), g["y"], rtol=tol, atol=tol * float(np.abs(g["y"]).max()))
    assert_grad_close(da.cpu().numpy(), g["agrad"], rtol=tol)
    assert_grad_close(db.cpu().numpy(), g["bgrad"], rtol=tol)


def test_autograd_through_v4_wrapper(cuda):
    import mamtorch_b200 as mamtorch

    g = load_golden("random_37x70x29")
    a = torch.from_numpy(g["a"]).to(cuda).requires_grad_()
    b = torch.from_numpy(g["b"]).to(cuda).requires_grad_()
    c, imax, imin = mamtorch.kernel.v4.fullyconnected(a, b)
    assert torch.equal(c.detach().cpu(), torch.from_numpy(g["y"]))
    c.backward(torch.from_numpy(g["g"]).to(cuda))
    assert_grad_close(a.grad.cpu().numpy(), g["agrad"])
    assert_grad_close(b.grad.cpu().numpy(), g["bgrad"])


def test_fullyconnected_module_matches_oracle(cuda):
    import mamtorch_b200 as mamtorch

    torch.manual_seed(0)
    layer = mamtorch.nn.FullyConnected(96, 40, store_args=True).to(cuda)
    x = _rand((3, 17, 96), 4, cuda).requires_grad_()
    y = layer(x)
    y_ref, imax_ref, imin_ref = mam_oracle.mam_forward(x.detach().reshape(-1, 96).cpu(),
                                                       layer.weight.detach().T.contiguous().cpu(),
                                                       layer.bias.detach().cpu())
    assert y.shape == (3, 17, 40)
    assert torch.equal(y.detach().reshape(-1, 40).cpu(), y_ref)
    assert torch.equal(layer.argmax.cpu().long(), imax_ref) and torch.equal(layer.argmin.cpu().long(), imin_ref)
    gy = _rand((3, 17, 40), 5, cuda)
    y.backward(gy)
    da_ref, db_ref = mam_oracle.mam_backward(x.detach().reshape(-1, 96).cpu(), layer.weight.detach().T.cpu(),
                                             gy.reshape(-1, 40).cpu(), imax_ref, imin_ref)
    assert_grad_close(x.grad.reshape(-1, 96).cpu().numpy(), da_ref.numpy())
    assert_grad_close(layer.weight.grad.cpu().numpy(), db_ref.T.numpy())
    assert_grad_close(layer.bias.grad.cpu().numpy(), gy.reshape(-1, 40).sum(0).cpu().numpy())
    # selection count: two calls accumulate, exactly as the reference module's update does
    layer.update_selection_count()
    layer.update_selection_count()
    want = mam_oracle.selection_count_update(torch.zeros(40, 96, dtype=torch.int32), imax_ref, imin_ref)
    want = mam_oracle.selection_count_update(want, imax_ref, imin_ref)
    assert torch.equal(layer.max_selection_count.cpu(), want)
    assert int(layer.min_selection_count.abs().sum()) == 0
    # eval mode without stored args uses the values-only kernel and gives the same numbers
    layer2 = mamtorch.nn.FullyConnected(96, 40).to(cuda).eval()
    layer2.load_state_dict(layer.state_dict())
    with torch.no_grad():
        assert torch.equal(layer2(x.detach()), y.detach())


def test_module_beta_blend_splits_and_relu(cuda):
    import mamtorch_b200 as mamtorch

    torch.manual_seed(1)
    x = _rand((50, 64), 6, cuda)
    layer = mamtorch.nn.FullyConnected(64, 24, vcon_steps=4, relu_in=True).to(cuda)
    layer.vcon_step()  # beta 0.75
    y = layer(x)
    xr = torch.relu(x).cpu()
    y_ref, _, _ = mam_oracle.mam_forward(xr, layer.weight.detach().T.contiguous().cpu(), layer.bias.detach().cpu(), 0.75)
    np.testing.assert_allclose(y.detach().cpu().numpy(), y_ref.numpy(), rtol=1e-3, atol=1e-3 * float(y_ref.abs().max()))
    y.sum().backward()
    assert layer.weight.grad is not None and torch.isfinite(layer.weight.grad).all()
    # K cut into 3 slices: the sum of the three per-slice (max+min) terms
    sp = mamtorch.nn.FullyConnected(64, 24, splits=3, bias=False).to(cuda)
    ys = sp(x)
    w = sp.weight.detach().cpu()
    want = 0
    for s0, width in [(0, 22), (22, 22), (44, 20)]:
        part, _, _ = mam_oracle.mam_forward(x.cpu()[:, s0:s0 + width], w[:, s0:s0 + width].T.contiguous())
        want = want + part
    np.testing.assert_allclose(ys.detach().cpu().numpy(), want.numpy(), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("case", [(300, 768, 200, 3, True, 0), (129, 200, 65, 2, False, 0), (64, 1024, 130, 4, True, 3),
                                  (77, 96, 40, 3, True, 0), (90, 520, 31, 5, False, 0), (70, 156, 50, 5, True, 0)])
def test_split_module_in_one_launch_equals_the_slice_by_slice_sum(case, cuda):
    """Inference with `splits` > 1: one launch where every slice width is a multiple of 32 (an empty result
    tells the module to go slice by slice: (200, 2) has 100-wide slices), bit for bit the ordered sum of the
    per-slice oracle outputs, also under the beta blend and with the ragged last slice."""
    import mamtorch_b200 as mamtorch

    M, K, N, splits, bias, vsteps = case
    torch.manual_seed(K + splits)
    layer = mamtorch.nn.FullyConnected(K, N, splits=splits, bias=bias, vcon_steps=4 if vsteps else 0).to(cuda)
    for _ in range(vsteps):
        layer.vcon_step()
    x = _rand((M, K), K, cuda)
    layer.eval()
    with torch.no_grad():
        y = layer(x)
    sub = -(-K // splits)
    fused = torch.ops.mamtorch_b200.linear_forward_splits(x, layer.weight.detach(), None, None, 1.0, 0.0, sub)
    assert (fused.dim() == 2) == (sub % 32 == 0 and K % 4 == 0)
    w = layer.weight.detach().cpu()
    want = None
    for s0 in range(0, K, sub):
        part, _, _ = mam_oracle.mam_forward(x.cpu()[:, s0:s0 + sub], w[:, s0:s0 + sub].T.contiguous())
        want = part if want is None else want + part
    if fused.dim() == 2:
        assert torch.equal(fused.cpu(), want)
    if vsteps:
        want = float(layer.alpha) * want + float(layer.beta) * (x.cpu() @ w.T)
        if bias:
            want = want + layer.bias.detach().cpu()
        np.testing.assert_allclose(y.cpu().numpy(), want.numpy(), rtol=2e-3, atol=2e-3 * float(want.abs().max()))
    else:
        if bias:
            want = want + layer.bias.detach().cpu()
        assert torch.equal(y.cpu(), want)
    # training mode goes slice by slice with indices and must give the same values
    layer.train()
    yt = layer(x)
    if vsteps:
        np.testing.assert_allclose(yt.detach().cpu().numpy(), y.cpu().numpy(), rtol=1e-5, atol=1e-5)
    else:
        assert torch.equal(yt.detach(), y)


def test_v1_module_and_mamdense(cuda):
    import mamtorch_b200 as mamtorch

    x = _rand((9, 32), 7, cuda)
    for layer in (mamtorch.nn.v1.FullyConnected(32, 12).to(cuda), mamtorch.MAMDense(32, 12).to(cuda)):
        y = layer(x)
        bias = layer.bias.detach().cpu()
        y_ref, imax, imin = mam_oracle.mam_forward(x.cpu(), layer.weight.detach().T.contiguous().cpu(), bias)
        assert torch.equal(y.detach().cpu(), y_ref)
        assert torch.equal(layer.argmax.cpu().long(), imax)
        layer.update_selection_count()
        assert int(layer.max_selection_count.sum()) > 0


def test_conv2d_matches_im2col_oracle(cuda):
    import mamtorch_b200 as mamtorch

    torch.manual_seed(2)
    conv = mamtorch.nn.MAMConv2d(5, 7, 3, padding=1).to(cuda)
    x = _rand((2, 5, 9, 8), 8, cuda).requires_grad_()
    y = conv(x)
    y_ref, imax_ref, imin_ref = mam_oracle.mam_conv2d_forward(x.detach().cpu(), conv.weight.detach().cpu(),
                                                              conv.bias.detach().cpu(), stride=1, padding=1)
    assert y.shape == (2, 7, 9, 8)
    assert torch.equal(y.detach().cpu(), y_ref)
    assert torch.equal(conv.argmax.cpu().long(), imax_ref) and torch.equal(conv.argmin.cpu().long(), imin_ref)
    y.sum().backward()
    assert x.grad.shape == x.shape and conv.weight.grad.shape == conv.weight.shape
    # gradient check against autograd through the oracle's selected products
    xw = x.detach().cpu().requires_grad_()
    ww = conv.weight.detach().cpu().requires_grad_()
    rows = mam_oracle.conv2d_as_rows(xw, (3, 3), padding=1)
    wf = ww.reshape(7, -1)
    im = imax_ref.permute(0, 2, 3, 1).reshape(-1, 7)
    imn = imin_ref.permute(0, 2, 3, 1).reshape(-1, 7)
    r = torch.arange(rows.shape[0])[:, None].expand_as(im)
    c = torch.arange(7)[None, :].expand_as(im)
    (rows[r, im] * wf[c, im] + rows[r, imn] * wf[c, imn]).sum().backward()
    assert_grad_close(x.grad.cpu().numpy(), xw.grad.numpy())
    assert_grad_close(conv.weight.grad.cpu().numpy(), ww.grad.numpy())
    conv.update_selection_count()
    assert conv.max_selection_count.shape == conv.weight.shape and int(conv.max_selection_count.sum()) > 0


def test_conv1d(cuda):
    """MAMConv1d against the convolution oracle on the input with a height of one: all values, all indices
    (k = c*kW + kw in both), gradients through the oracle's selected products, and the selection count."""
    import mamtorch_b200 as mamtorch

    torch.manual_seed(4)
    conv = mamtorch.nn.MAMConv1d(4, 6, 3, padding=1, bias=True).to(cuda)
    x = _rand((3, 4, 11), 9, cuda).requires_grad_()
    y = conv(x)
    w4 = conv.weight.detach().cpu().unsqueeze(2)                       # [F,C,1,kW]
    y_ref, imax_ref, imin_ref = mam_oracle.mam_conv2d_forward(x.detach().cpu().unsqueeze(2), w4, conv.bias.detach().cpu(),
                                                              stride=1, padding=(0, 1))
    assert y.shape == (3, 6, 11)
    assert torch.equal(y.detach().cpu(), y_ref.squeeze(2))
    assert torch.equal(conv.argmax.cpu().long(), imax_ref.squeeze(2))
    assert torch.equal(conv.argmin.cpu().long(), imin_ref.squeeze(2))
    gy = _rand((3, 6, 11), 10, cuda)
    y.backward(gy)
    xw = x.detach().cpu().requires_grad_()
    ww = conv.weight.detach().cpu().requires_grad_()
    rows = mam_oracle.conv2d_as_rows(xw.unsqueeze(2), (1, 3), padding=(0, 1))
    wf = ww.reshape(6, -1)
    im = imax_ref.permute(0, 2, 3, 1).reshape(-1, 6)
    imn = imin_ref.permute(0, 2, 3, 1).reshape(-1, 6)
    r = torch.arange(rows.shape[0])[:, None].expand_as(im)
    c = torch.arange(6)[None, :].expand_as(im)
    ((rows[r, im] * wf[c, im] + rows[r, imn] * wf[c, imn]) * gy.cpu().permute(0, 2, 1).reshape(-1, 6)).sum().backward()
    assert_grad_close(x.grad.cpu().numpy(), xw.grad.numpy())
    assert_grad_close(conv.weight.grad.cpu().numpy(), ww.grad.numpy())
    # the convolution modules keep the two counts apart (mamtorch/nn/backup/mamconv2d.txt:90-114): +1 per call for
    # every weight some output pixel selected as max, likewise for min
    conv.update_selection_count()
    hmax, hmin = mam_oracle.selection_hits(im, imn, 12)
    assert torch.equal(conv.max_selection_count.cpu().reshape(6, 12), (hmax > 0).int())
    assert torch.equal(conv.min_selection_count.cpu().reshape(6, 12), (hmin > 0).int())


def test_conv2d_selection_count_against_the_oracle(cuda):
    import mamtorch_b200 as mamtorch

    torch.manual_seed(5)
    conv = mamtorch.nn.MAMConv2d(5, 7, 3, padding=1, stride=2).to(cuda)
    x = _rand((2, 5, 9, 8), 12, cuda)
    conv(x)
    conv.update_selection_count()
    conv(x * -1.5)
    conv.update_selection_count()
    want_max = torch.zeros(7, 45, dtype=torch.int32)
    want_min = torch.zeros(7, 45, dtype=torch.int32)
    for xs in (x, x * -1.5):
        _, imax, imin = mam_oracle.mam_conv2d_forward(xs.cpu(), conv.weight.detach().cpu(), conv.bias.detach().cpu(),
                                                      stride=2, padding=1)
        hmax, hmin = mam_oracle.selection_hits(imax.permute(0, 2, 3, 1).reshape(-1, 7),
                                               imin.permute(0, 2, 3, 1).reshape(-1, 7), 45)
        want_max += (hmax > 0).int()      # +1 per call and weight, max and min kept apart
        want_min += (hmin > 0).int()      # (mamtorch/nn/backup/mamconv2d.txt:90-114)
    assert torch.equal(conv.max_selection_count.cpu().reshape(7, 45), want_max)
    assert torch.equal(conv.min_selection_count.cpu().reshape(7, 45), want_min)


def test_store_args_before_the_first_vcon_step(cuda):
    """While beta is still 1 (every layer with vcon_steps > 0 starts there) the output is the dense term alone,
    but the indices are stored all the same, as in the reference (mamtorch/nn/v4/fullyconnected.py:178-186), so a
    loop that updates the counts from step 0 works."""
    import mamtorch_b200 as mamtorch

    torch.manual_seed(6)
    layer = mamtorch.nn.FullyConnected(48, 20, vcon_steps=4, store_args=True).to(cuda)
    assert layer.beta == 1.0
    x = _rand((9, 48), 13, cuda)
    y = layer(x)
    _, imax_ref, imin_ref = mam_oracle.mam_forward(x.cpu(), layer.weight.detach().T.contiguous().cpu())
    assert torch.equal(layer.argmax.cpu().long(), imax_ref) and torch.equal(layer.argmin.cpu().long(), imin_ref)
    want_y = x.cpu() @ layer.weight.detach().cpu().T + layer.bias.detach().cpu()
    assert torch.allclose(y.detach().cpu(), want_y, rtol=1e-5, atol=1e-5)
    layer.update_selection_count()
    want = mam_oracle.selection_count_update(torch.zeros(20, 48, dtype=torch.int32), imax_ref, imin_ref)
    assert torch.equal(layer.max_selection_count.cpu(), want)


def test_device_flag_checks_are_exposed_to_torch_users(cuda):
    """`check_device_flag` (waits for the device) and `poll_device_flag` (does not) are operators of the package;
    after healthy launches neither raises."""
    import mamtorch_b200 as mamtorch
    from mamtorch_b200.nn import functional as MF

    layer = mamtorch.nn.FullyConnected(64, 32, store_args=True).to(cuda)
    layer(_rand((40, 64), 14, cuda)).sum().backward()
    layer.update_selection_count()
    MF.poll_device_flag()
    torch.cuda.synchronize()
    MF.poll_device_flag()
    MF.check_device_flag()
    torch.ops.mamtorch_b200.check_device_flag()


def test_beta_blended_training_step(cuda):
    """The blended-training configuration at reduced size (M=N=K=1024, beta=0.5, x and W with
    variance K^-0.5): the MAM term is bit-exact (checked through a beta=0 call on the same inputs
    and through the indices of the beta=0.5 call), the blended output and the gradients are within
    1e-3 relative of the fp32 oracle because the dense term runs in TF32 on the tensor cores."""
    import mamtorch_b200 as mamtorch
    from oracle import c_oracle

    M = N = K = 1024
    beta = 0.5
    g = torch.Generator().manual_seed(0)
    std = K ** -0.25
    x = torch.randn(M, K, generator=g) * std
    w = torch.randn(N, K, generator=g) * std
    gy = torch.randn(M, N, generator=g)
    b = w.T.contiguous()
    s_ref, imax_ref, imin_ref = c_oracle.forward(x.numpy(), w.numpy(), b_is_nk=True)
    zero_bias = torch.zeros(N, device=cuda)
    xd, bd = x.to(cuda), b.to(cuda)
    c0, imax0, imin0 = mamtorch.kernel.v3.fullyconnected(xd, bd, zero_bias, 0.0)
    assert torch.equal(c0.cpu(), torch.from_numpy(s_ref))
    c, imax, imin = mamtorch.kernel.v3.fullyconnected(xd, bd, zero_bias, beta)
    for got, ref in ((imax0, imax_ref), (imin0, imin_ref), (imax, imax_ref), (imin, imin_ref)):
        assert torch.equal(got.cpu().long(), torch.from_numpy(ref))
    y_ref = beta * (x.double() @ b.double()) + (1 - beta) * torch.from_numpy(s_ref).double()
    np.testing.assert_allclose(c.cpu().double().numpy(), y_ref.numpy(), rtol=1e-3, atol=1e-3 * float(y_ref.abs().max()))
    da, db = torch.ops.mamtorch_kernel_v3.fullyconnected_backward(xd, bd, gy.to(cuda), imax, imin, beta)
    da_m, dw_m = c_oracle.backward(x.numpy(), w.numpy(), gy.numpy(), imax_ref, imin_ref, b_is_nk=True)
    da_ref = beta * (gy.double() @ w.double()) + (1 - beta) * torch.from_numpy(da_m).double()
    db_ref = beta * (x.double().T @ gy.double()) + (1 - beta) * torch.from_numpy(dw_m).double().T
    assert_grad_close(da.cpu().numpy(), da_ref.numpy(), rtol=1e-3)
    assert_grad_close(db.cpu().numpy(), db_ref.numpy(), rtol=1e-3)


def test_beta_blended_configuration_full_size(cuda):
    """The blended-training configuration at its full size (M=N=K=4096, beta=0.5, x and W with
    variance K^-0.5).  Too large for the CPU oracle, so check what holds at any size: the MAM term of a
    beta=0 call equals the sum of the two products its indices point at, bit for bit; the beta=0.5 call
    returns the same indices; and its output is within 1e-3 relative of 0.5*MAM + 0.5*(x.W^T) with the
    product taken in full fp32."""
    import mamtorch_b200 as mamtorch

    M = N = K = 4096
    beta = 0.5
    g = torch.Generator().manual_seed(0)
    std = K ** -0.25
    x = (torch.randn(M, K, generator=g) * std).to(cuda)
    w = (torch.randn(N, K, generator=g) * std).to(cuda)
    b = w.T.contiguous()
    zero_bias = torch.zeros(N, device=cuda)
    c0, imax0, imin0 = mamtorch.kernel.v3.fullyconnected(x, b, zero_bias, 0.0)
    c, imax, imin = mamtorch.kernel.v3.fullyconnected(x, b, zero_bias, beta)
    assert torch.equal(imax, imax0) and torch.equal(imin, imin0)
    assert int(imax.min()) >= 0 and int(imax.max()) < K and int(imin.min()) >= 0 and int(imin.max()) < K
    cols = torch.arange(N, device=cuda)[None, :].expand(M, N)
    want = x.gather(1, imax.long()) * w[cols, imax.long()] + x.gather(1, imin.long()) * w[cols, imin.long()]
    assert torch.equal(c0, want)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        dense = x @ b
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    ref = beta * dense.double() + (1 - beta) * c0.double()
    err = (c.double() - ref).abs().max().item()
    assert err <= 1e-3 * ref.abs().max().item()


def test_conv_benchmark_shape_properties(cuda):
    """The convolution configuration at full size (input [128,64,56,56], 3x3, 64->128 channels,
    stride 1, pad 1: GEMM M=401408, K=576, N=128).  Too large for the CPU oracle, so check what holds
    at any size: the output equals the sum of the two selected products bit for bit, indices are in
    range, and a sample of pixels agrees with a direct evaluation of their patches."""
    import mamtorch_b200 as mamtorch

    g = torch.Generator().manual_seed(0)
    x = torch.randn(128, 64, 56, 56, generator=g).to(cuda)
    conv = mamtorch.nn.MAMConv2d(64, 128, 3, padding=1, bias=False).to(cuda)
    with torch.no_grad():
        conv.weight.copy_(torch.randn(128, 64, 3, 3, generator=g) * 576 ** -0.5)
        y = conv(x)
    assert y.shape == (128, 128, 56, 56)
    assert int(conv.argmax.min()) >= 0 and int(conv.argmax.max()) < 576
    xp = torch.nn.functional.pad(x, (1, 1, 1, 1))
    w = conv.weight.detach()
    for (b_, f, i, j) in [(0, 0, 0, 0), (127, 127, 55, 55), (64, 3, 17, 40), (5, 99, 55, 0)]:
        p = (xp[b_, :, i:i + 3, j:j + 3] * w[f]).reshape(-1)
        assert y[b_, f, i, j].item() == (p.max() + p.min()).item()
        assert conv.argmax[b_, f, i, j].item() == int(p.argmax()) and conv.argmin[b_, f, i, j].item() == int(p.argmin())
    # every output is the sum of the products its two indices point at
    rows = torch.nn.functional.unfold(x[:8], 3, padding=1).transpose(1, 2).reshape(-1, 576)
    wf = w.reshape(128, -1)
    im = conv.argmax[:8].permute(0, 2, 3, 1).reshape(-1, 128).long()
    imn = conv.argmin[:8].permute(0, 2, 3, 1).reshape(-1, 128).long()
    r = torch.arange(rows.shape[0], device=cuda)[:, None].expand_as(im)
    c = torch.arange(128, device=cuda)[None, :].expand_as(im)
    want = rows[r, im] * wf[c, im] + rows[r, imn] * wf[c, imn]
    assert torch.equal(y[:8].permute(0, 2, 3, 1).reshape(-1, 128), want)


def test_output_dropout_in_the_kernel_epilogue(cuda):
    """Training-mode output dropout rides in the forward epilogue: y = mask * (mam + bias) / (1 - p) with a mask
    that depends only on (seed, element), so the values-only and index-producing kernels, the any-shape kernel and
    `drop_apply` all form the same one; the backward routes mask * gy / (1 - p) through the selected pairs."""
    from mamtorch_b200.nn import functional as MF

    ops = torch.ops.mamtorch_b200
    p, seed = 0.3, 123456789
    for (M, K, N) in ((300, 96, 200), (70, 65, 66)):          # tiled kernels / any-shape kernel (K % 4 != 0)
        x, w, bias = _rand((M, K), 20, cuda), _rand((N, K), 21, cuda, K ** -0.5), _rand((N,), 22, cuda)
        y0, imax0, imin0 = ops.linear_forward(x, w, bias, None, 1.0, 0.0, True)
        y1, imax1, imin1 = ops.linear_forward_drop(x, w, bias, None, 1.0, 0.0, True, p, seed)
        y2, = ops.linear_forward_drop(x, w, bias, None, 1.0, 0.0, False, p, seed)
        mask = ops.drop_apply(torch.ones_like(y0), p, 1.0, seed)
        assert set(mask.unique().tolist()) == {0.0, 1.0}
        assert abs(float(mask.mean()) - (1 - p)) < 0.02
        want = mask * (y0 * (1.0 / (1.0 - p)))
        assert torch.equal(y1, want) and torch.equal(y2, want)
        assert torch.equal(imax1, imax0) and torch.equal(imin1, imin0)
        other = ops.drop_apply(torch.ones_like(y0), p, 1.0, seed + 1)
        assert not torch.equal(other, mask)
        # autograd: the same function written with the explicit mask
        xa, wa = x.clone().requires_grad_(), w.clone().requires_grad_()
        xb, wb = x.clone().requires_grad_(), w.clone().requires_grad_()
        gy = _rand((M, N), 23, cuda)
        ya, _, _ = MF.mam_linear(xa, wa, bias, drop_rate=p, drop_seed=seed)
        yb, _, _ = MF.mam_linear(xb, wb, bias)
        ya.backward(gy)
        (yb * mask * (1.0 / (1.0 - p))).backward(gy)
        assert torch.equal(ya, want)
        assert_grad_close(xa.grad.cpu().numpy(), xb.grad.cpu().numpy())
        assert_grad_close(wa.grad.cpu().numpy(), wb.grad.cpu().numpy())


def test_module_weight_drop_and_output_dropout(cuda):
    """FullyConnected with wdrop_rate and drop_rate: in training both masks come from the library's generator
    (reproducible under torch.manual_seed, different from call to call), weight drop is unscaled as in the
    reference (mamtorch/nn/v4/fullyconnected.py:143-148), dropped weights and dropped outputs get no gradient;
    in eval mode the layer is the plain one."""
    import mamtorch_b200 as mamtorch
    from mamtorch_b200.nn import functional as MF

    torch.manual_seed(7)
    layer = mamtorch.nn.FullyConnected(128, 96, wdrop_rate=0.25, drop_rate=0.4).to(cuda)
    plain = mamtorch.nn.FullyConnected(128, 96).to(cuda)
    plain.load_state_dict(layer.state_dict())
    x = _rand((50, 128), 30, cuda)
    layer.eval()
    plain.eval()
    assert torch.equal(layer(x), plain(x))
    layer.train()
    torch.manual_seed(99)
    y1 = layer(x)
    torch.manual_seed(99)
    y2 = layer(x)
    y3 = layer(x)
    assert torch.equal(y1, y2) and not torch.equal(y1, y3)
    frac_zero = float((y1 == 0).float().mean())
    assert abs(frac_zero - 0.4) < 0.05
    # the two pieces on their own
    w = layer.weight.detach()
    wd = MF.weight_drop(w, 0.25, seed=5)
    kept = wd != 0
    assert torch.equal(wd[kept], w[kept]) and abs(float(kept.float().mean()) - 0.75) < 0.02
    wr = w.clone().requires_grad_()
    MF.weight_drop(wr, 0.25, seed=5).sum().backward()
    assert torch.equal(wr.grad, kept.float())
    # gradients flow and dropped outputs contribute nothing
    xg = x.clone().requires_grad_()
    torch.manual_seed(99)
    yg = layer(xg)
    yg.backward(torch.ones_like(yg))
    assert torch.equal(yg, y1) and xg.grad.shape == x.shape and layer.weight.grad.shape == layer.weight.shape
    assert float(layer.bias.grad.min()) >= 0 and abs(float(layer.bias.grad.sum()) - float((y1 != 0).sum()) / 0.6) < 1.0


@pytest.mark.parametrize("shape,splits", [((200, 256, 130), 2), ((300, 768, 200), 4), ((70, 160, 66), 3), ((129, 96, 40), 2)])
def test_training_splits_in_one_launch(shape, splits, cuda):
    """`splits` in training: every slice of K contributes its own max + min and routes gradients through its own
    selected pairs (mamtorch/nn/v4/fullyconnected.py:164-176).  One launch for all slices must equal the
    slice-by-slice composition: values and per-slice indices bit for bit (against the oracle on each slice),
    gradients to rounding.  (160 / 3 -> slices of 54: not a multiple of 32, the module goes slice by slice.)"""
    import math

    import mamtorch_b200 as mamtorch
    from mamtorch_b200.nn import functional as MF

    M, K, N = shape
    width = math.ceil(K / splits)
    x, w, bias = _rand((M, K), 40, cuda), _rand((N, K), 41, cuda, K ** -0.5), _rand((N,), 42, cuda)
    gy = _rand((M, N), 43, cuda)
    # oracle: slice by slice
    y_ref = torch.zeros(M, N)
    idx_ref = []
    for s0 in range(0, K, width):
        ys, imax, imin = mam_oracle.mam_forward(x[:, s0:s0 + width].cpu(), w[:, s0:s0 + width].T.contiguous().cpu())
        y_ref = ys if s0 == 0 else y_ref + ys
        idx_ref.append((imax + s0, imin + s0))
    y_ref = y_ref + bias.cpu()
    out = torch.ops.mamtorch_b200.linear_forward_splits_idx(x, w, bias, None, 1.0, 0.0, width)
    if width % 32 == 0:
        y, amax, amin = out
        assert amax.shape == (len(idx_ref), M, N)
        assert torch.equal(y.cpu(), y_ref)
        for s, (imax, imin) in enumerate(idx_ref):
            assert torch.equal(amax[s].cpu().long(), imax) and torch.equal(amin[s].cpu().long(), imin)
        da, dw = torch.ops.mamtorch_b200.linear_backward_splits(x, w, gy, amax, amin, 1.0)
        da_ref = torch.zeros(M, K, dtype=torch.float64)
        dw_ref = torch.zeros(N, K, dtype=torch.float64)
        for imax, imin in idx_ref:
            a_, b_ = mam_oracle.mam_backward(x.cpu(), w.T.contiguous().cpu(), gy.cpu(), imax, imin)
            da_ref += a_.double()
            dw_ref += b_.T.double()
        assert_grad_close(da.cpu().numpy(), da_ref.numpy())
        assert_grad_close(dw.cpu().numpy(), dw_ref.numpy())
    else:
        assert len(out) == 0 and MF.mam_linear_splits(x, w, width, bias) is None
    # the module, in training mode, whichever route it takes
    torch.manual_seed(1)
    layer = mamtorch.nn.FullyConnected(K, N, splits=splits).to(cuda).train()
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.bias.copy_(bias)
    xg = x.clone().requires_grad_()
    ym = layer(xg)
    ym.backward(gy)
    assert torch.allclose(ym.detach().cpu(), y_ref, rtol=1e-6, atol=1e-6) if width % 32 else torch.equal(ym.detach().cpu(), y_ref)
    da_ref = torch.zeros(M, K, dtype=torch.float64)
    dw_ref = torch.zeros(N, K, dtype=torch.float64)
    for imax, imin in idx_ref:
        a_, b_ = mam_oracle.mam_backward(x.cpu(), w.T.contiguous().cpu(), gy.cpu(), imax, imin)
        da_ref += a_.double()
        dw_ref += b_.T.double()
    assert_grad_close(xg.grad.cpu().numpy(), da_ref.numpy())
    assert_grad_close(layer.weight.grad.cpu().numpy(), dw_ref.numpy())
    assert_grad_close(layer.bias.grad.cpu().numpy(), gy.sum(0).cpu().numpy())
    torch.ops.mamtorch_b200.check_device_flag()
