"""The reference's ViT call pattern on the B200 kernels: dense layers of a transformer MLP block
swapped for MAM layers (examples/vitb16_imagenet1k/utils.py:67-77), the vanishing-contribution
schedule stepped for all of them (vit_training.py:521-524), and one training step captured in a
CUDA graph.  Synthetic tokens and random-init weights: no checkpoint or dataset is involved."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close
from oracle import c_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture()
def fp32_dense():
    from mamtorch_b200.nn import functional as MF

    MF.set_dense_backend("fp32")
    yield
    MF.set_dense_backend("auto")


def test_swapped_hf_vit_starts_dense_and_ends_mam(cuda, fp32_dense):
    transformers = pytest.importorskip("transformers")
    from mamtorch_b200.nn import vit as mv

    cfg = transformers.ViTConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                                 image_size=32, patch_size=8, num_labels=10)
    torch.manual_seed(0)
    model = transformers.ViTForImageClassification(cfg).to(cuda).eval()
    pix = torch.randn(3, 3, 32, 32, generator=torch.Generator().manual_seed(1)).to(cuda)
    with torch.no_grad():
        ref_logits = model(pixel_values=pix).logits
    paths = mv.mlp_dense_paths(num_layers=2)
    assert paths == ["vit.encoder.layer.0.intermediate.dense", "vit.encoder.layer.1.intermediate.dense",
                     "vit.encoder.layer.0.output.dense", "vit.encoder.layer.1.output.dense"]
    mv.swap_linear_for_mam(model, paths, vcon_steps=4)
    layers = mv.mam_layers(model)
    assert len(layers) == 4 and all(l.beta == 1.0 and l.alpha == 0.0 for l in layers)
    # beta = 1: every swapped layer still computes the dense layer it replaced
    with torch.no_grad():
        logits = model(pixel_values=pix).logits
    np.testing.assert_allclose(logits.cpu().numpy(), ref_logits.cpu().numpy(), rtol=1e-5, atol=1e-5)
    for _ in range(4):
        mv.vcon_step_all(model)
    assert all(l.beta == 0 and l.alpha == 1.0 for l in layers)
    # beta = 0: every swapped layer is a pure MAM layer; check each against the oracle on the
    # input it actually received
    seen = []
    hooks = [l.register_forward_hook(lambda m, inp, out: seen.append((m, inp[0].detach(), out.detach()))) for l in layers]
    with torch.no_grad():
        model(pixel_values=pix)
    for h in hooks:
        h.remove()
    assert len(seen) == 4
    for m, x, y in seen:
        y_ref, _, _ = c_oracle.forward(x.reshape(-1, x.size(-1)).cpu().numpy(), m.weight.detach().cpu().numpy(),
                                       b_is_nk=True, bias=m.bias.detach().cpu().numpy())
        assert np.array_equal(y.reshape(y_ref.shape).cpu().numpy(), y_ref)


def test_mlp_block_matches_oracle_composition(cuda):
    from mamtorch_b200.nn.vit import MAMMlpBlock

    torch.manual_seed(3)
    blk = MAMMlpBlock(hidden=64, intermediate=160).to(cuda)
    x = torch.randn(2, 37, 64, generator=torch.Generator().manual_seed(4)).to(cuda)
    y = blk(x)
    h = torch.nn.functional.layer_norm(x, (64,), blk.norm.weight, blk.norm.bias, blk.norm.eps)
    h1, _, _ = c_oracle.forward(h.reshape(-1, 64).detach().cpu().numpy(), blk.fc1.weight.detach().cpu().numpy(),
                                b_is_nk=True, bias=blk.fc1.bias.detach().cpu().numpy())
    g = torch.nn.functional.gelu(torch.from_numpy(h1).to(cuda))
    h2, _, _ = c_oracle.forward(g.cpu().numpy(), blk.fc2.weight.detach().cpu().numpy(), b_is_nk=True,
                                bias=blk.fc2.bias.detach().cpu().numpy())
    expect = x + torch.from_numpy(h2).to(cuda).view_as(x)
    assert torch.equal(y.detach(), expect)


def test_graphed_step_replays_forward_and_backward(cuda):
    from mamtorch_b200.nn.vit import GraphedStep, MAMMlpBlock

    torch.manual_seed(5)
    blk = MAMMlpBlock(hidden=64, intermediate=128, store_args=True).to(cuda)
    g = torch.Generator().manual_seed(6)
    x0, gy0 = torch.randn(4, 50, 64, generator=g).to(cuda), torch.randn(4, 50, 64, generator=g).to(cuda)
    step = GraphedStep(blk, x0, gy0)
    import copy

    eager = copy.deepcopy(blk)   # same weights, its own .grad tensors
    for trial in range(2):   # two different inputs through the same captured graph
        x, gy = torch.randn(4, 50, 64, generator=g).to(cuda), torch.randn(4, 50, 64, generator=g).to(cuda)
        y = step(x, gy)
        for p in eager.parameters():
            p.grad = None
        xe = x.clone().requires_grad_()
        ye = eager(xe)
        ye.backward(gy)
        assert torch.equal(y, ye.detach())
        assert_grad_close(step.grad_input.cpu().numpy(), xe.grad.cpu().numpy())
        for (n, p), (_, pe) in zip(blk.named_parameters(), eager.named_parameters()):
            assert_grad_close(p.grad.cpu().numpy(), pe.grad.cpu().numpy())
    # the indices of the last replay are visible on the layers, as in eager mode
    assert torch.equal(blk.fc1.argmax, eager.fc1.argmax) and torch.equal(blk.fc2.argmin, eager.fc2.argmin)
