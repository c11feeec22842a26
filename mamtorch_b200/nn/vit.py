"""Putting MAM layers into a transformer MLP block, the way the reference's ViT example does it.

The reference fine-tunes a Hugging Face ViT-B/16 after replacing the two dense layers of every MLP
block (`vit.encoder.layer.{i}.intermediate.dense`, `.output.dense`) by `mamtorch.nn.FullyConnected`
that start from the dense weights (`examples/vitb16_imagenet1k/utils.py:23-77`), and steps the
vanishing-contribution schedule of every MAM layer once per optimiser step
(`examples/vitb16_imagenet1k/vit_training.py:521-524`).  This module carries that call pattern,
without the example's dependence on a checkpoint or a dataset:

  * `swap_linear_for_mam` / `mlp_dense_paths`  the layer replacement (works on any module tree);
  * `vcon_step_all`                            one schedule step for every MAM layer of a model;
  * `MAMMlpBlock`                              LayerNorm -> MAM(d, 4d) -> GELU -> MAM(4d, d) + residual,
                                               the MLP half of a ViT encoder layer, for runs on
                                               synthetic tokens;
  * `GraphedStep`                              forward + backward of a module captured in one CUDA
                                               graph on static buffers (the kernels take the current
                                               stream and allocate through torch's caching allocator,
                                               so they capture like any other torch operator).
"""
from __future__ import annotations

import torch
from torch import nn

from .v4.fullyconnected import FullyConnected

__all__ = ["mlp_dense_paths", "swap_linear_for_mam", "vcon_step_all", "mam_layers", "MAMMlpBlock", "GraphedStep"]


def mlp_dense_paths(num_layers: int = 12, intermediate: bool = True, output: bool = True,
                    prefix: str = "vit.encoder.layer") -> list[str]:
    """Attribute paths of the MLP dense layers of a Hugging Face ViT, as `generate_paths` builds
    them in the reference (`examples/vitb16_imagenet1k/utils.py:23-48`).  A negative `num_layers`
    selects the last |num_layers| of 12 encoder layers, as there."""
    layers = range(num_layers) if num_layers >= 0 else range(12 + num_layers, 12)
    paths = []
    if intermediate:
        paths += [f"{prefix}.{i}.intermediate.dense" for i in layers]
    if output:
        paths += [f"{prefix}.{i}.output.dense" for i in layers]
    return paths


def _resolve(model: nn.Module, path: str):
    parent = model
    parts = path.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    return parent, parts[-1]


def swap_linear_for_mam(model: nn.Module, paths, vcon_steps: int = 0, vcon_type: str = "linear", splits: int = 1,
                        train_mam_only: bool = False, **mam_kwargs) -> nn.Module:
    """Replaces the `nn.Linear` at every path by a `FullyConnected` that takes over its weight and
    bias (`add_mam_to_ViT`, `examples/vitb16_imagenet1k/utils.py:67-77`).  With `vcon_steps > 0` the
    new layers start as the dense layers they replace (beta = 1) and turn into MAM layers over that
    many `vcon_step()` calls."""
    for path in paths:
        parent, attr = _resolve(model, path)
        lin = getattr(parent, attr)
        if not isinstance(lin, nn.Linear):
            raise TypeError(f"{path} is a {type(lin).__name__}, not an nn.Linear")
        mam = FullyConnected(lin.in_features, lin.out_features, bias=lin.bias is not None, vcon_steps=vcon_steps,
                             vcon_type=vcon_type, splits=splits, train_mam_only=train_mam_only,
                             device=lin.weight.device, dtype=lin.weight.dtype, **mam_kwargs)
        mam.weight.data = lin.weight.data
        if lin.bias is not None:
            mam.bias.data = lin.bias.data
        setattr(parent, attr, mam)
    return model


def mam_layers(model: nn.Module):
    """Every MAM fully-connected layer of a model, in module order."""
    return [m for m in model.modules() if isinstance(m, FullyConnected)]


def vcon_step_all(model: nn.Module) -> None:
    """One step of the vanishing-contribution schedule on every MAM layer: what the reference's
    training loop does after each optimiser step (`vit_training.py:521-524`)."""
    for layer in mam_layers(model):
        layer.vcon_step()


class MAMMlpBlock(nn.Module):
    """The MLP half of a pre-norm transformer encoder layer with MAM dense layers:
    x + MAM_2(GELU(MAM_1(LayerNorm(x)))), shapes [..., hidden] -> [..., hidden].

    ViT-B/16: hidden 768, intermediate 3072, 197 tokens per image."""

    def __init__(self, hidden: int = 768, intermediate: int = 3072, vcon_steps: int = 0, vcon_type: str = "linear",
                 store_args: bool = False, residual: bool = True, layer_norm_eps: float = 1e-12, device=None,
                 dtype=None):
        super().__init__()
        self.norm = nn.LayerNorm(hidden, eps=layer_norm_eps, device=device, dtype=dtype)
        self.fc1 = FullyConnected(hidden, intermediate, vcon_steps=vcon_steps, vcon_type=vcon_type,
                                  store_args=store_args, device=device, dtype=dtype)
        self.act = nn.GELU()
        self.fc2 = FullyConnected(intermediate, hidden, vcon_steps=vcon_steps, vcon_type=vcon_type,
                                  store_args=store_args, device=device, dtype=dtype)
        self.residual = residual

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.fc2(self.act(self.fc1(self.norm(x))))
        return x + y if self.residual else y

    def vcon_step(self) -> None:
        self.fc1.vcon_step()
        self.fc2.vcon_step()


class GraphedStep:
    """Forward + backward of `module` on inputs of one fixed shape, captured once in a CUDA graph.

        step = GraphedStep(block, example_x, example_grad_out)
        y = step(x, grad_out)          # replays: y, step.grad_input and the parameters' .grad are refreshed

    Parameter gradients are written into the same `.grad` tensors on every replay (zeroed inside the
    graph), so an optimiser can read them after the call.  The blend weights alpha / beta of a MAM
    layer are kernel arguments and therefore frozen into the graph: capture after the
    vanishing-contribution schedule has ended, or call `recapture()` after each `vcon_step()`.
    """

    def __init__(self, module: nn.Module, example_input: torch.Tensor, example_grad_output: torch.Tensor,
                 warmup: int = 3):
        if not example_input.is_cuda:
            raise ValueError("GraphedStep needs CUDA tensors")
        self.module = module
        self.x = example_input.detach().clone().requires_grad_()
        self.gy = example_grad_output.detach().clone()
        self.warmup = warmup
        self.graph = None
        self.y = None
        self.grad_input = None
        self.recapture()

    def _run(self):
        for p in self.module.parameters():
            if p.grad is not None:
                p.grad.zero_()
        if self.x.grad is not None:
            self.x.grad.zero_()
        y = self.module(self.x)
        y.backward(self.gy)
        return y

    def recapture(self) -> None:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.warmup):   # allocates the .grad tensors and warms the allocator
                self._run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            y = self._run()
        self.y = y.detach()
        self.grad_input = self.x.grad

    def __call__(self, x: torch.Tensor, grad_output: torch.Tensor) -> torch.Tensor:
        self.x.data.copy_(x)
        self.gy.copy_(grad_output)
        self.graph.replay()
        return self.y
