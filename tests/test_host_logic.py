"""Host-side logic that needs no device: the ViT layer-swap helpers, the pruning thresholds and masks,
the module's vanishing-contribution schedule, and argument checks of the newer C-ABI entry points."""
import ctypes
import math

import pytest
import torch
from torch import nn

from mamtorch_b200 import _lib
from mamtorch_b200.nn import FullyConnected
from mamtorch_b200.nn import vit as mv
from mamtorch_b200.sparse import (PrunedFullyConnected, global_magnitude_threshold, magnitude_keep_mask,
                                  magnitude_threshold)


def test_mlp_dense_paths_follow_the_reference_naming():
    assert mv.mlp_dense_paths(2) == ["vit.encoder.layer.0.intermediate.dense", "vit.encoder.layer.1.intermediate.dense",
                                     "vit.encoder.layer.0.output.dense", "vit.encoder.layer.1.output.dense"]
    assert mv.mlp_dense_paths(-1, output=False) == ["vit.encoder.layer.11.intermediate.dense"]
    assert mv.mlp_dense_paths(1, intermediate=False, prefix="enc") == ["enc.0.output.dense"]


class _Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.block = nn.ModuleDict({"fc1": nn.Linear(6, 10), "act": nn.ReLU(), "fc2": nn.Linear(10, 4, bias=False)})
        self.norm = nn.LayerNorm(4)


def test_swap_takes_over_weights_and_schedule_steps_every_layer():
    torch.manual_seed(0)
    m = _Tiny()
    w1, b1, w2 = m.block["fc1"].weight.data, m.block["fc1"].bias.data, m.block["fc2"].weight.data
    mv.swap_linear_for_mam(m, ["block.fc1", "block.fc2"], vcon_steps=4, vcon_type="linear")
    l1, l2 = m.block["fc1"], m.block["fc2"]
    assert isinstance(l1, FullyConnected) and isinstance(l2, FullyConnected)
    assert l1.weight.data_ptr() == w1.data_ptr() and l1.bias.data_ptr() == b1.data_ptr()
    assert l2.weight.data_ptr() == w2.data_ptr() and l2.bias is None
    assert mv.mam_layers(m) == [l1, l2]
    assert (l1.beta, l1.alpha) == (1.0, 0.0)
    for expect in (0.75, 0.5, 0.25, 0.0):
        mv.vcon_step_all(m)
        assert l1.beta == pytest.approx(expect) and l2.beta == pytest.approx(expect)
        assert l1.alpha == pytest.approx(1.0 - expect)
    mv.vcon_step_all(m)   # stays at zero
    assert l1.beta == 0 and l1.alpha == 1.0
    with pytest.raises(TypeError):
        mv.swap_linear_for_mam(m, ["norm"])


def test_exponential_schedule_reaches_eps_after_its_steps():
    layer = FullyConnected(4, 3, vcon_steps=10, vcon_type="exponential", vcon_eps=1e-3)
    for _ in range(9):
        layer.vcon_step()
    assert layer.beta == pytest.approx(math.exp(math.log(1e-3) * 0.9))
    layer.vcon_step()
    assert layer.beta == 0 and layer.alpha == 1.0


def test_magnitude_thresholds_and_masks_match_the_reference_rule():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(40, 30, generator=g)
    for p in (0.0, 0.3, 0.9, 1.0):
        thr = magnitude_threshold(w, p)
        assert torch.equal(thr, torch.quantile(w.flatten().abs(), p))
        keep = magnitude_keep_mask(w, thr)
        zeroed = w.clone()
        zeroed[zeroed.abs() <= thr] = 0          # examples/vitb16_imagenet1k/pruning_utils.py:105-107
        assert torch.equal(w * keep, zeroed)
    w2 = torch.randn(10, 30, generator=g) * 3
    # the global rule is the reference's literal one: sorted magnitudes, element int(p * n), clamped
    # (examples/vitb16_imagenet1k/pruning_utils.py:147-151)
    both = torch.cat([w.flatten().abs(), w2.flatten().abs()]).sort().values
    for p in (0.0, 0.37, 0.5, 1.0):
        thr_g = global_magnitude_threshold([w, w2], p)
        assert torch.equal(thr_g, both[max(0, min(int(p * len(both)), len(both) - 1))])
    with pytest.raises(ValueError):
        magnitude_threshold(w, 1.5)


def test_pruned_layer_bookkeeping_on_cpu():
    torch.manual_seed(2)
    lin = nn.Linear(20, 12)
    layer = PrunedFullyConnected.from_dense(lin, fraction=0.75)
    assert torch.equal(layer.weight.detach(), lin.weight.detach()) and torch.equal(layer.bias.detach(), lin.bias.detach())
    assert abs(layer.sparsity() - 0.75) <= 1.0 / lin.weight.numel() + 1e-6
    csr = layer._weight_csr()
    assert csr.layout == torch.sparse_csr and csr.values().numel() == int(layer.keep_mask.sum())
    assert layer._weight_csr() is csr
    layer.prune_(threshold=float("inf"))
    assert layer.sparsity() == 1.0 and layer._weight_csr().values().numel() == 0
    with pytest.raises(ValueError):
        layer.prune_()


def test_newer_entry_points_reject_bad_arguments_without_a_device():
    L = _lib.lib()
    null = None
    one = ctypes.c_void_p(16)   # never dereferenced: every call below fails its argument check first
    assert L.mam_csr_fwd_workspace_bytes(0, 64, 64, 10) == 0
    assert L.mam_csr_fwd_workspace_bytes(16, 64, 64, 10) == 0            # fewer than 32 rows: lane-per-entry kernel
    need = L.mam_csr_fwd_workspace_bytes(4096, 4096, 4096, 1 << 20)
    assert need >= 4096 * 4096 * 4 + (1 << 20) * 16 and need % 256 == 0
    assert L.mam_csr_fwd_ws_f32(null, one, one, one, 0, null, one, null, null, 64, 64, 64, null, 0, null) == 1
    assert L.mam_csr_fwd_ws_f32(one, one, one, one, 0, null, one, one, null, 64, 64, 64, null, 0, null) == 1
    assert L.mam_im2col_f32(one, one, 1, 1, 4, 4, 5, 5, 1, 1, 0, 0, null) == 1                 # kernel larger than input
    assert L.mam_im2col_f32(one, null, 1, 1, 4, 4, 3, 3, 1, 1, 0, 0, null) == 1
    assert L.mam_col2im_f32(one, one, 1, 1, 4, 4, 3, 3, 0, 1, 0, 0, null) == 1                 # zero stride
    assert L.mam_bwd_count_ex_f32(one, one, 1, one, one, one, one, 7, one, null, null, 1.0, 4, 4, 4, null) == 1


def test_spmm_workspace_query_steers_small_and_very_sparse_products_to_the_row_kernel():
    L = _lib.lib()
    assert L.mam_spmm_csr_workspace_bytes(4096, 4096, 4096, 4096 * 410) > 0      # ~10 % dense, 6.9e9 multiply-adds
    assert L.mam_spmm_csr_workspace_bytes(4096, 4096, 4096, 4096 * 40) == 0       # ~1 % dense: too few per stage
    assert L.mam_spmm_csr_workspace_bytes(1024, 1024, 1024, 1024 * 102) == 0      # too little work
    assert L.mam_spmm_csr_workspace_bytes(4096, 4096, 62, 4096 * 410) == 0        # columns not a multiple of 4


def test_reference_cuda_arm_reports_unavailable_without_a_device(tmp_path):
    import json
    import os
    import subprocess
    import sys

    if torch.cuda.is_available():
        pytest.skip("covers the machine without a GPU")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference_cuda", "--steps", "1"],
                         capture_output=True, text=True, timeout=300, cwd=str(tmp_path))
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference_cuda" and "unavailable" in line


def test_reference_cuda_build_is_a_no_op_without_a_checkout(tmp_path):
    from oracle import build_ref_cuda

    assert build_ref_cuda.build(str(tmp_path)) == []


def test_implicit_convolution_applicability_needs_no_device():
    L = _lib.lib()
    assert L.mam_conv_fwd_applies(128, 64, 56, 56, 3, 3, 1, 1, 1, 1) == 1       # the benchmark's convolution
    assert L.mam_conv_fwd_applies(128, 3, 224, 224, 7, 7, 2, 2, 3, 3) == 0      # 3 input channels
    assert L.mam_conv_fwd_applies(1, 32, 8, 8, 3, 3, 1, 1, 1, 1) == 0           # input below 128 KiB
    assert L.mam_conv_fwd_applies(8, 64, 56, 56, 3, 3, 1, 1, 200, 1) == 0       # padding outside the corner field
    assert L.mam_conv_fwd_applies(8, 64, 56, 56, 60, 3, 1, 1, 1, 1) == 0        # kernel larger than the padded input
    null, one = None, ctypes.c_void_p(16)
    assert L.mam_conv_fwd_f32(null, one, null, null, 0, 1.0, 0.0, one, null, null, 8, 64, 56, 56, 3, 3, 1, 1, 1, 1, 8, null) == 1
    assert L.mam_conv_fwd_f32(one, one, null, null, 0, 1.0, 0.0, one, one, null, 8, 64, 56, 56, 3, 3, 1, 1, 1, 1, 8, null) == 1


def test_one_kernel_conv_backward_applicability_and_argument_checks_need_no_device():
    L = _lib.lib()
    ok = L.mam_conv_bwd_direct_applies
    assert ok(128, 64, 56, 56, 3, 3, 1, 1, 1, 1) == 1          # the benchmark convolution
    assert ok(1, 1, 1, 1, 1, 1, 1, 1, 0, 0) == 1
    assert ok(8, 512, 14, 14, 3, 3, 1, 1, 1, 1) == 1           # 512 channels x 3 rows x 14 columns = 86 KB
    assert ok(1, 4096, 64, 64, 3, 3, 1, 1, 1, 1) == 0          # one output row's tile of dx exceeds a CTA's shared memory
    assert ok(1, 3, 2, 2, 5, 5, 1, 1, 0, 0) == 0               # kernel larger than the padded input: no geometry
    assert ok(0, 3, 8, 8, 3, 3, 1, 1, 1, 1) == 0
    # null pointers are refused before any device work
    st = L.mam_conv_bwd_direct_f32(None, None, None, None, None, None, None, 1.0, 1, 3, 8, 8, 3, 3, 1, 1, 1, 1, 4, None)
    assert st == 1   # MAM_ERR_INVALID_ARGUMENT
    from mamtorch_b200.nn.conv import set_conv_backward_form
    with pytest.raises(ValueError):
        set_conv_backward_form("scatter")
    set_conv_backward_form("auto")


def test_tap_order_permutation_and_legacy_index():
    from mamtorch_b200.nn.conv import tap_order_permutation, to_legacy_index

    C, kH, kW = 5, 3, 2
    perm = tap_order_permutation(C, kH, kW)
    assert sorted(perm.tolist()) == list(range(C * kH * kW))
    for pos, k in enumerate(perm.tolist()):
        c, kh, kw = k // (kH * kW), (k // kW) % kH, k % kW
        assert pos == (kw * kH + kh) * C + c
    # position in tap order == the legacy index of the reference's text
    assert torch.equal(to_legacy_index(perm, C, kH, kW), torch.arange(C * kH * kW))


def test_entry_points_of_the_fused_training_paths_check_arguments_without_a_device():
    L = _lib.lib()
    null = None
    one = ctypes.c_void_p(16)   # never dereferenced: every call below fails its argument check first
    # hits riding on the dW reductions: where the size query advises it, and where it cannot be exact
    assert L.mam_bwd_count_workspace_bytes(12608, 3072, 768) == 3072 * 768 * 16       # CTA-shared kernel, records in L2
    assert L.mam_bwd_count_workspace_bytes(12608, 768, 3072) == 0                     # row-per-warp band: second sweep
    assert L.mam_bwd_count_workspace_bytes(4096, 4096, 4096) == 0                     # records beyond L2
    assert L.mam_bwd_count_workspace_bytes(1 << 24, 512, 512) == 0                    # fp32 counts no longer exact
    assert L.mam_bwd_count_workspace_bytes(0, 512, 512) == 0
    assert L.mam_bwd_splits_f32(one, one, 1, one, one, one, 0, one, 0, one, null, null, 1.0, 8, 64, 8, null, 0, null) == 1
    assert L.mam_bwd_splits_f32(one, one, 1, one, one, one, 2, one, 7, one, null, null, 1.0, 8, 64, 8, null, 0, null) == 1
    # dropout: rate outside [0, 1) is refused
    assert L.mam_drop_f32(one, one, 16, 1.0, 1.0, 5, null) == 1
    assert L.mam_drop_f32(one, one, 16, -0.1, 1.0, 5, null) == 1
    assert L.mam_drop_f32(null, one, 16, 0.5, 1.0, 5, null) == 1
    assert L.mam_drop_f32(one, one, 0, 0.5, 1.0, 5, null) == 1
    # splits with indices: slice width must be a positive multiple of 32 below K
    args = (one, one, null, null, 0, 1.0, 0.0, one, one, one, 64, 256, 64)
    assert L.mam_fwd_splits_idx_f32(*args, 0, null) == 1
    assert L.mam_fwd_splits_idx_f32(*args, 48, null) == 2
    assert L.mam_fwd_splits_idx_f32(*args, 256, null) == 2
    assert L.mam_fwd_splits_idx_f32(one, one, null, null, 0, 1.0, 0.0, one, null, one, 64, 256, 64, 64, null) == 1
    # tuning knobs live in their own header and reject unknown knobs and values
    assert L.mam_tune_set(3, 9) == 1 and L.mam_tune_set(7, 0) == 1 and L.mam_tune_set(3, 0) == 0
    assert L.mam_fwd_variant_name(1, 0).decode().startswith("idx_") and L.mam_fwd_variant_name(1, -1) == b"auto"


def test_overlapped_grad_sync_is_inert_without_gradients():
    from mamtorch_b200.dist import OverlappedGradSync

    p = torch.nn.Parameter(torch.zeros(3))
    frozen = torch.nn.Parameter(torch.zeros(3), requires_grad=False)
    sync = OverlappedGradSync([p, frozen], deferred=True)
    assert len(sync._handles) == 1            # only parameters that can receive a gradient get a hook
    sync.enabled = False
    (p * 2).sum().backward()                  # hook fires, disabled: nothing noted, no process group needed
    sync.finish()
    assert torch.equal(p.grad, torch.full((3,), 2.0))
    sync.remove()
