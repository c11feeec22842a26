"""CPU-side checks of the boundary: the C-ABI library loads, exports every symbol the header
declares, rejects bad arguments without touching a device, and the Python surface mirrors the
reference's names."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
from mamtorch_b200 import _lib


def header_functions():
    names = set()
    for header in ("mam_b200.h", "mam_b200_tuning.h"):
        src = open(os.path.join(ROOT, "include", header)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names |= set(re.findall(r"\b(mam_[a-z0-9_]+)\s*\(", src))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = header_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/*.h but not exported"
    assert sorted(_lib.ABI) == names, "ctypes table and header disagree"


def test_status_strings_and_version():
    L = _lib.lib()
    assert L.mam_abi_version() == 1
    assert _lib.status_str(0) == "ok"
    seen = {_lib.status_str(i) for i in range(8)}
    assert len(seen) == 8 and "unknown status" not in seen
    assert _lib.status_str(99) == "unknown status"


def test_bad_arguments_are_rejected_before_any_device_work():
    L = _lib.lib()
    null = None
    one = ctypes.c_void_p(16)  # never dereferenced: extents are invalid
    assert L.mam_fwd_f32(null, one, 0, null, null, 0, 1.0, 0.0, one, null, null, 4, 4, 4, null, 0, null) == 1
    assert L.mam_fwd_f32(one, one, 0, null, null, 0, 1.0, 0.0, one, null, null, 4, 0, 4, null, 0, null) == 1
    assert L.mam_fwd_f32(one, one, 7, null, null, 0, 1.0, 0.0, one, null, null, 4, 4, 4, null, 0, null) == 1
    assert L.mam_fwd_f32(one, one, 0, null, null, 0, 1.0, 0.0, one, one, null, 4, 4, 4, null, 0, null) == 1
    assert L.mam_bwd_f32(one, one, 0, one, one, one, one, null, 1.0, 4, 4, 4, null) == 1
    assert L.mam_selcount_i32(one, one, one, one, 0, 4, 4, null) == 1
    assert L.mam_transpose_f32(one, null, 4, 4, null) == 1
    assert L.mam_tune_set(0, 99) == 1
    assert L.mam_tune_set(99, 0) == 1
    assert L.mam_tune_set(0, -1) == 0


def test_workspace_query():
    L = _lib.lib()
    assert L.mam_fwd_workspace_bytes(128, 64, 32, _lib.MAM_B_NK, 1) == 0
    assert L.mam_fwd_workspace_bytes(128, 64, 32, _lib.MAM_B_KN, 1) == 64 * 32 * 4
    assert L.mam_fwd_workspace_bytes(128, 65, 32, _lib.MAM_B_KN, 1) == 0  # generic path needs none
    assert L.mam_fwd_variant_name(1, 0).decode().startswith("idx_")


def test_python_surface_mirrors_the_reference():
    import mamtorch_b200 as mamtorch

    assert callable(mamtorch.kernel.v1.fullyconnected)
    assert callable(mamtorch.kernel.v4.fullyconnected) and callable(mamtorch.kernel.v4.fullyconnected_fast)
    assert callable(mamtorch.kernel.v2.dense) and callable(mamtorch.kernel.v3.fullyconnected_fast)
    assert mamtorch.nn.FullyConnected is mamtorch.nn.v4.FullyConnected
    for ns, ops in {"mamtorch_kernel_v1": ["fullyconnected", "fullyconnected_backward"],
                    "mamtorch_kernel_v2": ["fullyconnected", "fullyconnected_backward", "dense"],
                    "mamtorch_kernel_v3": ["fullyconnected", "fullyconnected_fast", "fullyconnected_backward"],
                    "mamtorch_kernel_v4": ["fullyconnected", "fullyconnected_fast", "fullyconnected_backward"]}.items():
        for op in ops:
            assert hasattr(getattr(torch.ops, ns), op)
    schema = str(torch.ops.mamtorch_kernel_v4.fullyconnected.default._schema)
    assert schema == "mamtorch_kernel_v4::fullyconnected(Tensor a, Tensor b) -> Tensor[]"
    schema = str(torch.ops.mamtorch_kernel_v3.fullyconnected_backward.default._schema)
    assert "Tensor argmin, float beta) -> Tensor[]" in schema


def test_cpu_tensors_fail_loudly():
    import mamtorch_b200 as mamtorch

    with pytest.raises(NotImplementedError):
        mamtorch.kernel.v4.fullyconnected(torch.randn(3, 4), torch.randn(4, 5))
    with pytest.raises(NotImplementedError):
        mamtorch.nn.FullyConnected(4, 5)(torch.randn(2, 4))


def test_fake_kernels_give_shapes_and_dtypes():
    import mamtorch_b200  # noqa: F401

    a = torch.empty(6, 8, device="meta")
    b = torch.empty(8, 5, device="meta")
    c, imax, imin = torch.ops.mamtorch_kernel_v4.fullyconnected(a, b)
    assert c.shape == (6, 5) and imax.dtype == torch.int32 and imin.shape == (6, 5)
    assert torch.ops.mamtorch_kernel_v4.fullyconnected_fast(a, b).shape == (6, 5)
    bias = torch.empty(5, device="meta")
    assert torch.ops.mamtorch_kernel_v3.fullyconnected(a, b, bias, 0.3)[0].shape == (6, 5)
    with pytest.raises(Exception):
        torch.ops.mamtorch_kernel_v4.fullyconnected(a, torch.empty(7, 5, device="meta"))


def test_vcon_schedule_and_module_attributes():
    import mamtorch_b200 as mamtorch

    m = mamtorch.nn.FullyConnected(16, 8, vcon_steps=4, store_args=True)
    assert (m.beta, m.alpha) == (1.0, 0.0) and m.weight.shape == (8, 16) and m.bias.shape == (8,)
    betas = []
    for _ in range(5):
        m.vcon_step()
        betas.append(m.beta)
    assert betas[:3] == [0.75, 0.5, 0.25] and betas[3] == 0 and betas[4] <= 0
    e = mamtorch.nn.FullyConnected(16, 8, vcon_steps=3, vcon_type="exponential", vcon_eps=1e-3, vcon_expand=True)
    e.vcon_step()
    assert abs(e.beta - 0.1) < 1e-9 and abs(e.alpha - 0.9 * 16 / 2) < 1e-9
    with pytest.raises(Exception):
        mamtorch.nn.FullyConnected(4, 4).reset_selection_count()
    # keyword the reference's ViT example still passes although its own v4 module rejects it
    mamtorch.nn.FullyConnected(4, 4, beta_zero_gain=1.0)
    sd = mamtorch.nn.FullyConnected(4, 3).state_dict()
    assert sorted(sd) == ["bias", "weight"]
    d = mamtorch.MAMDense(4, 3, beta=True)
    d.adjust_beta(0)
    assert d.beta == 1
    c = mamtorch.nn.MAMConv2d(3, 5, 3, padding=1)
    assert c.weight.shape == (5, 3, 3, 3)
