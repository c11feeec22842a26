"""Loads the native pieces of the package and exposes the C ABI through ctypes.

There is no CPU path and no fallback: if libmam_b200.so or the operator shim _C.so is missing the
import fails with instructions, and every operator raises if it is handed CPU tensors.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmam_b200.so")
SHIM_PATH = os.path.join(_HERE, "_C.so")

# name -> (restype, argtypes) for every symbol include/mam_b200.h and include/mam_b200_tuning.h declare
_vp, _i64, _i32, _f32, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
ABI = {
    "mam_status_str": (ctypes.c_char_p, [_i32]),
    "mam_abi_version": (_i32, []),
    "mam_last_cuda_error": (ctypes.c_char_p, []),
    "mam_check_device_flag": (_i32, []),
    "mam_poll_device_flag": (_i32, [_vp]),
    "mam_tune_set": (_i32, [_i32, _i32]),
    "mam_fwd_variant_name": (ctypes.c_char_p, [_i32, _i32]),
    "mam_timer_arm": (_i32, [ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i32, _i32]),
    "mam_timer_disarm": (_i32, []),
    "mam_fwd_workspace_bytes": (_sz, [_i64, _i64, _i64, _i32, _i32]),
    "mam_fwd_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _i32, _f32, _f32, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp]),
    "mam_fwd_drop_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _i32, _f32, _f32, _f32, ctypes.c_uint64, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp]),
    "mam_drop_f32": (_i32, [_vp, _vp, _i64, _f32, _f32, ctypes.c_uint64, _vp]),
    "mam_fwd_kn_static_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mam_bwd_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _vp]),
    "mam_bwd_count_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _vp]),
    "mam_bwd_count_ex_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _vp]),
    "mam_fwd_splits_idx_f32": (_i32, [_vp, _vp, _vp, _vp, _i32, _f32, _f32, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "mam_bwd_splits_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _i32, _vp, _i32, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _vp, _sz, _vp]),
    "mam_bwd_count_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "mam_bwd_count_ws_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _vp, _sz, _vp]),
    "mam_conv_bwd_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i64, _vp]),
    "mam_conv_bwd_direct_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i64, _vp]),
    "mam_conv_bwd_direct_applies": (_i32, [_i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32]),
    "mam_fwd_splits_f32": (_i32, [_vp, _vp, _vp, _vp, _i32, _f32, _f32, _vp, _i64, _i64, _i64, _i64, _vp]),
    "mam_nchw_to_nhwc_f32": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "mam_conv_fwd_applies": (_i32, [_i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32]),
    "mam_conv_fwd_f32": (_i32, [_vp, _vp, _vp, _vp, _i32, _f32, _f32, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i64, _vp]),
    "mam_im2col_f32": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "mam_col2im_f32": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "mam_selcount_i32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mam_selcount_indicator_i32": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "mam_dense_tf32": (_i32, [_vp, _vp, _vp, _f32, _f32, _i64, _i64, _i64, _vp]),
    "mam_csr_fwd_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mam_csr_fwd_workspace_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64]),
    "mam_csr_fwd_ws_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, ctypes.c_size_t, _vp]),
    "mam_csr_fwd_ws_ex_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, ctypes.c_size_t, _i32, _vp]),
    "mam_csr_fwd_entries_bytes": (ctypes.c_size_t, [_i64, _i64, _i64]),
    "mam_spmm_csr_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mam_spmm_csr_workspace_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64]),
    "mam_spmm_csr_ws_f32": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _vp, ctypes.c_size_t, _vp]),
    "mam_transpose_f32": (_i32, [_vp, _vp, _i64, _i64, _vp]),
}

MAM_B_KN, MAM_B_NK = 0, 1

_lib = None
_shim_loaded = False


def _missing(path: str) -> ImportError:
    return ImportError(
        f"mamtorch_b200: native library {path} is missing. Build it in-tree with "
        f"`python mamtorch_b200/_build.py` (needs nvcc and g++); there is no CPU fallback.")


def lib() -> ctypes.CDLL:
    """The C-ABI library, with argument/return types set for every declared symbol."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise _missing(LIB_PATH)
        h = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in ABI.items():
            fn = getattr(h, name)  # AttributeError here = header and library out of sync
            fn.restype = res
            fn.argtypes = args
        _lib = h
    return _lib


def load_ops() -> None:
    """Registers torch.ops.mamtorch_kernel_v{1,2,3,4}.* and torch.ops.mamtorch_b200.*."""
    global _shim_loaded
    if not _shim_loaded:
        lib()
        if not os.path.exists(SHIM_PATH):
            raise _missing(SHIM_PATH)
        torch.ops.load_library(SHIM_PATH)
        _shim_loaded = True


def status_str(code: int) -> str:
    return lib().mam_status_str(code).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        extra = ""
        if code == 4:
            extra = ": " + lib().mam_last_cuda_error().decode()
        raise RuntimeError(f"{what}: {status_str(code)}{extra}")
