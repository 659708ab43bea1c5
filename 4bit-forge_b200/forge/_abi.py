"""ctypes binding of libforge_b200.so (the C ABI declared in include/forge_b200.h).

The library is the product path: there is no CPU or eager fallback.  If it is missing, or a call
fails, a RuntimeError is raised — the same behaviour as the reference's stub module when CUDA is
absent (forge/backend/cuda/__init__.py:74-87).
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_ROOT, "libforge_b200.so")

F32, BF16 = 0, 1
HESS_MIRROR, HESS_SIMT = 1, 2
FWD_SIMT = 1
ROUTE_MODES = {"softmax": 0, "sigmoid": 1, "sigmoid_group": 2}
ERR_INVALID, ERR_TIMEOUT = 1, 3

_c_i64 = ctypes.c_int64
_c_int = ctypes.c_int
_c_f32 = ctypes.c_float
_ptr = ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/forge_b200.h one to one
_PROTOS = {
    "forge_version": (_c_int, []),
    "forge_last_error": (ctypes.c_char_p, []),
    "forge_launch_count": (ctypes.c_longlong, []),
    "forge_fp8_block_dequant": (_c_int, [_ptr, _ptr, _ptr, _c_i64, _c_i64, _c_i64, _c_i64, _ptr]),
    "forge_route_topk": (_c_int, [_ptr, _ptr, _c_i64, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr]),
    "forge_route_build_lists": (_c_int, [_ptr, _c_i64, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr]),
    "forge_expert_swiglu_grouped": (_c_int, [_ptr, _c_i64, _c_i64, _c_i64, _c_i64, _ptr, _c_i64, _ptr, _c_int, _ptr, _ptr,
                                             _ptr, _c_i64, _c_int, _ptr, _ptr]),
    "forge_recon_loss": (_c_int, [_ptr, _c_int, _ptr, _ptr, _ptr, _c_int, _c_int, _c_i64, _c_i64, _ptr, _c_i64, _c_i64,
                                  _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "forge_hessian_grouped": (_c_int, [_ptr, _c_i64, _c_i64, _c_i64, _ptr, _c_i64, _ptr, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr]),
    "forge_selftest_bounded_wait": (_c_int, [_ptr, _c_i64, _ptr]),
    "forge_selftest_mma_rate": (_c_int, [_c_int, _c_int, _c_int, _ptr, _ptr, _ptr]),
    "forge_int4_packed_dequant": (_c_int, [_ptr, _ptr, _c_i64, _c_i64, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr]),
    "forge_mxfp4_dequant": (_c_int, [_ptr, _ptr, _c_i64, _c_i64, _ptr, _c_int, _ptr]),
    "forge_counts_add": (_c_int, [_ptr, _ptr, _c_int, _ptr]),
    "forge_hessian_scan": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "forge_weight_apply_pruned": (_c_int, [_ptr, _c_int, _c_int, _c_i64, _c_i64, _ptr, _ptr, _ptr]),
    "forge_weight_zero_cols": (_c_int, [_ptr, _c_int, _c_int, _c_i64, _c_i64, _ptr, _ptr]),
    "forge_hessian_gather_damp": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _c_f32, _ptr, _ptr, _ptr, _ptr]),
    "forge_chol_workspace_bytes": (_c_i64, [_c_int, _c_i64]),
    "forge_chol_factor_batched": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr]),
    "forge_chol_inv_upper_batched": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr]),
    "forge_noalloc_max_c": (_c_i64, []),
    "forge_chol_inv_upper_noalloc": (_c_int, [_ptr, _c_i64, _ptr, _ptr, _ptr, _c_int, _ptr]),
    "forge_quant_grid": (_c_int, [_ptr, _c_int, _c_i64, _c_i64, _c_int, _c_int, _c_int, _ptr, _c_int, _c_f32, _ptr, _ptr, _ptr]),
    "forge_quant_grid_mse": (_c_int, [_ptr, _c_int, _c_i64, _c_i64, _c_int, _c_int, _c_int, _ptr, _c_int, _c_f32, _ptr, _ptr, _ptr]),
    "forge_solve_workspace_bytes": (_c_i64, [_c_int, _c_i64, _c_i64]),
    "forge_gptq_solve_cr": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_i64, _c_i64, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "forge_solve_split_u_bytes": (_c_i64, [_c_int, _c_i64]),
    "forge_solve_split_u": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr]),
    "forge_gptq_solve_batched": (_c_int, [_ptr, _c_int, _c_int, _c_i64, _c_i64, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr,
                                          _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "forge_dequantize": (_c_int, [_ptr, _ptr, _ptr, _c_i64, _c_i64, _c_int, _ptr, _c_int, _ptr]),
    "forge_pack_int4": (_c_int, [_ptr, _ptr, _c_i64, _c_i64, _c_int, _ptr, _ptr]),
    "forge_pack_sparse14": (_c_int, [_ptr, _ptr, _ptr, _c_i64, _c_i64, _ptr, _ptr]),
    "forge_pack_sparse14_batched": (_c_int, [_ptr, _ptr, _ptr, _c_int, _c_i64, _c_i64, _ptr, _ptr]),
    "forge_sparse14_gemm": (_c_int, [_ptr, _ptr, _c_i64, _c_i64, _c_i64, _c_i64, _ptr, _ptr]),
    "forge_sparse14_moe_w13_swiglu": (_c_int, [_ptr, _ptr, _c_i64, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _c_i64, _c_i64, _ptr, _ptr]),
    "forge_sparse14_moe_w2": (_c_int, [_ptr, _ptr, _c_i64, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _c_i64, _c_i64, _ptr, _ptr]),
}

_lib = None


def exported_symbols():
    return sorted(_PROTOS)


def load_library():
    """dlopen the in-tree library and attach prototypes (no CUDA call is made)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"forge_b200: {LIB_PATH} is missing; build it with `python 4bit-forge_b200/build.py` "
                "(there is no CPU fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _require_cuda():
    if not torch.cuda.is_available():
        raise RuntimeError("forge_b200 CUDA kernels are unavailable because torch.cuda.is_available() is False")


def ptr(t):
    if t is None:
        return None
    _require_cuda()
    if not (t.is_cuda and t.is_contiguous()):
        raise RuntimeError("forge_b200 expects contiguous CUDA tensors (there is no CPU path)")
    return t.data_ptr()


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise RuntimeError(f"forge_b200: unsupported weight dtype {t.dtype} (float32 / bfloat16)")


def call(name: str, *args):
    """Invoke an entry point; a non-zero return raises RuntimeError with the library's message."""
    _require_cuda()
    lib = load_library()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.forge_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{name} failed (code {rc}): {msg}")
    return rc


def query(name: str, *args) -> int:
    return int(getattr(load_library(), name)(*args))
