"""ctypes binding of ``libb200moe.so`` (the C ABI declared in ``include/b200moe.h``).

There is no CPU fallback: if the shared library is missing or fails to load,
every kernel entry raises.  Errors reported by the library are raised as
``AssertionError`` with the reference's ``kernel_assert`` prefix
(core/utils/kernel_assert.py:15-16) so negative tests written against the
reference keep their meaning.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# B200MOE_LIBRARY lets a caller point at another build of the same C ABI (A/B timing of kernel variants)
LIB_PATH = os.environ.get("B200MOE_LIBRARY") or os.path.join(_PKG, "libb200moe.so")
ERROR_PREFIX = "[INTERNAL_ERROR] [NCC_INKI016] Kernel validation exception: "

F32, BF16, I32 = 0, 1, 2
LAYOUT_ROWS, LAYOUT_NKI_X4 = 0, 1
W_E4M3, W_E5M2, W_E2M1 = 0, 1, 5  # weight element formats (B200MOE_W_*)
ROUTING_INDEX, ROUTING_MASK = 0, 1
# per-call variant word of the grouped contractions (B200MOE_IMPL_* / B200MOE_GEMM_*)
IMPL_SIMT, GEMM_TILE_N128, GEMM_NO_PAIR, GEMM_FORCE_PAIR, GEMM_NO_SPLIT, GEMM_NO_OVERLAP = 1, 0x100, 0x200, 0x400, 0x800, 0x1000
ROUTER_AUTO, ROUTER_SPLIT_K, ROUTER_TCGEN05 = 0, 1, 2

# name -> (restype, argtypes); must list every symbol of include/b200moe.h
SIGNATURES = {
    "b200moe_last_error": (c_char_p, []),
    "b200moe_version": (c_int, []),
    "b200moe_sf_bytes": (c_size_t, [c_int64, c_int64]),
    "b200moe_router_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200moe_router_topk": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_size_t,
                                    c_void_p]),
    "b200moe_find_nonzero_workspace_bytes": (c_size_t, [c_int, c_int]),
    "b200moe_find_nonzero_indices": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                             c_void_p, c_size_t, c_void_p]),
    "b200moe_cumsum": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_indexed_flatten": (c_int, [c_void_p, c_int, c_int, c_int, c_int64, c_void_p, c_int, c_void_p, c_int,
                                        c_void_p, c_void_p]),
    "b200moe_group_tokens_workspace_bytes": (c_size_t, [c_int, c_int]),
    "b200moe_group_tokens": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                     c_void_p]),
    "b200moe_group_tokens_static_max_bytes": (c_size_t, []),
    "b200moe_group_tokens_static": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_build_position_table": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                             c_void_p]),
    "b200moe_gather_quantize_mxfp8": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                              c_void_p, c_void_p]),
    "b200moe_scatter_quantize_mxfp8": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int64, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p]),
    "b200moe_prepare_gate_up": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p]),
    "b200moe_prepare_down": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_weight_bytes": (c_int64, [c_int64, c_int64, c_int]),
    "b200moe_prepare_gate_up_bias": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200moe_grouped_gemm1_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                             c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                             c_void_p]),
    "b200moe_grouped_gemm2_scale": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                            c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "b200moe_scatter_rows_bf16": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int64, c_void_p, c_int, c_int,
                                          c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_dense_gemm1_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                           c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float,
                                           c_void_p, c_void_p, c_int, c_void_p]),
    "b200moe_dense_gemm2_scale": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                          c_void_p, c_int, c_void_p]),
    "b200moe_combine": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200moe_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                c_void_p]),
    "b200moe_rmsnorm_quantize_mxfp8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                               c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                               c_void_p]),
    "b200moe_ipc_export": (c_int, [c_void_p, c_void_p, c_void_p]),
    "b200moe_ipc_open": (c_int, [c_void_p, c_int64, c_void_p]),
    "b200moe_ipc_close": (c_int, [c_void_p, c_int64]),
    "b200moe_ep_exchange_counts": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                           c_void_p]),
    "b200moe_ep_signal_wait": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_ep_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p]),
    "b200moe_ep_scales_to_atoms": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "b200moe_ep_dispatch_quantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p]),
    "b200moe_ep_gemm2_scale_return": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                              c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p]),
    "b200moe_ep_return_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int64,
                                       c_void_p]),
}

_lib = None


def load_library() -> ctypes.CDLL:
    """Load the shared library and attach argument types (no device needed)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m nki_library_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return c_void_p(t.data_ptr())


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype in (torch.int32, torch.uint32):
        return I32
    raise AssertionError(ERROR_PREFIX + f"unsupported dtype {t.dtype}")


def kernel_assert(cond: bool, msg: str) -> None:
    if not cond:
        raise AssertionError(ERROR_PREFIX + msg)


def call(name: str, *args) -> None:
    """Invoke an ``int``-returning entry point and raise on a non-zero status."""
    lib = load_library()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.b200moe_last_error().decode("utf-8", "replace")
        raise AssertionError(ERROR_PREFIX + f"{name} failed ({rc}): {msg}")


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise AssertionError(ERROR_PREFIX + "all tensors must live on a CUDA device (no CPU path exists)")
