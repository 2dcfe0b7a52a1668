"""ctypes binding of librtxb (the C ABI declared in include/rtxb.h).

The library is built in-tree by `rtx_b200.build` (nvcc, sm_100a).  There is no
fallback: if the shared object is missing or a call fails, an exception is
raised.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("RTXB_LIBRARY") or os.path.join(_HERE, "_lib", "librtxb.so")

OK = 0
SCALE_ROW_MAJOR, SCALE_MMA64, SCALE_MMA128 = 0, 1, 2
ROUND_FLOOR, ROUND_INFINITY = 0, 1
OUT_BF16, OUT_F32 = 0, 1
TENSOR_SCALE_EXACT, TENSOR_SCALE_POWER2 = 0, 1
E_SCRATCH_CAPACITY = -7
NOALLOC_SCRATCH_BYTES = 32 * 1024 * 1024

DEVICE_STATUS_NAMES = {
    0: "ok",
    1: "TMA producer wait ran out",
    2: "MMA issuer wait ran out",
    3: "epilogue wait ran out",
    4: "quantizer wait ran out",
    5: "self-test wait ran out (expected: nothing completes its barrier)",
    6: "node barrier: another rank's flag never arrived",
}

_P, _I, _L, _Z = c_void_p, c_int, c_int64, c_size_t

# name -> (restype, argtypes); must list every symbol include/rtxb.h declares
SIGNATURES = {
    "rtxb_version": (_I, []),
    "rtxb_error_string": (c_char_p, [_I]),
    "rtxb_last_cuda_error": (c_char_p, []),
    "rtxb_set_gemm_schedule": (_I, [_I]),
    "rtxb_get_gemm_schedule": (_I, []),
    "rtxb_set_sm_margin": (_I, [_I]),
    "rtxb_get_sm_margin": (_I, []),
    "rtxb_mxfp8_storage_k": (_L, [_L]),
    "rtxb_nvfp4_storage_k": (_L, [_L]),
    "rtxb_mxfp8_scale_bytes": (_Z, [_L, _L, _I]),
    "rtxb_nvfp4_scale_bytes": (_Z, [_L, _L, _I]),
    "rtxb_mxfp8_quantize": (_I, [_P, _L, _L, _L, _P, _P, _I, _I, _P]),
    "rtxb_mxfp8_quantize_transposed": (_I, [_P, _L, _L, _L, _P, _P, _I, _I, _P]),
    "rtxb_mxfp8_quantize_dual": (_I, [_P, _L, _L, _L, _P, _P, _P, _P, _I, _I, _P]),
    "rtxb_mxfp8_gemm": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P, _P]),
    "rtxb_mxfp8_gemm_row_blocks": (_I, [_P, _P, _P, _P, _P, _I, _L, _L, _L, _L, _L, _I, _I, _P, _P]),
    "rtxb_mxfp8_gemm_glu": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "rtxb_mxfp8_gemm_glu_mx": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "rtxb_mxfp8_linear_fwd_fused_x": (_I, [_P, _L, _P, _P, _P, _L, _L, _L, _L, _I, _P, _P]),
    "rtxb_mxfp8_gemm_glu_mx_fused_x": (_I, [_P, _L, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "rtxb_mxfp8_linear_workspace_bytes": (_Z, [_L, _L, _L]),
    "rtxb_mxfp8_linear_fwd": (_I, [_P, _P, _P, _L, _L, _L, _I, _P, _Z, _P, _P]),
    "rtxb_mxfp8_linear_fwd_noalloc": (_I, [_P, _P, _P, _L, _L, _L, _I, _P, _P]),
    "rtxb_mxfp8_glu_mlp_workspace_bytes": (_Z, [_L, _L, _L, _L]),
    "rtxb_mxfp8_glu_mlp_fwd": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _Z, _P, _P]),
    "rtxb_mxfp8_backward_workspace_bytes": (_Z, [_L, _L, _L]),
    "rtxb_mxfp8_linear_bwd": (_I, [_P, _P, _P, _P, _P, _I, _L, _L, _L, _P, _Z, _P, _P]),
    "rtxb_sum_parts_f32_to_bf16": (_I, [_P, _I, _L, _L, _P, _P]),
    "rtxb_selftest_wait_timeout": (_I, [_L, _P, _P, _P]),
    "rtxb_peer_barrier": (_I, [_P, _I, _I, _P, _L, _P, _P]),
    "rtxb_nvfp4_tensor_scale": (_I, [_P, _L, _L, _L, _I, _P, _P, _P, _P, _P]),
    "rtxb_nvfp4_quantize": (_I, [_P, _L, _L, _L, _P, _P, _I, _P, _P]),
    "rtxb_nvfp4_gemm": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P, _P, _P]),
    "rtxb_nvfp4_linear_workspace_bytes": (_Z, [_L, _L, _L]),
    "rtxb_nvfp4_linear_fwd": (_I, [_P, _P, _P, _L, _L, _L, _I, _P, _Z, _P, _P]),
    "rtxb_nvfp4_quantize_delayed": (_I, [_P, _L, _L, _L, _P, _P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _P]),
    "rtxb_nvfp4_linear_fwd_delayed": (_I, [_P, _P, _P, _L, _L, _L, _P, _P, _P, _P, _I, _I, _I, _P, _Z, _P, _P]),
    "rtxb_nvfp4_region_scales": (_I, [_P, _L, _L, _L, _L, _I, _P, _P, _P]),
    "rtxb_nvfp4_quantize_regions": (_I, [_P, _L, _L, _L, _P, _P, _I, _P, _L, _P]),
    "rtxb_nvfp4_gemm_regions": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _L, _P, _L, _P, _P]),
    "rtxb_nvfp4_linear_regions_workspace_bytes": (_Z, [_L, _L, _L, _L, _L]),
    "rtxb_nvfp4_linear_fwd_regions": (_I, [_P, _P, _P, _L, _L, _L, _L, _L, _I, _P, _Z, _P, _P]),
    "rtxb_nvfp4_quantize_dynamic": (_I, [_P, _L, _L, _L, _I, _P, _P, _I, _P, _P, _P, _P, _P]),
    "rtxb_nvfp4_linear_prequant_w_workspace_bytes": (_Z, [_L, _L]),
    "rtxb_nvfp4_linear_fwd_prequant_w": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _I, _P, _Z, _P, _P]),
}


class NativeError(RuntimeError):
    """A librtxb call returned a non-zero code."""


_lib = None


def load() -> ctypes.CDLL:
    """Load librtxb once and attach argument types to every export."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: run `python -m rtx_b200.build` (needs nvcc). "
                "rtx_b200 has no CPU or PyTorch fallback."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(code: int, what: str) -> None:
    if code != OK:
        lib = load()
        msg = lib.rtxb_error_string(code).decode()
        detail = lib.rtxb_last_cuda_error().decode()
        raise NativeError(f"{what} failed: {msg} ({code}){': ' + detail if detail else ''}")


def call(name: str, *args) -> None:
    """Call an int-returning entry point and raise on a non-zero code."""
    check(getattr(load(), name)(*args), name)


def query(name: str, *args):
    """Call a size/version query."""
    return getattr(load(), name)(*args)
