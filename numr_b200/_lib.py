"""ctypes binding of libnumr_b200.so (the C ABI declared in include/numr_b200.h).

The library is the product: if it is missing it is built with nvcc, and if that
fails the import raises. Nothing here falls back to PyTorch or CPU arithmetic.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libnumr_b200.so"

# numr_b200_status
OK, EINVAL, EUNSUPPORTED, ECUDA, EWORKSPACE, ETIMEOUT, ESHAPE, EDTYPE = range(8)

# numr_b200_dtype
F32, BF16, F16, FP8E4M3, FP8E5M2, I8, I32, I64, I16, U8, U16, U32, U64 = range(13)

# numr_b200_b_layout / numr_b200_f32_mode
B_KN, B_NK = 0, 1
F32_EXACT, F32_TF32 = 0, 1


class GemmDesc(ctypes.Structure):
    """numr_b200_gemm_desc"""
    _fields_ = [
        ("a_dtype", c_int32), ("b_dtype", c_int32), ("out_dtype", c_int32), ("bias_dtype", c_int32),
        ("batch", c_uint32), ("m", c_uint32), ("n", c_uint32), ("k", c_uint32),
        ("a_batch", c_uint32), ("b_batch", c_uint32),
        ("b_layout", c_int32), ("activation", c_int32), ("f32_mode", c_int32),
        ("scale_a", c_float), ("scale_b", c_float),
    ]


class ConvDesc(ctypes.Structure):
    """numr_b200_conv_desc"""
    _fields_ = [
        ("dtype", c_int32), ("batch", c_uint32), ("c_in", c_uint32), ("c_out", c_uint32), ("groups", c_uint32),
        ("in_h", c_uint32), ("in_w", c_uint32), ("kernel_h", c_uint32), ("kernel_w", c_uint32),
        ("stride_h", c_uint32), ("stride_w", c_uint32),
        ("pad_top", c_uint32), ("pad_bottom", c_uint32), ("pad_left", c_uint32), ("pad_right", c_uint32),
        ("dilation_h", c_uint32), ("dilation_w", c_uint32), ("output_padding", c_uint32), ("f32_mode", c_int32),
    ]


CONV1D, CONV2D, CONV_TRANSPOSE1D = 0, 1, 2


class TensorDesc(ctypes.Structure):
    """numr_b200_tensor"""
    _fields_ = [
        ("ptr", c_uint64), ("dtype", c_int32), ("ndim", c_int32),
        ("shape", c_int64 * 8), ("strides", c_int64 * 8),
    ]


# Every symbol include/numr_b200.h declares, with its signature.
_T = POINTER(TensorDesc)
_WS = [c_void_p, c_size_t]
_LAUNCH_HEAD = [c_void_p, c_int, c_int32]
SIGNATURES = {
    "numr_b200_version": (c_char_p, []),
    "numr_b200_last_error": (c_char_p, []),
    "numr_b200_gemm_workspace_bytes": (c_size_t, [POINTER(GemmDesc), c_void_p, c_void_p]),
    "numr_b200_gemm": (c_int, [POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_size_t, c_void_p, c_int]),
    "numr_b200_gemm_allgather": (c_int, [POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, POINTER(c_uint64),
                                         c_uint32, c_uint32, c_void_p, c_size_t, c_void_p, c_int]),
    "numr_b200_device_status": (c_int, [POINTER(c_int)]),
    "numr_b200_reload_tuning": (None, []),
    "numr_b200_init": (c_int, [c_int]),
    "numr_b200_static_scratch_bytes": (c_size_t, []),
    "numr_b200_gemm_static_scratch": (c_int, [POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int]),
    "numr_b200_launch_matmul_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 3 + [c_size_t] * 3 + _WS),
    "numr_b200_launch_matmul_batched_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 3 + [c_size_t] * 6 + _WS),
    "numr_b200_launch_matmul_bias_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 4 + [c_size_t] * 3 + _WS),
    "numr_b200_launch_matmul_bias_batched_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 4 + [c_size_t] * 6 + _WS),
    "numr_b200_launch_gemm_bias_act_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 4 + [c_size_t] * 3 + [c_int32] + _WS),
    "numr_b200_launch_gemm_bias_act_batched_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 4 + [c_size_t] * 4 + [c_int32] + _WS),
    "numr_b200_launch_gemm_bias_residual_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 5 + [c_size_t] * 3 + _WS),
    "numr_b200_launch_gemm_bias_residual_batched_kernel": (c_int, _LAUNCH_HEAD + [c_uint64] * 5 + [c_size_t] * 4 + _WS),
    "numr_b200_launch_fp8_matmul_e4m3": (c_int, _LAUNCH_HEAD + [c_uint64] * 3 + [c_float] * 2 + [c_size_t] * 4 + _WS),
    "numr_b200_launch_fp8_matmul_e5m2": (c_int, _LAUNCH_HEAD + [c_uint64] * 3 + [c_float] * 2 + [c_size_t] * 4 + _WS),
    "numr_b200_matmul_out_shape": (c_int, [_T, _T, _T, POINTER(c_int64), POINTER(c_int32), POINTER(c_int32)]),
    "numr_b200_op_workspace_bytes": (c_size_t, [_T, _T, c_int32, c_int32]),
    "numr_b200_op_workspace_bytes_for": (c_size_t, [_T, _T, _T, _T, c_int32, c_int32]),
    "numr_b200_matmul": (c_int, [_T, _T, _T, c_int32] + _WS + [c_void_p, c_int]),
    "numr_b200_matmul_bias": (c_int, [_T, _T, _T, _T, c_int32] + _WS + [c_void_p, c_int]),
    "numr_b200_matmul_bias_activation": (c_int, [_T, _T, _T, c_int32, _T, c_int32] + _WS + [c_void_p, c_int]),
    "numr_b200_matmul_activation": (c_int, [_T, _T, c_int32, _T, c_int32] + _WS + [c_void_p, c_int]),
    "numr_b200_matmul_bias_residual": (c_int, [_T, _T, _T, _T, _T, c_int32] + _WS + [c_void_p, c_int]),
    "numr_b200_fp8_matmul": (c_int, [_T, _T, c_float, c_float, c_int32, _T] + _WS + [c_void_p, c_int]),
    "numr_b200_fp8_matmul_fused": (c_int, [_T, _T, c_float, c_float, _T, c_int32, _T, _T] + _WS + [c_void_p, c_int]),
    "numr_b200_grouped_gemm_workspace_bytes": (c_size_t, [POINTER(GemmDesc), c_uint32, c_void_p, c_void_p]),
    "numr_b200_grouped_gemm": (c_int, [POINTER(GemmDesc), c_uint32, c_void_p, c_void_p, c_void_p, c_void_p] + _WS
                               + [c_void_p, c_int]),
    "numr_b200_grouped_matmul_workspace_bytes": (c_size_t, [_T, _T, c_int32]),
    "numr_b200_grouped_matmul": (c_int, [_T, _T, _T, c_int32, _T, c_int32] + _WS + [c_void_p, c_int]),
    "numr_b200_matmul_bias_activation_bwd_workspace_bytes": (c_size_t, [_T, _T, _T, _T, c_int32]),
    "numr_b200_matmul_bias_activation_bwd": (c_int, [_T, _T, _T, _T, c_int32, _T, _T, _T, c_int32] + _WS
                                             + [c_void_p, c_int]),
    "numr_b200_conv_out_shape": (c_int, [POINTER(ConvDesc), c_int32, POINTER(c_uint32), POINTER(c_uint32)]),
    "numr_b200_conv_workspace_bytes": (c_size_t, [POINTER(ConvDesc), c_int32, c_void_p]),
    "numr_b200_conv1d": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p] + _WS + [c_void_p, c_int]),
    "numr_b200_conv2d": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p] + _WS + [c_void_p, c_int]),
    "numr_b200_conv_transpose1d": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p] + _WS
                                   + [c_void_p, c_int]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads (building first if needed) the shared library and types every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    override = os.environ.get("NUMR_B200_LIBRARY")   # another build of the same interface (A/B timing)
    if override:
        lib = ctypes.CDLL(override)
    else:
        if not LIB_PATH.exists():
            from . import build as _build
            _build.build()
        lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().numr_b200_last_error().decode("utf-8", "replace")
