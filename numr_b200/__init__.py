"""numr_b200: the B200 (sm_100a) dense-GEMM path of numr behind its own op surface.

The product is libnumr_b200.so (hand-written tcgen05/TMEM/TMA kernels behind the C ABI
in include/numr_b200.h); this package binds it and mirrors numr's client methods.
"""
from ._lib import LIB_PATH, load
from .client import (CudaClient, DTypeMismatch, GemmActivation, Internal, InvalidArgument, NumrError,
                     ShapeMismatch, UnsupportedDType, dtype_code)

__all__ = [
    "CudaClient", "GemmActivation", "NumrError", "InvalidArgument", "UnsupportedDType", "Internal",
    "ShapeMismatch", "DTypeMismatch", "dtype_code", "load", "LIB_PATH",
]
