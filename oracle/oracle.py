"""TEST INFRASTRUCTURE: ctypes binding of the CPU oracle (oracle/numr_oracle.cpp).

Only tests, the smoke check and the CPU-baseline leg of the benchmark import this
module. It works on numpy arrays; 16-bit and 8-bit float types travel as raw
uint16 / uint8 bit patterns.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "libnumr_oracle.so"

F32, BF16, F16, E4M3, E5M2, I8, I32 = range(7)
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU, ACT_SIGMOID, ACT_TANH = range(6)

_NP = {F32: np.float32, BF16: np.uint16, F16: np.uint16, E4M3: np.uint8, E5M2: np.uint8,
       I8: np.int8, I32: np.int32}


def build(force: bool = False) -> Path:
    """Compiles the oracle with the Makefile beside it."""
    src = _DIR / "numr_oracle.cpp"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B"], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = ctypes.CDLL(str(_LIB_PATH))
        vp, ci, cf, cd = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_double
        L.orc_f32_to_e4m3.argtypes = [cf]; L.orc_f32_to_e4m3.restype = ctypes.c_uint8
        L.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]; L.orc_e4m3_to_f32.restype = cf
        L.orc_f32_to_e5m2.argtypes = [cf]; L.orc_f32_to_e5m2.restype = ctypes.c_uint8
        L.orc_e5m2_to_f32.argtypes = [ctypes.c_uint8]; L.orc_e5m2_to_f32.restype = cf
        L.orc_f32_to_bf16.argtypes = [cf]; L.orc_f32_to_bf16.restype = ctypes.c_uint16
        L.orc_bf16_to_f32.argtypes = [ctypes.c_uint16]; L.orc_bf16_to_f32.restype = cf
        L.orc_f32_to_f16.argtypes = [cf]; L.orc_f32_to_f16.restype = ctypes.c_uint16
        L.orc_f16_to_f32.argtypes = [ctypes.c_uint16]; L.orc_f16_to_f32.restype = cf
        L.orc_encode.argtypes = [vp, vp, ctypes.c_size_t, ci]; L.orc_encode.restype = None
        L.orc_decode.argtypes = [vp, vp, ctypes.c_size_t, ci]; L.orc_decode.restype = None
        L.orc_matmul_f32.argtypes = [vp, vp, vp, vp] + [ci] * 8; L.orc_matmul_f32.restype = None
        L.orc_matmul_i8_i32.argtypes = [vp, vp, vp, vp] + [ci] * 5; L.orc_matmul_i8_i32.restype = None
        L.orc_fp8_matmul.argtypes = [vp, vp, ci, ci, vp, vp, vp, ci, ci, ci, ci, ci, cf, cf, ci, ci]
        L.orc_fp8_matmul.restype = None
        L.orc_gemm.argtypes = [ci, ci, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci]; L.orc_gemm.restype = ci
        L.orc_truth_f64.argtypes = [ci, ci, ci, vp, vp, vp, vp, vp, ci, ci, ci, ci, cd, ci, vp, ci, ci]
        L.orc_truth_f64.restype = None
        L.orc_matmul_wide_int.argtypes = [ci, ci, vp, vp, vp, vp, ci, ci, ci, ci]; L.orc_matmul_wide_int.restype = ci
        L.orc_conv.argtypes = [ci, ci, ci, vp, vp, vp, vp] + [ci] * 16; L.orc_conv.restype = None
        L.orc_max_threads.argtypes = []; L.orc_max_threads.restype = ci
        _lib = L
    return _lib


def _p(x):
    return None if x is None else x.ctypes.data_as(ctypes.c_void_p)


def _c(x, dt):
    """Contiguous array of the storage type of `dt` (or None)."""
    if x is None:
        return None
    x = np.ascontiguousarray(x)
    assert x.dtype == _NP[dt], f"expected storage dtype {_NP[dt]} for dtype code {dt}, got {x.dtype}"
    return x


def encode(x: np.ndarray, dt: int) -> np.ndarray:
    """float32 values -> storage of `dt` with numr's rounding (RNE; FP8 saturation rules)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=_NP[dt])
    if dt == F32:
        out[...] = x
    elif dt in (I8, I32):
        out[...] = x.astype(_NP[dt])
    else:
        lib().orc_encode(_p(x), _p(out), x.size, dt)
    return out


def decode(x: np.ndarray, dt: int) -> np.ndarray:
    """storage of `dt` -> float32 (exact)."""
    x = _c(x, dt)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_decode(_p(x), _p(out), x.size, dt)
    return out


def max_threads() -> int:
    return int(lib().orc_max_threads())


def gemm(dt, a, b, bias=None, residual=None, act=ACT_NONE, b_transposed=False, mode=0, threads=0):
    """One matrix op of numr's CPU backend on storage arrays.

    a: [M,K]; b: [K,N], or [N,K] when b_transposed; bias: [N] in the output type (int32 for I8);
    residual: [M,N] in the output type. mode 0 = f32 accumulation, 1 = literal in-dtype loops.
    """
    a = _c(a, dt); b = _c(b, dt)
    m, k = a.shape
    n = b.shape[0] if b_transposed else b.shape[1]
    assert (b.shape[1] if b_transposed else b.shape[0]) == k
    out_dt = I32 if dt == I8 else dt
    bias = _c(bias, out_dt); residual = _c(residual, out_dt)
    out = np.empty((m, n), dtype=_NP[out_dt])
    rc = lib().orc_gemm(dt, mode, _p(a), _p(b), _p(bias), _p(residual), _p(out), m, n, k,
                        int(b_transposed), act, threads)
    if rc != 0:
        raise ValueError(f"oracle: unsupported combination (code {rc})")
    return out


def matmul_wide_int(a, b, bias=None, b_transposed=False):
    """numr's matmul / matmul_bias for I16, I32, I64, U8, U16, U32, U64 numpy arrays: exact 128-bit
    accumulation seeded by the bias (same dtype), one saturating store, output of the operands' dtype."""
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    assert a.dtype == b.dtype and a.dtype.kind in "iu"
    m, k = a.shape
    n = b.shape[0] if b_transposed else b.shape[1]
    if bias is not None:
        bias = np.ascontiguousarray(bias)
        assert bias.dtype == a.dtype
    out = np.empty((m, n), dtype=a.dtype)
    rc = lib().orc_matmul_wide_int(a.dtype.itemsize, int(a.dtype.kind == "i"), _p(a), _p(b), _p(bias), _p(out),
                                   m, n, k, int(b_transposed))
    if rc != 0:
        raise ValueError("oracle: unsupported integer width")
    return out


def _act_derivative(x, act):
    """d activation / dx in the precision of x (src/runtime/cpu/kernels/gemm_epilogue/backward.rs:247-281);
    non-finite values count as 0 (backward.rs:201-202)."""
    one = x.dtype.type(1)
    if act == ACT_RELU:
        d = (x > 0).astype(x.dtype)
    elif act == ACT_GELU:
        c, k = x.dtype.type(0.7978845608028654), x.dtype.type(0.044715)
        t = np.tanh(c * (x + k * x * x * x))
        d = x.dtype.type(0.5) * (one + t) + x.dtype.type(0.5) * x * (one - t * t) * c * (one + x.dtype.type(3) * k * x * x)
    elif act == ACT_SILU:
        sg = one / (one + np.exp(-x))
        d = sg + x * sg * (one - sg)
    elif act == ACT_SIGMOID:
        sg = one / (one + np.exp(-x))
        d = sg * (one - sg)
    elif act == ACT_TANH:
        t = np.tanh(x)
        d = one - t * t
    else:
        d = np.ones_like(x)
    return np.where(np.isfinite(d), d, x.dtype.type(0))


def gemm_bias_act_bwd(dt, grad, a, b, bias, act, precision=np.float32):
    """numr's matmul_bias_activation_bwd on storage arrays (backward.rs:165-245): pre = a @ b + bias and
    grad_pre = grad * act'(pre) in the accumulation type (f32; float64 gives the ground truth), then
    d_a = grad_pre @ b^T, d_b = a^T @ grad_pre, d_bias = column sums, each narrowed once.
    Returns (d_a, d_b, d_bias) as storage arrays of `dt` (float64 arrays when precision is float64)."""
    with np.errstate(over="ignore", invalid="ignore"):
        A = decode(a, dt).astype(precision); B = decode(b, dt).astype(precision)
        G = decode(grad, dt).astype(precision); bias_f = decode(bias, dt).astype(precision)
        pre = A @ B + bias_f[None, :]
        gp = G * _act_derivative(pre, act)
        d_a, d_b, d_bias = gp @ B.T, A.T @ gp, gp.sum(axis=0)
    if precision is np.float64:
        return d_a, d_b, d_bias
    return encode(d_a, dt), encode(d_b, dt), encode(d_bias, dt)


def fp8_matmul(a, b, scale_a, scale_b, out_dt, a_dt=E4M3, b_dt=E4M3, bias=None, residual=None,
               act=ACT_NONE, b_transposed=False, threads=0):
    """numr's fp8_matmul (scalar f32 accumulation in k order), plus the fused bias/act/residual form."""
    a = _c(a, a_dt); b = _c(b, b_dt)
    m, k = a.shape
    n = b.shape[0] if b_transposed else b.shape[1]
    bias = _c(bias, out_dt); residual = _c(residual, out_dt)
    out = np.empty((m, n), dtype=_NP[out_dt])
    lib().orc_fp8_matmul(_p(a), _p(b), a_dt, b_dt, _p(bias), _p(residual), _p(out), out_dt, m, n, k,
                         int(b_transposed), float(scale_a), float(scale_b), act, threads)
    return out


def conv_out_size(n, k, stride, dilation, pad_a, pad_b):
    """compute_output_size (src/ops/conv_common.rs:146-161)."""
    eff, padded = dilation * (k - 1) + 1, n + pad_a + pad_b
    return 0 if padded < eff else (padded - eff) // stride + 1


def conv_transpose_out_size(n, k, stride, dilation, pad_a, pad_b, output_padding):
    """compute_transpose_output_size (src/ops/conv_transpose_common.rs:52-67)."""
    if n == 0:
        return 0
    return max(0, (n - 1) * stride + dilation * (k - 1) + 1 + output_padding - (pad_a + pad_b))


def conv2d(dt, x, w, bias=None, stride=(1, 1), padding=(0, 0, 0, 0), dilation=(1, 1), truth=False, threads=0):
    """numr's CPU conv2d, groups = 1, on storage arrays: x [N, C_in, H, W], w [C_out, C_in, Kh, Kw],
    padding (top, bottom, left, right). f32 accumulation and one narrowing, or float64 (truth=True)."""
    x = _c(x, dt); w = _c(w, dt); bias = _c(bias, dt)
    n, c_in, h, wd = x.shape
    c_out, c_in_w, kh, kw = w.shape
    assert c_in_w == c_in
    oh = conv_out_size(h, kh, stride[0], dilation[0], padding[0], padding[1])
    ow = conv_out_size(wd, kw, stride[1], dilation[1], padding[2], padding[3])
    out = np.empty((n, c_out, oh, ow), dtype=np.float64 if truth else _NP[dt])
    lib().orc_conv(dt, 0, int(truth), _p(x), _p(w), _p(bias), _p(out), n, c_in, c_out, h, wd, kh, kw, oh, ow,
                   stride[0], stride[1], padding[0], padding[2], dilation[0], dilation[1], threads)
    return out


def conv1d(dt, x, w, bias=None, stride=1, padding=(0, 0), dilation=1, truth=False, threads=0):
    """numr's CPU conv1d (groups = 1): x [N, C_in, L], w [C_out, C_in, K], padding (left, right)."""
    out = conv2d(dt, x[:, :, None, :], w[:, :, None, :], bias, (1, stride), (0, 0, padding[0], padding[1]),
                 (1, dilation), truth, threads)
    return out[:, :, 0, :]


def conv_transpose1d(dt, x, w, bias=None, stride=1, padding=(0, 0), output_padding=0, dilation=1, truth=False,
                     threads=0):
    """numr's CPU conv_transpose1d (groups = 1): x [N, C_in, L], w [C_in, C_out, K], padding (left, right)."""
    x = _c(x, dt); w = _c(w, dt); bias = _c(bias, dt)
    n, c_in, length = x.shape
    c_in_w, c_out, k = w.shape
    assert c_in_w == c_in
    ol = conv_transpose_out_size(length, k, stride, dilation, padding[0], padding[1], output_padding)
    out = np.empty((n, c_out, ol), dtype=np.float64 if truth else _NP[dt])
    lib().orc_conv(dt, 1, int(truth), _p(x), _p(w), _p(bias), _p(out), n, c_in, c_out, 1, length, 1, k, 1, ol,
                   1, stride, 0, padding[0], 1, dilation, threads)
    return out


def truth_f64(a_dt, a, b_dt, b, epi_dt=F32, bias=None, residual=None, act=ACT_NONE, scale=1.0,
              b_transposed=False, rows=None, threads=0):
    """float64 ground truth act(scale * A@B + bias) + residual on the decoded operands.

    rows: optional int array selecting which output rows to compute (returns [len(rows), N])."""
    a = _c(a, a_dt); b = _c(b, b_dt)
    m, k = a.shape
    n = b.shape[0] if b_transposed else b.shape[1]
    bias = _c(bias, epi_dt); residual = _c(residual, epi_dt)
    rows_arr = None if rows is None else np.ascontiguousarray(rows, dtype=np.int32)
    count = m if rows_arr is None else len(rows_arr)
    out = np.empty((count, n), dtype=np.float64)
    lib().orc_truth_f64(a_dt, b_dt, epi_dt, _p(a), _p(b), _p(bias), _p(residual), _p(out), m, n, k,
                        int(b_transposed), float(scale), act, _p(rows_arr), count, threads)
    return out


def rel_frobenius(x: np.ndarray, truth: np.ndarray) -> float:
    """||x - truth||_F / ||truth||_F in float64."""
    x = np.asarray(x, dtype=np.float64)
    t = np.asarray(truth, dtype=np.float64)
    den = np.linalg.norm(t.ravel())
    return float(np.linalg.norm((x - t).ravel()) / (den if den > 0 else 1.0))
