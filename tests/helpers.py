"""Shared helpers for the parity tests: deterministic inputs, storage conversions
between numpy (what the oracle takes) and torch CUDA tensors (what the client takes),
and the tolerance rules of numr's own test suite.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import oracle as O

# oracle dtype code -> torch dtype, numpy storage dtype
TORCH_DT = {
    O.F32: torch.float32, O.BF16: torch.bfloat16, O.F16: torch.float16,
    O.E4M3: torch.float8_e4m3fn, O.E5M2: torch.float8_e5m2, O.I8: torch.int8, O.I32: torch.int32,
}
NAMES = {O.F32: "f32", O.BF16: "bf16", O.F16: "f16", O.E4M3: "e4m3", O.E5M2: "e5m2", O.I8: "i8", O.I32: "i32"}

# BASELINE tolerances: relative Frobenius error against float64 ground truth.
FROB_TOL = {"f32_exact": 1e-5, "f32_tf32": 1e-3, O.BF16: 1e-2, O.F16: 1e-2, O.E4M3: 2e-2, O.E5M2: 2e-2}


def det_values(n: int, phase: float) -> np.ndarray:
    """numr's closed-form test generator (tests/backend_parity/gemm_epilogue.rs:116-122):
    sin(0.013 i + phase) * 0.5 + cos(0.0047 i + phase) * 0.3, evaluated in float64."""
    i = np.arange(n, dtype=np.float64)
    return np.sin(0.013 * i + phase) * 0.5 + np.cos(0.0047 * i + phase) * 0.3


PHASE_A, PHASE_B, PHASE_BIAS, PHASE_RES = 0.0, 1.7, 3.1, 5.3


def to_torch(x: np.ndarray, dt: int, device) -> torch.Tensor:
    """numpy storage array -> torch tensor of the matching dtype on `device`."""
    x = np.ascontiguousarray(x)
    if dt in (O.BF16, O.F16):
        t = torch.from_numpy(x.view(np.int16)).view(TORCH_DT[dt])
    elif dt in (O.E4M3, O.E5M2):
        t = torch.from_numpy(x).view(TORCH_DT[dt])
    else:
        t = torch.from_numpy(x)
    return t.to(device)


def to_numpy(t: torch.Tensor, dt: int) -> np.ndarray:
    """torch tensor -> numpy storage array (bit patterns for 16/8-bit floats)."""
    t = t.detach().contiguous().cpu()
    if dt in (O.BF16, O.F16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if dt in (O.E4M3, O.E5M2):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def as_f64(x: np.ndarray, dt: int) -> np.ndarray:
    if dt in (O.F32, O.I8, O.I32):
        return x.astype(np.float64)
    return O.decode(x, dt).astype(np.float64)


def numr_tolerance(dt: int):
    """tolerance_for_dtype (tests/common/mod.rs:227-237): (rtol, atol)."""
    return {O.F32: (1e-5, 1e-6), O.F16: (1e-2, 0.1), O.BF16: (1e-2, 0.1), O.E4M3: (0.3, 2.5),
            O.E5M2: (1.0, 2.5)}[dt]


def long_k_bound(dt: int, k: int, operand_scale: float) -> float:
    """gemm_long_k_tolerance (tests/common/mod.rs:270-277): absolute bound atol + rtol*sqrt(K)*max(1, scale)."""
    rtol, atol = numr_tolerance(dt)
    return atol + rtol * math.sqrt(k) * max(1.0, operand_scale)


def assert_allclose_numr(got: np.ndarray, want: np.ndarray, dt: int, k: int = 0, operand_scale: float = 1.0,
                         what: str = ""):
    """|got - want| <= atol + rtol*|want|, or the long-K absolute bound when k is given."""
    g = as_f64(got, dt)
    w = as_f64(want, dt)
    assert g.shape == w.shape, f"{what}: shape {g.shape} vs {w.shape}"
    rtol, atol = numr_tolerance(dt)
    bound = atol + rtol * np.abs(w)
    if k:
        bound = np.maximum(bound, long_k_bound(dt, k, operand_scale))
    both_nan = np.isnan(g) & np.isnan(w)
    bad = ~(np.abs(g - w) <= bound) & ~both_nan
    if bad.any():
        idx = np.argwhere(bad)[0]
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements out of tolerance; first at {tuple(idx)}: "
                             f"got {g[tuple(idx)]}, want {w[tuple(idx)]}")


def random_operand(rng, shape, dt: int, scale: float = 1.0) -> np.ndarray:
    """Random storage array of dtype `dt` (normal values scaled, or uniform ints for I8)."""
    if dt == O.I8:
        return rng.integers(-127, 128, size=shape).astype(np.int8)
    if dt == O.I32:
        return rng.integers(-1000, 1001, size=shape).astype(np.int32)
    return O.encode((rng.standard_normal(shape) * scale).astype(np.float32), dt)


_MANTISSA_BITS = {O.BF16: 7, O.F16: 10, O.F32: 23, O.E4M3: 3, O.E5M2: 2}


def assert_ulp_close(got: np.ndarray, want: np.ndarray, dt: int, floor: float, max_ulp: float = 1.0,
                     max_frac: float = 0.05, what: str = ""):
    """Two roundings of the same sums: every element within `max_ulp` units in the last place of the
    output type (plus `floor`, the summation-order error of the f32 accumulation itself, which decides
    results next to a rounding boundary or next to zero), and at most `max_frac` of them different at
    all. This is what "same result up to the order of the f32 additions" means for a narrowed output;
    the (rtol, atol) rule numr's tests use is far looser when the outputs are small."""
    g, w = as_f64(got, dt), as_f64(want, dt)
    assert g.shape == w.shape, f"{what}: shape {g.shape} vs {w.shape}"
    mag = np.maximum(np.abs(g), np.abs(w))
    with np.errstate(divide="ignore"):
        ulp = np.exp2(np.floor(np.log2(np.where(mag > 0, mag, 1.0))) - _MANTISSA_BITS[dt])
    diff = np.abs(g - w)
    bad = ~(diff <= max_ulp * ulp + floor) & ~(np.isnan(g) & np.isnan(w))
    if bad.any():
        idx = tuple(np.argwhere(bad)[0])
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements differ by more than {max_ulp} ulp; "
                             f"first at {idx}: got {g[idx]}, want {w[idx]}")
    frac = float((diff > floor).mean())
    assert frac <= max_frac, f"{what}: {frac:.2%} of the elements differ (allowed {max_frac:.0%})"
    return frac
