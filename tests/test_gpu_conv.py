"""Convolutions through the GEMM path (conv1d, conv2d, conv_transpose1d; groups = 1) against the CPU
oracle's direct convolutions, on the shapes and closed-form inputs of the reference's own parity
tests for this path (tests/backend_parity/conv2d_im2col.rs:113-257, conv_transpose1d_gemm.rs:131-183)
plus conv1d shapes that clear its gate (src/ops/cuda/conv1d_im2col.rs:38-98: contraction >= 2048).
The GEMM reassociates the sum of the direct kernel, so the bar is the reference's accumulation-aware
bound (gemm_long_k_tolerance, tests/common/mod.rs:270-277) against the oracle and the stated
relative-Frobenius bounds against float64.
"""
import numpy as np
import pytest
import torch

from helpers import FROB_TOL, NAMES, as_f64, assert_allclose_numr, to_numpy, to_torch
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [O.F32, O.BF16, O.F16]


def gemm_input(n):    # conv2d_im2col.rs:32-34
    return ((np.arange(n) % 13).astype(np.float64) - 6.0) * 0.05


def gemm_weight(n):   # conv2d_im2col.rs:39-41
    return ((np.arange(n) % 9).astype(np.float64) - 4.0) * 0.03


def gemm_bias(n):     # conv2d_im2col.rs:43-45
    return np.arange(n).astype(np.float64) * 0.01 - 0.02


def _enc(values, shape, dt):
    return O.encode(np.asarray(values, np.float32).reshape(shape), dt)


def _check(got_t, want, truth, dt, contraction, scale, what):
    got = to_numpy(got_t, dt)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert_allclose_numr(got, want, dt, k=contraction, operand_scale=scale, what=what)
    rel = O.rel_frobenius(as_f64(got, dt), truth)
    assert rel <= FROB_TOL["f32_exact" if dt == O.F32 else dt], f"{what}: relative Frobenius error {rel:.3e}"


CONV2D_CASES = [   # (label, input shape, weight shape, bias?, stride, padding (t, b, l, r), dilation)
    ("plain", (1, 16, 6, 6), (4, 16, 4, 4), True, (1, 1), (0, 0, 0, 0), (1, 1)),
    ("asymmetric_spatial", (1, 16, 10, 8), (4, 16, 8, 4), False, (1, 1), (0, 0, 0, 0), (1, 1)),
    ("stride_dilation_asymmetric_padding", (1, 16, 9, 11), (4, 16, 4, 4), True, (2, 1), (1, 0, 2, 1), (1, 2)),
    ("batched", (2, 16, 6, 6), (4, 16, 4, 4), True, (1, 1), (0, 0, 0, 0), (1, 1)),
    ("partial_tile", (1, 16, 6, 10), (4, 16, 4, 4), False, (1, 1), (0, 0, 0, 0), (1, 1)),
    ("wide", (3, 64, 20, 24), (200, 64, 3, 3), True, (1, 1), (1, 1, 1, 1), (1, 1)),        # several tiles in M and N
    ("odd_contraction", (2, 7, 9, 9), (33, 7, 3, 3), True, (1, 2), (0, 1, 1, 0), (1, 1)),  # contraction 63: weight re-pitched
]


@pytest.mark.parametrize("dt", DTYPES, ids=lambda d: NAMES[d])
@pytest.mark.parametrize("case", CONV2D_CASES, ids=lambda c: c[0])
def test_conv2d_as_gemm(client, case, dt):
    label, xs, ws, use_bias, stride, padding, dilation = case
    x, w = _enc(gemm_input(int(np.prod(xs))), xs, dt), _enc(gemm_weight(int(np.prod(ws))), ws, dt)
    b = _enc(gemm_bias(ws[0]), (ws[0],), dt) if use_bias else None
    out = client.conv2d(to_torch(x, dt, DEV), to_torch(w, dt, DEV), to_torch(b, dt, DEV) if use_bias else None,
                        stride, padding, dilation)
    want = O.conv2d(dt, x, w, b, stride, padding, dilation)
    truth = O.conv2d(dt, x, w, b, stride, padding, dilation, truth=True)
    _check(out, want, truth, dt, ws[1] * ws[2] * ws[3], 0.3, f"conv2d {label} {NAMES[dt]}")


CONV1D_CASES = [   # (label, input shape, weight shape, bias?, stride, padding (l, r), dilation)
    ("gate", (1, 512, 20), (8, 512, 4), True, 1, (0, 0), 1),                 # contraction 2048, the gate's floor
    ("stride_dilation_padding", (2, 256, 37), (16, 256, 8), True, 2, (3, 1), 2),
    ("long_output", (1, 128, 1000), (130, 128, 16), False, 1, (8, 7), 1),
    ("moving_sum", (1, 1, 5), (1, 1, 3), False, 1, (0, 0), 1),               # tests/backend_parity/conv.rs:18-20
]


@pytest.mark.parametrize("dt", DTYPES, ids=lambda d: NAMES[d])
@pytest.mark.parametrize("case", CONV1D_CASES, ids=lambda c: c[0])
def test_conv1d_as_gemm(client, case, dt):
    label, xs, ws, use_bias, stride, padding, dilation = case
    x, w = _enc(gemm_input(int(np.prod(xs))), xs, dt), _enc(gemm_weight(int(np.prod(ws))), ws, dt)
    if label == "moving_sum":
        x, w = _enc([1, 2, 3, 4, 5], xs, dt), _enc([1, 1, 1], ws, dt)
    b = _enc(gemm_bias(ws[0]), (ws[0],), dt) if use_bias else None
    out = client.conv1d(to_torch(x, dt, DEV), to_torch(w, dt, DEV), to_torch(b, dt, DEV) if use_bias else None,
                        stride, padding, dilation)
    want = O.conv1d(dt, x, w, b, stride, padding, dilation)
    truth = O.conv1d(dt, x, w, b, stride, padding, dilation, truth=True)
    _check(out, want, truth, dt, ws[1] * ws[2], 0.3, f"conv1d {label} {NAMES[dt]}")
    if label == "moving_sum":
        assert as_f64(to_numpy(out, dt), dt).ravel().tolist() == [6.0, 9.0, 12.0]


CONVT_CASES = [   # (label, input shape, weight shape [c_in, c_out, k], bias?, stride, padding, output_padding, dilation)
    ("boundary", (1, 2048, 5), (2048, 4, 4), False, 1, (0, 0), 0, 1),        # conv_transpose1d_gemm.rs:140-156
    ("stride_dilation_output_padding", (2, 1024, 6), (1024, 8, 8), True, 2, (2, 1), 1, 2),   # :165-182
    ("upsample", (1, 1, 4), (1, 1, 3), False, 2, (0, 0), 0, 1),              # tests/backend_parity/conv.rs:271-274
    ("wide", (2, 96, 50), (96, 150, 5), True, 3, (1, 2), 2, 1),
]


@pytest.mark.parametrize("dt", DTYPES, ids=lambda d: NAMES[d])
@pytest.mark.parametrize("case", CONVT_CASES, ids=lambda c: c[0])
def test_conv_transpose1d_as_gemm(client, case, dt):
    label, xs, ws, use_bias, stride, padding, output_padding, dilation = case
    x, w = _enc(gemm_input(int(np.prod(xs))), xs, dt), _enc(gemm_weight(int(np.prod(ws))), ws, dt)
    if label == "upsample":
        x, w = _enc([1.0, -2.0, 0.5, 3.0], xs, dt), _enc([0.5, -1.5, 2.0], ws, dt)
    b = _enc(gemm_bias(ws[1]), (ws[1],), dt) if use_bias else None
    out = client.conv_transpose1d(to_torch(x, dt, DEV), to_torch(w, dt, DEV),
                                  to_torch(b, dt, DEV) if use_bias else None, stride, padding, output_padding, dilation)
    want = O.conv_transpose1d(dt, x, w, b, stride, padding, output_padding, dilation)
    truth = O.conv_transpose1d(dt, x, w, b, stride, padding, output_padding, dilation, truth=True)
    _check(out, want, truth, dt, ws[0] * ws[2], 0.3, f"conv_transpose1d {label} {NAMES[dt]}")


def test_conv_rejections(client):
    x = torch.zeros((1, 4, 8), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((6, 2, 3), dtype=torch.bfloat16, device=DEV)
    from numr_b200.client import ShapeMismatch, UnsupportedDType
    with pytest.raises(UnsupportedDType):
        client.conv1d(x, torch.zeros((6, 4, 3), dtype=torch.bfloat16, device=DEV), groups=2)
    with pytest.raises(ShapeMismatch):
        client.conv1d(x, w)
    with pytest.raises(UnsupportedDType):
        client.conv1d(x.to(torch.int8), torch.zeros((6, 4, 3), dtype=torch.int8, device=DEV))
    # kernel larger than the padded input: empty output, nothing launched
    out = client.conv1d(x, torch.zeros((6, 4, 20), dtype=torch.bfloat16, device=DEV))
    assert tuple(out.shape) == (1, 6, 0)
