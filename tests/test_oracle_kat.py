"""Pins the CPU oracle against the known answers of numr's own tests
(tests/golden/numr_kat.json, transcribed from the numr sources each entry cites), against
an independent implementation of the narrow float codecs (torch's CPU casts) and against
float64 ground truth. Runs without a GPU.
"""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import det_values

KAT = json.loads((Path(__file__).parent / "golden" / "numr_kat.json").read_text())


def _batched(oracle, dt, a, b, bias=None):
    """Applies the 2-D oracle op per batch (both operands carry the same batch dims here)."""
    if a.ndim == 2:
        return oracle.gemm(dt, a, b, bias=bias)
    return np.stack([oracle.gemm(dt, a[i], b[i], bias=bias) for i in range(a.shape[0])])


@pytest.mark.parametrize("case", KAT["i8_matmul"], ids=lambda c: c["src"])
def test_i8_matmul_known_answers(oracle, case):
    a = np.array(case["a"], np.int8).reshape(case["a_shape"])
    b = np.array(case["b"], np.int8).reshape(case["b_shape"])
    out = _batched(oracle, oracle.I8, a, b)
    assert out.dtype == np.int32
    assert out.ravel().tolist() == case["out"]


@pytest.mark.parametrize("case", KAT["i8_matmul_bias"], ids=lambda c: c["src"])
def test_i8_matmul_bias_known_answers(oracle, case):
    a = np.array(case["a"], np.int8).reshape(case["a_shape"])
    b = np.array(case["b"], np.int8).reshape(case["b_shape"])
    bias = np.array(case["bias"], np.int32)
    assert _batched(oracle, oracle.I8, a, b, bias).ravel().tolist() == case["out"]


def test_i8_generated_shape_matches_int64_numpy(oracle):
    # tests/backend_parity/matmul/i8_cuda.rs:243-246: 20x9 @ 9x5 modular ramps.
    a = np.array([(i % 61) - 30 for i in range(20 * 9)], np.int8).reshape(20, 9)
    b = np.array([(i * 7 % 59) - 29 for i in range(9 * 5)], np.int8).reshape(9, 5)
    want = a.astype(np.int64) @ b.astype(np.int64)
    assert np.array_equal(oracle.gemm(oracle.I8, a, b), want.astype(np.int32))


def test_i8_saturates_once_with_bias(oracle):
    # The bias joins the wide sum before the single clamp (matmul_int.cu:87-103).
    a = np.full((1, 4), 127, np.int8)
    b = np.full((4, 1), 127, np.int8)
    big = np.array([2**31 - 1], np.int32)
    assert oracle.gemm(oracle.I8, a, b, bias=big).ravel().tolist() == [2**31 - 1]
    neg = np.array([-(2**31)], np.int32)
    assert oracle.gemm(oracle.I8, a, -b, bias=neg).ravel().tolist() == [-(2**31)]


@pytest.mark.parametrize("case", KAT["fp8_matmul"], ids=lambda c: c["src"])
def test_fp8_matmul_known_answers(oracle, case):
    a = oracle.encode(np.array(case["a"], np.float32).reshape(case["a_shape"]), oracle.E4M3)
    b = oracle.encode(np.array(case["b"], np.float32).reshape(case["b_shape"]), oracle.E4M3)
    for out_dt in (oracle.F32, oracle.F16, oracle.BF16):
        out = oracle.fp8_matmul(a, b, case["scale_a"], case["scale_b"], out_dt)
        got = oracle.decode(out, out_dt).ravel() if out_dt != oracle.F32 else out.ravel()
        want = np.array(case["out"], np.float64)
        assert np.all(np.abs(got - want) <= case["atol"] + case["rtol"] * np.abs(want))
    # These inputs are exactly representable, so the f32 result is exact too.
    assert oracle.fp8_matmul(a, b, case["scale_a"], case["scale_b"], oracle.F32).ravel().tolist() == case["out"]


def test_e4m3_codec_known_answers(oracle):
    k = KAT["fp8_e4m3_codec"]
    L = oracle.lib()
    enc, dec = L.orc_f32_to_e4m3, L.orc_e4m3_to_f32
    c = k["constants"]
    assert dec(c["ONE"]) == 1.0 and dec(c["NEG_ONE"]) == -1.0 and dec(c["MAX"]) == 448.0
    assert dec(c["MIN_POSITIVE"]) == 2.0 ** -6 and math.isnan(dec(c["NAN"])) and dec(c["ZERO"]) == 0.0
    for value, bits in k["encode_bits"]:
        assert enc(value) == bits, value
    for m in k["subnormals_roundtrip"]:
        v = m * 2.0 ** -9
        assert enc(v) == m and dec(m) == v and enc(-v) == (0x80 | m) and dec(0x80 | m) == -v
    for v in k["flush_to_zero"]:
        assert dec(enc(v)) == 0.0 and dec(enc(-v)) == 0.0
    for v, want in k["rounding"]:
        assert dec(enc(v)) == want
    for v in k["exact_normals"]:
        assert dec(enc(v)) == v and dec(enc(-v)) == -v
    for v in k["saturate_to_448"]:
        assert dec(enc(v)) == 448.0 and dec(enc(-v)) == -448.0
    assert math.isnan(dec(enc(float("nan"))))


def test_e5m2_codec_known_answers(oracle):
    k = KAT["fp8_e5m2_codec"]
    L = oracle.lib()
    enc, dec = L.orc_f32_to_e5m2, L.orc_e5m2_to_f32
    for value, bits in k["encode_bits"]:
        assert enc(value) == bits
    for m in k["subnormals_roundtrip"]:
        v = m * 2.0 ** -16
        assert enc(v) == m and dec(m) == v and enc(-v) == (0x80 | m)
    for v in k["flush_to_zero"]:
        assert dec(enc(v)) == 0.0 and dec(enc(-v)) == 0.0
    for v, want in k["rounding"]:
        assert dec(enc(v)) == want
    for v in k["exact_normals"]:
        assert dec(enc(v)) == v and dec(enc(-v)) == -v
    for v in k["infinity_preserved"]:
        assert math.isinf(dec(enc(v))) and dec(enc(-v)) < 0
    assert math.isinf(dec(enc(1e9)))          # overflow goes to infinity, not to the largest finite
    assert math.isnan(dec(enc(float("nan"))))


def _independent_bits(x: np.ndarray, torch_dt) -> np.ndarray:
    t = torch.from_numpy(x).to(torch_dt)
    if torch_dt in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.view(torch.uint8).numpy()


def test_codecs_agree_with_torch_cpu_casts(oracle):
    # An independent implementation of RNE narrowing: torch's CPU casts. Compared on values
    # spread over every exponent each format reaches (E4M3 only inside its finite range,
    # where torch does not saturate the same way).
    rng = np.random.default_rng(7)
    x = (rng.standard_normal(400_000) * np.exp(rng.uniform(-45, 20, 400_000))).astype(np.float32)
    x = np.concatenate([x, np.float32([0.0, -0.0, 1.0, -1.0, 448.0, 57344.0, 65504.0])])
    assert np.array_equal(oracle.encode(x, oracle.BF16), _independent_bits(x, torch.bfloat16))
    assert np.array_equal(oracle.encode(x, oracle.F16), _independent_bits(x, torch.float16))
    xe5 = x[np.abs(x) < 57344.0 * 1.06]
    assert np.array_equal(oracle.encode(xe5, oracle.E5M2), _independent_bits(xe5, torch.float8_e5m2))
    xe4 = x[np.abs(x) <= 448.0]
    assert np.array_equal(oracle.encode(xe4, oracle.E4M3), _independent_bits(xe4, torch.float8_e4m3fn))
    # Decoding: all 256 codes.
    codes = np.arange(256, dtype=np.uint8)
    for dt, tdt in ((oracle.E4M3, torch.float8_e4m3fn), (oracle.E5M2, torch.float8_e5m2)):
        d = oracle.decode(codes, dt)
        t = torch.from_numpy(codes).view(tdt).float().numpy()
        assert np.all((d == t) | (np.isnan(d) & np.isnan(t)))
        assert np.array_equal(np.signbit(d), np.signbit(t))
    halfs = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    d = oracle.decode(halfs, oracle.F16)
    t = torch.from_numpy(halfs.view(np.int16)).view(torch.float16).float().numpy()
    assert np.all((d == t) | (np.isnan(d) & np.isnan(t)))


def test_shape_tables(nb_lib):
    """The op layer's shape rules against numr's tables (src/ops/matmul.rs:266-421)."""
    import ctypes
    from numr_b200 import _lib

    def tdesc(shape, dtype=_lib.F32, strides=None):
        d = _lib.TensorDesc()
        d.ptr = 0
        d.dtype = dtype
        d.ndim = len(shape)
        st = strides
        if st is None:
            st, acc = [], 1
            for s in reversed(shape):
                st.insert(0, acc)
                acc *= s
        for i, (s, t) in enumerate(zip(shape, st)):
            d.shape[i] = s
            d.strides[i] = t
        return d

    def out_shape(a, b, bias=None):
        shape = (ctypes.c_int64 * 8)()
        nd = ctypes.c_int32()
        dt = ctypes.c_int32()
        da, db = tdesc(a), tdesc(b)
        dbias = tdesc(bias) if bias is not None else None
        st = nb_lib.numr_b200_matmul_out_shape(ctypes.byref(da), ctypes.byref(db),
                                               ctypes.byref(dbias) if dbias is not None else None, shape,
                                               ctypes.byref(nd), ctypes.byref(dt))
        return None if st != _lib.OK else [shape[i] for i in range(nd.value)]

    s = KAT["shapes"]
    for c in s["validate_matmul_shapes"]:
        got = out_shape(c["a"], c["b"])
        if c["mkn"] is None:
            assert got is None
        else:
            assert got[-2:] == [c["mkn"][0], c["mkn"][2]]
    for c in s["matmul_output_shape"]:
        assert out_shape(c["a"], c["b"]) == c["out"]
    for c in s["matmul_bias_shapes"]:
        assert (out_shape(c["a"], c["b"], c["bias"]) is not None) == c["ok"]
    for c in s["batch_indices"]:
        assert out_shape(c["a"], c["b"]) == c["out"]


def test_f32_blocked_gemm_against_f64_truth(oracle):
    # numr's 128x130x128 f32 parity shape (tests/backend_parity/gemm_epilogue.rs:127-480) with its
    # closed-form inputs, all six activations, against float64.
    m, k, n = 128, 130, 128
    a = det_values(m * k, 0.0).astype(np.float32).reshape(m, k)
    b = det_values(k * n, 1.7).astype(np.float32).reshape(k, n)
    bias = det_values(n, 3.1).astype(np.float32)
    for act in range(6):
        got = oracle.gemm(oracle.F32, a, b, bias=bias, act=act)
        truth = oracle.truth_f64(oracle.F32, a, oracle.F32, b, bias=bias, act=act)
        assert oracle.rel_frobenius(got, truth) < 1e-5
    # transposed-B storage gives the bitwise-same result (tests/matmul_transposed_b.rs).
    bt = np.ascontiguousarray(b.T)
    assert np.array_equal(oracle.gemm(oracle.F32, a, b, bias=bias), oracle.gemm(oracle.F32, a, bt, bias=bias, b_transposed=True))
    # thread count does not change the result (tests/matmul_column_determinism.rs).
    big_a = det_values(300 * 520, 0.0).astype(np.float32).reshape(300, 520)
    big_b = det_values(520 * 700, 1.7).astype(np.float32).reshape(520, 700)
    assert np.array_equal(oracle.gemm(oracle.F32, big_a, big_b, threads=1), oracle.gemm(oracle.F32, big_a, big_b, threads=0))


def test_fused_equals_unfused_identities(oracle):
    # tests/backend_parity/gemm_epilogue.rs:1236-1312.
    m, k, n = 64, 48, 80
    a = det_values(m * k, 0.0).astype(np.float32).reshape(m, k)
    b = det_values(k * n, 1.7).astype(np.float32).reshape(k, n)
    bias = det_values(n, 3.1).astype(np.float32)
    res = det_values(m * n, 5.3).astype(np.float32).reshape(m, n)
    plain = oracle.gemm(oracle.F32, a, b, bias=bias)
    assert np.array_equal(oracle.gemm(oracle.F32, a, b, bias=bias, act=oracle.ACT_NONE), plain)
    assert np.array_equal(oracle.gemm(oracle.F32, a, b, bias=bias, act=oracle.ACT_RELU), np.maximum(plain, 0))
    fused = oracle.gemm(oracle.F32, a, b, bias=bias, residual=res)
    assert np.allclose(fused, plain + res, rtol=1e-5, atol=1e-6)


def test_bf16_modes(oracle):
    # f32-accumulate mode meets the 1e-2 Frobenius bound at K = 4096; the literal in-dtype loop of
    # numr's CPU epilogue ops does not (documented divergence), but agrees at the small K its tests use.
    rng = np.random.default_rng(1)
    m, k, n = 16, 4096, 24
    a = oracle.encode((rng.standard_normal((m, k)) / 64).astype(np.float32), oracle.BF16)
    b = oracle.encode((rng.standard_normal((k, n)) / 64).astype(np.float32), oracle.BF16)
    bias = oracle.encode((rng.standard_normal(n) / 64).astype(np.float32), oracle.BF16)
    truth = oracle.truth_f64(oracle.BF16, a, oracle.BF16, b, epi_dt=oracle.BF16, bias=bias, act=oracle.ACT_RELU)
    f32acc = oracle.decode(oracle.gemm(oracle.BF16, a, b, bias=bias, act=oracle.ACT_RELU), oracle.BF16)
    assert oracle.rel_frobenius(f32acc, truth) < 1e-2
    literal = oracle.decode(oracle.gemm(oracle.BF16, a, b, bias=bias, act=oracle.ACT_RELU, mode=1), oracle.BF16)
    assert oracle.rel_frobenius(literal, truth) > oracle.rel_frobenius(f32acc, truth)
    ks = 48
    small = oracle.gemm(oracle.BF16, a[:, :ks].copy(), b[:ks].copy(), bias=bias, act=oracle.ACT_SILU)
    small_lit = oracle.gemm(oracle.BF16, a[:, :ks].copy(), b[:ks].copy(), bias=bias, act=oracle.ACT_SILU, mode=1)
    d = np.abs(oracle.decode(small, oracle.BF16) - oracle.decode(small_lit, oracle.BF16))
    assert np.all(d <= 0.1 + 1e-2 * np.abs(oracle.decode(small, oracle.BF16)))


@pytest.mark.parametrize("np_t", [np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64])
@pytest.mark.parametrize("b_transposed", [False, True])
def test_wide_int_oracle_against_python_integers(oracle, np_t, b_transposed):
    """The 128-bit-accumulator integer matmul (src/runtime/cpu/kernels/matmul/kernel.rs,
    `matmul_scalar_acc::<T, i128>`; tests in tests/backend_parity/matmul.rs use small values and
    compare exactly): checked here against Python's unbounded integers with full-range operands,
    so the single saturating store, the bias seed and the i128 saturation of the two 64-bit widths
    (wide_acc.rs:109-135) are pinned too."""
    info = np.iinfo(np_t)
    rng = np.random.default_rng(1)
    m, n, k = 7, 9, 13
    a = rng.integers(info.min, info.max, size=(m, k), dtype=np_t, endpoint=True)
    b = rng.integers(info.min, info.max, size=(k, n), dtype=np_t, endpoint=True)
    a[0] = rng.integers(0, 3, size=k).astype(np_t)          # an in-range row
    bias = rng.integers(info.min, info.max, size=n, dtype=np_t, endpoint=True)
    lo128, hi128 = -(1 << 127), (1 << 127) - 1
    clamp = lambda v: min(max(v, lo128), hi128)
    for use_bias in (False, True):
        want = np.empty((m, n), dtype=np_t)
        for i in range(m):
            for j in range(n):
                acc = int(bias[j]) if use_bias else 0
                for p in range(k):                               # k order, i128 saturating mul and add
                    acc = clamp(acc + clamp(int(a[i, p]) * int(b[p, j])))
                want[i, j] = min(max(acc, info.min), info.max)
        got = oracle.matmul_wide_int(a, b.T.copy() if b_transposed else b, bias=bias if use_bias else None,
                                     b_transposed=b_transposed)
        np.testing.assert_array_equal(got, want)


# ------------------------------------------------------------------ convolutions (oracle of the conv-as-GEMM callers)
@pytest.mark.parametrize("case", KAT["conv_transpose1d"], ids=lambda c: c["src"])
def test_conv_transpose1d_known_answers(oracle, case):
    x = np.array(case["x"], np.float32).reshape(1, 1, -1)
    w = np.array(case["w"], np.float32).reshape(1, 1, -1)
    out = oracle.conv_transpose1d(oracle.F32, x, w, stride=case["stride"], padding=tuple(case["padding"]),
                                  output_padding=case["output_padding"], dilation=case["dilation"])
    assert out.ravel().tolist() == case["out"]
    truth = oracle.conv_transpose1d(oracle.F32, x, w, stride=case["stride"], padding=tuple(case["padding"]),
                                    output_padding=case["output_padding"], dilation=case["dilation"], truth=True)
    assert truth.dtype == np.float64 and truth.ravel().tolist() == case["out"]


@pytest.mark.parametrize("case", KAT["conv_forward"], ids=lambda c: c["src"])
def test_conv_forward_known_answers(oracle, case):
    x = np.array(case["x"], np.float32).reshape(case["x_shape"])
    w = np.array(case["w"], np.float32).reshape(case["w_shape"])
    out = oracle.conv1d(oracle.F32, x, w) if case["kind"] == "conv1d" else oracle.conv2d(oracle.F32, x, w)
    assert out.ravel().tolist() == case["out"]


def test_conv_oracle_agrees_with_torch_cpu(oracle):
    """An independent implementation of the same definitions: torch's CPU convolutions in float64,
    with stride, dilation, asymmetric padding (applied as explicit zero padding) and output_padding."""
    import torch.nn.functional as F
    rng = np.random.default_rng(8)
    x = rng.standard_normal((2, 5, 9, 11)).astype(np.float32)
    w = rng.standard_normal((4, 5, 3, 2)).astype(np.float32)
    b = rng.standard_normal(4).astype(np.float32)
    got = oracle.conv2d(oracle.F32, x, w, b, stride=(2, 1), padding=(1, 0, 2, 1), dilation=(1, 2), truth=True)
    xt = F.pad(torch.from_numpy(x).double(), (2, 1, 1, 0))     # (left, right, top, bottom)
    want = F.conv2d(xt, torch.from_numpy(w).double(), torch.from_numpy(b).double(), stride=(2, 1), dilation=(1, 2))
    assert got.shape == tuple(want.shape) and np.allclose(got, want.numpy(), rtol=1e-12, atol=1e-12)
    x1 = rng.standard_normal((2, 6, 7)).astype(np.float32)
    w1 = rng.standard_normal((6, 3, 4)).astype(np.float32)       # [c_in, c_out, k]
    b1 = rng.standard_normal(3).astype(np.float32)
    got = oracle.conv_transpose1d(oracle.F32, x1, w1, b1, stride=2, padding=(2, 2), output_padding=1, dilation=2,
                                  truth=True)
    want = F.conv_transpose1d(torch.from_numpy(x1).double(), torch.from_numpy(w1).double(),
                              torch.from_numpy(b1).double(), stride=2, padding=2, output_padding=1, dilation=2)
    assert got.shape == tuple(want.shape) and np.allclose(got, want.numpy(), rtol=1e-12, atol=1e-12)
    f32 = oracle.conv_transpose1d(oracle.F32, x1, w1, b1, stride=2, padding=(2, 2), output_padding=1, dilation=2)
    assert np.allclose(f32, got, rtol=1e-5, atol=1e-5)
