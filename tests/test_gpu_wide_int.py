"""GPU parity, bit-exact: matmul / matmul_bias for I16, I32, I64, U8, U16, U32, U64 — the widths
numr runs with a 128-bit accumulator and one saturating store (src/runtime/cuda/kernels/matmul_int.cu,
benches/matmul_int.rs) — against the CPU oracle on identical seeded inputs.
"""
import zlib

import numpy as np
import pytest
import torch

from numr_b200 import GemmActivation, UnsupportedDType
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
NP_TYPES = [np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64]
IDS = ["i16", "i32", "i64", "u8", "u16", "u32", "u64"]


def _dev(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _host(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy()


def _rand(rng, shape, np_t, span):
    info = np.iinfo(np_t)
    lo = max(info.min, -span) if info.min < 0 else 0
    hi = min(info.max, span)
    return rng.integers(lo, hi, size=shape, dtype=np.int64 if info.min < 0 else np.uint64, endpoint=True).astype(np_t)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("shape", [(64, 64, 64), (65, 67, 17), (1, 130, 33), (200, 3, 129)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("np_t", NP_TYPES, ids=IDS)
def test_wide_int_matmul_in_range(client, np_t, shape, layout):
    m, n, k = shape
    rng = np.random.default_rng(zlib.crc32(repr((np.dtype(np_t).name, shape, layout)).encode()))
    a = _rand(rng, (m, k), np_t, 11)
    b = _rand(rng, (k, n), np_t, 11)
    tb = _dev(b) if layout == "kn" else _dev(b.T.copy()).t()
    out = client.matmul(_dev(a), tb)
    assert out.dtype == _dev(a).dtype and tuple(out.shape) == (m, n)
    np.testing.assert_array_equal(_host(out), O.matmul_wide_int(a, b))


@pytest.mark.parametrize("np_t", NP_TYPES, ids=IDS)
def test_wide_int_saturates_once_at_the_store(client, np_t):
    """Full-range operands: sums leave the element range; the 128-bit accumulator keeps them exact and
    the store clamps. Rows whose partial sums overflow and come back must not clamp early."""
    info = np.iinfo(np_t)
    rng = np.random.default_rng(7)
    m, n, k = 48, 40, 96
    a = rng.integers(info.min, info.max, size=(m, k), dtype=np_t, endpoint=True)
    b = rng.integers(info.min, info.max, size=(k, n), dtype=np_t, endpoint=True)
    # row 0 / column 0: +max*max then -max*max ... returns to a small in-range value
    a[0, :] = info.max
    b[:, 0] = 0
    if info.min < 0:
        b[0::2, 0] = info.max
        b[1::2, 0] = -info.max
    else:
        b[0, 0] = 1
    want = O.matmul_wide_int(a, b)
    got = _host(client.matmul(_dev(a), _dev(b)))
    np.testing.assert_array_equal(got, want)
    assert want[0, 0] == (0 if info.min < 0 else info.max)
    assert (want == info.max).any()
    if info.min < 0:
        assert (want == info.min).any()


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("np_t", NP_TYPES, ids=IDS)
def test_wide_int_bias_joins_the_accumulator(client, np_t, layout):
    """The bias seeds the wide accumulator: a product sum just past the range plus a bias that brings
    it back is exact, where clamp-then-add would be off."""
    info = np.iinfo(np_t)
    rng = np.random.default_rng(11)
    m, n, k = 33, 70, 20
    a = _rand(rng, (m, k), np_t, 9)
    b = _rand(rng, (k, n), np_t, 9)
    bias = _rand(rng, (n,), np_t, 100)
    if info.min < 0:
        # column 0: sum = max + 5 before the bias, bias = -9  ->  max - 4
        a[:, :] = np.where(np.arange(k) == 0, 1, a)
        b[:, 0] = 0
        b[0, 0] = info.max
        a[:, 1] = 5
        b[1, 0] = 1
        bias[0] = -9
    tb = _dev(b) if layout == "kn" else _dev(b.T.copy()).t()
    got = _host(client.matmul_bias(_dev(a), tb, _dev(bias)))
    want = O.matmul_wide_int(a, b, bias=bias)
    np.testing.assert_array_equal(got, want)
    if info.min < 0:
        assert (want[:, 0] == info.max - 4).all()


@pytest.mark.parametrize("np_t", [np.int32, np.int64, np.uint16], ids=["i32", "i64", "u16"])
def test_wide_int_batched_broadcast_and_empty(client, np_t):
    rng = np.random.default_rng(3)
    a = _rand(rng, (2, 3, 20, 24), np_t, 50)
    b = _rand(rng, (3, 24, 18), np_t, 50)          # broadcast over the leading 2
    got = _host(client.matmul(_dev(a), _dev(b)))
    assert got.shape == (2, 3, 20, 18)
    for i in range(2):
        for j in range(3):
            np.testing.assert_array_equal(got[i, j], O.matmul_wide_int(a[i, j], b[j]))
    # shared 2-D weight against a batch of A
    w = _rand(rng, (24, 10), np_t, 50)
    got = _host(client.matmul(_dev(a), _dev(w)))
    np.testing.assert_array_equal(got[1, 2], O.matmul_wide_int(a[1, 2], w))
    # K == 0: zeros, or the bias in every row; empty outputs are a no-op
    z = client.matmul(_dev(np.zeros((5, 0), np_t)), _dev(np.zeros((0, 7), np_t)))
    assert tuple(z.shape) == (5, 7) and not _host(z).any()
    bias = _rand(rng, (7,), np_t, 100)
    zb = client.matmul_bias(_dev(np.zeros((5, 0), np_t)), _dev(np.zeros((0, 7), np_t)), _dev(bias))
    np.testing.assert_array_equal(_host(zb), np.broadcast_to(bias, (5, 7)))
    e = client.matmul(_dev(np.zeros((0, 4), np_t)), _dev(np.zeros((4, 7), np_t)))
    assert tuple(e.shape) == (0, 7)


def test_wide_int_non_contiguous_operands(client):
    rng = np.random.default_rng(5)
    big_a = _rand(rng, (40, 60), np.int32, 1000)
    big_b = _rand(rng, (60, 50), np.int32, 1000)
    ta, tb = _dev(big_a)[::2, 1:31], _dev(big_b)[5:35, ::2]
    got = _host(client.matmul(ta, tb))
    np.testing.assert_array_equal(got, O.matmul_wide_int(big_a[::2, 1:31], big_b[5:35, ::2]))


def test_wide_int_has_no_epilogue_ops(client):
    a = _dev(np.ones((4, 4), np.int32))
    bias = _dev(np.ones((4,), np.int32))
    with pytest.raises(UnsupportedDType):
        client.matmul_bias_activation(a, a, bias, GemmActivation.RELU)
    with pytest.raises(UnsupportedDType):
        client.matmul_bias_residual(a, a, bias, a)
