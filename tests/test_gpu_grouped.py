"""GPU parity: grouped (MoE) matmul with device-side group offsets against the CPU oracle, on the
shapes numr's own tests use (tests/backend_parity/grouped_matmul.rs:93-300: even, uneven, empty
group, partial last tile, narrow output, ragged K, single group, fused activations, half types) and
on an expert-sized case. The oracle result is numr's definition: one matmul per group on its row range.
"""
import numpy as np
import pytest
import torch

from helpers import FROB_TOL, NAMES, as_f64, assert_allclose_numr, random_operand, to_numpy, to_torch
from numr_b200 import GemmActivation, InvalidArgument, ShapeMismatch
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _offsets(counts):
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


def _oracle(dt, a, b, offsets, act):
    out = np.zeros((a.shape[0], b.shape[2]), dtype=a.dtype)
    for g in range(b.shape[0]):
        s, e = int(offsets[g]), int(offsets[g + 1])
        if e <= s or e > a.shape[0]:
            continue
        out[s:e] = O.gemm(dt, a[s:e], b[g], act=act)
    return out


def _run(client, dt, counts, k, n, act=0, seed=0, frob_key=None):
    rng = np.random.default_rng(seed)
    rows, groups = int(sum(counts)), len(counts)
    a = random_operand(rng, (rows, k), dt, 1.0)
    b = random_operand(rng, (groups, k, n), dt, 1.0 / np.sqrt(max(k, 1)))
    off = _offsets(counts)
    ta, tb = to_torch(a, dt, DEV), to_torch(b, dt, DEV)
    toff = torch.from_numpy(off).to(DEV)
    sentinel = 7.0
    if act:
        out = client.grouped_matmul_activation(ta, tb, toff, GemmActivation(act))
    else:
        out = client.grouped_matmul(ta, tb, toff)
    assert tuple(out.shape) == (rows, n) and out.dtype == ta.dtype
    got = to_numpy(out, dt)
    want = _oracle(dt, a, b, off, act)
    what = f"grouped {NAMES[dt]} counts={counts} k={k} n={n} act={act}"
    assert_allclose_numr(got, want, dt, k=k, operand_scale=float(np.abs(as_f64(a, dt)).max()), what=what)
    truth = np.zeros((rows, n))
    for g in range(groups):
        s, e = int(off[g]), int(off[g + 1])
        if e > s:
            truth[s:e] = O.truth_f64(dt, a[s:e], dt, b[g], epi_dt=dt, act=act)
    rel = O.rel_frobenius(as_f64(got, dt), truth)
    assert rel <= FROB_TOL[frob_key if frob_key else dt], f"{what}: relative Frobenius error {rel:.3e}"
    return out, (ta, tb, toff)


@pytest.mark.parametrize("counts,k,n", [
    ([96, 96, 96, 96], 64, 160), ([5, 70, 33, 120], 64, 160), ([64, 0, 64], 48, 160),
    ([33, 65, 97], 48, 160), ([40, 72], 48, 48), ([48, 48], 37, 160), ([80], 64, 160),
    ([1, 0, 0, 300, 127, 129, 2], 136, 200),
], ids=["even", "uneven", "empty-group", "partial-tile", "narrow", "ragged-k", "single", "mixed"])
def test_grouped_f32_reference_shapes(client, counts, k, n):
    _run(client, O.F32, counts, k, n, frob_key="f32_exact")


@pytest.mark.parametrize("act", [O.ACT_SILU, O.ACT_GELU, O.ACT_RELU], ids=["silu", "gelu", "relu"])
def test_grouped_fused_activation(client, act):
    _run(client, O.F32, [5, 70, 33, 120], 64, 160 if act != O.ACT_RELU else 48, act=act, seed=act, frob_key="f32_exact")


@pytest.mark.parametrize("dt", [O.F16, O.BF16], ids=["f16", "bf16"])
@pytest.mark.parametrize("counts,k,n", [([5, 70, 33, 120], 64, 160), ([40, 72], 48, 48), ([130, 1, 260], 256, 320)],
                         ids=["uneven", "narrow", "multi-tile"])
def test_grouped_half_types(client, dt, counts, k, n):
    _run(client, dt, counts, k, n, seed=3)
    _run(client, dt, counts, k, n, act=O.ACT_SILU, seed=4)


def test_grouped_single_group_matches_dense_matmul(client):
    out, (ta, tb, toff) = _run(client, O.F32, [80], 64, 160, seed=9, frob_key="f32_exact")
    dense = client.matmul(ta, tb[0])
    assert torch.equal(out.view(torch.uint8), dense.view(torch.uint8))


@pytest.mark.parametrize("pair", ["0", "1"], ids=["single-cta", "cta-pair"])
def test_grouped_expert_sized_bf16(client, pair, tune):
    """8 experts, uneven token counts, K = 1024, N = 1536: many row tiles per group, tiles that end
    inside a group, TMA-stored full tiles next to predicated partial ones; with 128-row tiles of single
    CTAs and with 256-row tiles of CTA pairs (a pair's second CTA then often owns no row at all).
    Repeats bit for bit."""
    tune(FORCE_PAIR=pair)
    counts = [700, 0, 129, 1023, 64, 1, 257, 898]
    out, (ta, tb, toff) = _run(client, O.BF16, counts, 1024, 1536, act=O.ACT_SILU, seed=11)
    again = client.grouped_matmul_activation(ta, tb, toff, GemmActivation.SILU)
    assert torch.equal(out.view(torch.uint8), again.view(torch.uint8))


def test_grouped_rows_outside_every_group_are_left_alone(client):
    """Offsets that skip rows (not a partition): only the rows of valid groups are written; a group
    that ends past the row count is skipped, as on numr's CPU path."""
    rng = np.random.default_rng(2)
    dt = O.F32
    a = random_operand(rng, (200, 64), dt)
    b = random_operand(rng, (3, 64, 96), dt, 0.1)
    off = np.array([10, 50, 50, 260], dtype=np.int32)        # group 1 empty, group 2 runs past the rows
    out = client.grouped_matmul(to_torch(a, dt, DEV), to_torch(b, dt, DEV), torch.from_numpy(off).to(DEV))
    got = to_numpy(out, dt)
    want = O.gemm(dt, a[10:50], b[0])
    assert_allclose_numr(got[10:50], want, dt, k=64, what="grouped gap rows")


def test_grouped_zero_rows_and_zero_groups(client):
    a = torch.zeros((0, 32), device=DEV)
    b = torch.zeros((2, 32, 16), device=DEV)
    out = client.grouped_matmul(a, b, torch.zeros(3, dtype=torch.int32, device=DEV))
    assert tuple(out.shape) == (0, 16)
    a = torch.ones((5, 32), device=DEV)
    b0 = torch.zeros((0, 32, 16), device=DEV)
    out = client.grouped_matmul(a, b0, torch.zeros(1, dtype=torch.int32, device=DEV))
    assert tuple(out.shape) == (5, 16) and not out.any()


def test_grouped_argument_errors(client):
    a = torch.zeros((8, 32), device=DEV)
    b = torch.zeros((2, 32, 16), device=DEV)
    off = torch.tensor([0, 4, 8], dtype=torch.int32, device=DEV)
    with pytest.raises(InvalidArgument):
        client.grouped_matmul(a.reshape(2, 4, 32), b, off)                       # a not 2-D
    with pytest.raises(InvalidArgument):
        client.grouped_matmul(a, b[0], off)                                      # b not 3-D
    with pytest.raises(InvalidArgument):
        client.grouped_matmul(a, b, off.to(torch.int64))                         # offsets not I32
    with pytest.raises(InvalidArgument):
        client.grouped_matmul(a, b, off[:2])                                     # wrong offsets length
    with pytest.raises(InvalidArgument):
        client.grouped_matmul(a, b.to(torch.bfloat16), off)                      # dtype mismatch
    with pytest.raises(InvalidArgument):
        client.grouped_matmul(a.to(torch.int8), b.to(torch.int8), off)           # unsupported dtype
    with pytest.raises(ShapeMismatch):
        client.grouped_matmul(a, torch.zeros((2, 31, 16), device=DEV), off)      # k mismatch
