"""Parity on the five benchmark configurations themselves, at their stated shapes and seeds.

The inputs are exactly the ones `bench.py` times (`bench.Workload`, numpy `default_rng(seed)` on the
host). Every kernel form the benchmark uses runs here against the CPU oracle: CTA-pair tiles over
several persistent waves, both TMEM accumulators wrapping, several K blocks per stage, 4-D tensor
maps, the cut of the last wave. The reference pins this path the same way: the CPU result is the
truth, integers compare exactly (tests/backend_parity/matmul/i8_cuda.rs:45-95), floats within a
tolerance (tests/common/mod.rs:227-277). Bars here:
  c3 (I8)     the whole 4096 x 4096 output equal to the oracle's, bit for bit;
  c1 (F32)    whole output: numr's F32 tolerance against the oracle, <= 1e-5 relative Frobenius
              error against float64;
  c2 (BF16)   whole output within 1 bf16 ulp of the oracle (same f32 sums, other order), and
              <= 1e-2 relative Frobenius error against float64 on 256 sampled rows;
  c4 (FP8), c5 (BF16, one GPU's shard and the 1792-column shard of 8 GPUs): 256 rows spread over
              every row tile, against the oracle run on those rows and against float64.
"""
import numpy as np
import pytest
import torch

from bench import Workload
from helpers import FROB_TOL, as_f64, assert_allclose_numr, assert_ulp_close, to_numpy
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def _sample_rows(m, count=256, seed=99):
    """`count` rows: one from every block of m/count consecutive rows (so every 128-row tile of every
    CTA is hit), at a seeded offset inside its block."""
    rng = np.random.default_rng(seed)
    block = m // count
    return (np.arange(count) * block + rng.integers(0, block, count)).astype(np.int64)


def _dev(wl):
    return {k: v.to(DEV) for k, v in wl.host_inputs().items()}


def test_c1_f32_gelu_whole_output(client):
    wl = Workload("c1")
    out = wl.run(client, _dev(wl)).cpu().numpy()
    want = O.gemm(O.F32, wl.a.numpy(), wl.b.numpy(), bias=wl.bias.numpy(), act=O.ACT_GELU)
    assert_allclose_numr(out, want, O.F32, k=wl.k, what="c1 vs oracle")
    truth = O.truth_f64(O.F32, wl.a.numpy(), O.F32, wl.b.numpy(), bias=wl.bias.numpy(), act=O.ACT_GELU)
    rel = O.rel_frobenius(out, truth)
    assert rel <= FROB_TOL["f32_exact"], f"c1: relative Frobenius error {rel:.3e} against float64"


@pytest.fixture(scope="module")
def c2_case():
    wl = Workload("c2")
    a, w, bias = _bits16(wl.a), _bits16(wl.w_nk), _bits16(wl.bias)
    want = O.gemm(O.BF16, a, w, bias=bias, act=O.ACT_RELU, b_transposed=True)
    rows = _sample_rows(wl.m)
    truth = O.truth_f64(O.BF16, a, O.BF16, w, epi_dt=O.BF16, bias=bias, act=O.ACT_RELU, b_transposed=True,
                        rows=rows)
    return wl, _dev(wl), want, rows, truth


# Kernel forms chosen by the test, not by the library's cost model: single CTAs and CTA pairs, 1 / 2 / 4
# K blocks per stage, 3-D and 4-D tensor maps, the last wave whole or cut into column slices.
C2_FORMS = [
    {},                                             # what the library chooses for this shape
    {"FORCE_PAIR": 1, "KS": 1}, {"FORCE_PAIR": 1, "KS": 2, "TAIL_CUT": 0}, {"FORCE_PAIR": 1, "MAP4": 0},
    {"FORCE_PAIR": 1, "TAIL_CUT": 2}, {"FORCE_PAIR": 1, "TAIL_CUT": 4},
    {"FORCE_PAIR": 0, "KS": 1}, {"FORCE_PAIR": 0, "KS": 2}, {"FORCE_PAIR": 0, "KS": 4, "FORCE_TILE": 64},
    {"FORCE_PAIR": 0, "MAP4": 0}, {"FORCE_PAIR": 0, "TAIL_CUT": 2},
    {"FORCE_PAIR": 1, "FORCE_TILE": 128}, {"FORCE_PAIR": 0, "FORCE_TILE": 192},
    {"FORCE_PAIR": 1, "FORCE_TILE": 224}, {"FORCE_PAIR": 0, "FORCE_TILE": 160, "TAIL_CUT": 0},
]


@pytest.mark.parametrize("form", C2_FORMS, ids=lambda f: ",".join(f"{k}={v}" for k, v in f.items()) or "default")
def test_c2_bf16_relu_whole_output(client, c2_case, tune, form):
    wl, dev_in, want, rows, truth = c2_case
    tune(**form)
    out = to_numpy(wl.run(client, dev_in), O.BF16)
    # f32 summation-order error of one output: about 2^-22 * K * max|a| * max|b|
    floor = 2.0 ** -22 * wl.k * float(wl.a.float().abs().max()) * float(wl.w_nk.float().abs().max())
    assert_ulp_close(out, want, O.BF16, floor, what=f"c2 {form} vs oracle")
    rel = O.rel_frobenius(as_f64(out[rows], O.BF16), truth)
    assert rel <= FROB_TOL[O.BF16], f"c2 {form}: relative Frobenius error {rel:.3e} against float64"


@pytest.mark.parametrize("form", [{}, {"FORCE_PAIR": 0}, {"FORCE_PAIR": 1, "TAIL_CUT": 0}, {"FORCE_PAIR": 1, "TAIL_CUT": 2}],
                         ids=lambda f: ",".join(f"{k}={v}" for k, v in f.items()) or "default")
def test_c3_i8_whole_output_bit_exact(client, tune, form):
    wl = Workload("c3")
    tune(**form)
    out = wl.run(client, _dev(wl)).cpu().numpy()
    want = O.gemm(O.I8, wl.a.numpy(), wl.b.numpy())
    assert out.dtype == np.int32 and np.array_equal(out, want), "c3: I8 x I8 -> I32 is not bit exact"


def test_c4_fp8_fused_sampled_rows(client):
    wl = Workload("c4")
    out = to_numpy(wl.run(client, _dev(wl)), O.BF16)
    rows = _sample_rows(wl.m)
    a8 = wl.a.view(torch.uint8).numpy()
    b8 = wl.b.view(torch.uint8).numpy()
    bias, res = _bits16(wl.bias), _bits16(wl.residual)
    want = O.fp8_matmul(np.ascontiguousarray(a8[rows]), b8, wl.scale_a, wl.scale_b, O.BF16, bias=bias,
                        residual=np.ascontiguousarray(res[rows]), act=O.ACT_SILU)
    # f32 summation-order error, after the scales: 2^-22 * K * max|a| * max|b| * scale_a * scale_b
    floor = 2.0 ** -22 * wl.k * 448.0 * 448.0 * wl.scale_a * wl.scale_b
    assert_ulp_close(out[rows], want, O.BF16, floor, what="c4 vs oracle")
    truth = O.truth_f64(O.E4M3, a8, O.E4M3, b8, epi_dt=O.BF16, bias=bias, residual=res, act=O.ACT_SILU,
                        scale=float(np.float32(wl.scale_a) * np.float32(wl.scale_b)), rows=rows)
    rel = O.rel_frobenius(as_f64(out[rows], O.BF16), truth)
    assert rel <= FROB_TOL[O.E4M3], f"c4: relative Frobenius error {rel:.3e} against float64"


@pytest.mark.parametrize("world,rank", [(1, 0), (8, 3), (8, 7)], ids=["1gpu", "8gpu-rank3", "8gpu-rank7"])
def test_c5_bf16_silu_shard_sampled_rows(client, world, rank):
    """One GPU's whole problem, and two of the 1792-column shards of the 8-GPU run (each is the
    kernel launch that rank makes): the shard's rows equal the oracle's on the same columns."""
    wl = Workload("c5", world, rank)
    out = to_numpy(wl.run(client, _dev(wl)), O.BF16)
    assert out.shape == (16384, 14336 // world)
    rows = _sample_rows(wl.m)
    a, b = _bits16(wl.a), _bits16(wl.b)
    want = O.gemm(O.BF16, np.ascontiguousarray(a[rows]), b, act=O.ACT_SILU)
    floor = 2.0 ** -22 * wl.k * float(wl.a.float().abs().max()) * float(wl.b.float().abs().max())
    assert_ulp_close(out[rows], want, O.BF16, floor, what=f"c5 shard {rank}/{world} vs oracle")
    truth = O.truth_f64(O.BF16, a, O.BF16, b, epi_dt=O.BF16, act=O.ACT_SILU, rows=rows)
    rel = O.rel_frobenius(as_f64(out[rows], O.BF16), truth)
    assert rel <= FROB_TOL[O.BF16], f"c5 shard {rank}/{world}: relative Frobenius error {rel:.3e}"


def test_c5_shards_equal_the_single_gpu_columns(client):
    """The 8-GPU shards, concatenated, equal the one-GPU result on the same columns bit for bit (the
    order of the additions along K does not depend on how N is cut); checked on two shards."""
    from numr_b200.sharding import column_range
    whole_wl = Workload("c5", 1, 0)
    whole = wl_out = whole_wl.run(client, _dev(whole_wl))
    for rank in (0, 5):
        wl = Workload("c5", 8, rank)
        shard = wl.run(client, _dev(wl))
        cols = column_range(14336, 8, rank)
        assert torch.equal(shard.view(torch.int16), whole[:, cols].contiguous().view(torch.int16)), \
            f"shard {rank} of 8 differs from the one-GPU result on its columns"
    del wl_out


@pytest.mark.parametrize("dt,shape,world", [(O.BF16, (600, 192, 320), 3), (O.F32, (300, 96, 200), 2),
                                            (O.BF16, (2048, 512, 1024), 4)],
                         ids=["bf16-3ranks", "f32-2ranks", "bf16-4ranks-several-waves"])
def test_fused_allgather_store_pattern_on_one_gpu(client, dt, shape, world):
    """The all-gather fused into the epilogue, with the ranks emulated on one GPU: rank r's launch
    stores its column block into every "rank's" buffer (all local here). After all launches every
    buffer holds the whole row-major [M, world * N] result, equal bit for bit to the blocks the plain
    op computes, and nothing outside a block's columns is touched by its launch."""
    from helpers import random_operand, to_torch
    from numr_b200 import GemmActivation
    from numr_b200.sharding import GatheredOutput
    m, n, k = shape
    rng = np.random.default_rng(77)
    a = random_operand(rng, (m, k), dt)
    ta = to_torch(a, dt, DEV)
    tdt = ta.dtype
    bufs = [torch.full((m, n * world), float("nan"), dtype=tdt, device=DEV) for _ in range(world)]
    blocks = []
    for r in range(world):
        b = random_operand(rng, (k, n), dt, 0.1)
        tb = to_torch(b, dt, DEV) if r % 2 == 0 else to_torch(np.ascontiguousarray(b.T), dt, DEV).t()
        blocks.append(client.matmul_activation(ta, tb, GemmActivation.SILU))
        got = client.matmul_activation_allgather(ta, tb, GemmActivation.SILU, GatheredOutput.emulated(bufs, r))
        assert got.data_ptr() == bufs[r].data_ptr()
        torch.cuda.synchronize()
        for buf in bufs:   # columns of the ranks that have not run yet are still untouched
            assert torch.isnan(buf[:, (r + 1) * n:].float()).all()
    want = torch.cat(blocks, dim=1)
    for buf in bufs:
        assert torch.equal(buf.view(torch.uint8), want.view(torch.uint8))
