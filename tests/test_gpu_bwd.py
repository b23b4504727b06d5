"""GPU parity: backward of the fused GEMM epilogue (numr matmul_bias_activation_bwd) against the CPU
oracle (f32 restatement of src/runtime/cpu/kernels/gemm_epilogue/backward.rs) and float64 ground truth.
Tolerances: relative Frobenius error vs float64 1e-5 (exact F32), 1e-2 (BF16 / F16; grad_pre is kept
in the operand type between the GEMMs here, in f32 by the reference)."""
import numpy as np
import pytest
import torch

from helpers import NAMES, as_f64, random_operand, to_numpy, to_torch
from numr_b200 import DTypeMismatch, GemmActivation, UnsupportedDType
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {O.F32: 1e-5, O.BF16: 1e-2, O.F16: 1e-2}


def _case(client, dt, m, n, k, act, layout="kn", seed=0):
    rng = np.random.default_rng(seed)
    a = random_operand(rng, (m, k), dt, 1.0)
    b = random_operand(rng, (k, n), dt, 1.0 / np.sqrt(k))
    bias = random_operand(rng, (n,), dt, 0.5)
    grad = random_operand(rng, (m, n), dt, 1.0)
    tb = to_torch(b, dt, DEV) if layout == "kn" else to_torch(np.ascontiguousarray(b.T), dt, DEV).t()
    d_a, d_b, d_bias = client.matmul_bias_activation_bwd(to_torch(grad, dt, DEV), to_torch(a, dt, DEV), tb,
                                                         to_torch(bias, dt, DEV), GemmActivation(act))
    assert tuple(d_a.shape) == (m, k) and tuple(d_b.shape) == (k, n) and tuple(d_bias.shape) == (n,)
    truth = O.gemm_bias_act_bwd(dt, grad, a, b, bias, act, precision=np.float64)
    port = O.gemm_bias_act_bwd(dt, grad, a, b, bias, act)
    for name, got, tr, po in zip(("d_a", "d_b", "d_bias"), (d_a, d_b, d_bias), truth, port):
        g64 = as_f64(to_numpy(got, dt), dt)
        rel = O.rel_frobenius(g64, tr)
        rel_port = O.rel_frobenius(as_f64(po, dt), tr)
        what = f"{name} {NAMES[dt]} {layout} {m}x{n}x{k} act={act}"
        assert rel <= TOL[dt], f"{what}: relative Frobenius error {rel:.3e}"
        # no worse than a small multiple of what the f32 CPU restatement itself achieves
        assert rel <= max(4 * rel_port, TOL[dt] / 4), f"{what}: {rel:.3e} vs CPU port {rel_port:.3e}"


@pytest.mark.parametrize("act", [0, 1, 2, 3, 4, 5], ids=["none", "relu", "gelu", "silu", "sigmoid", "tanh"])
@pytest.mark.parametrize("dt", [O.F32, O.BF16], ids=["f32", "bf16"])
def test_bwd_every_activation(client, dt, act):
    _case(client, dt, 96, 160, 72, act, seed=act)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("dt,shape", [(O.F32, (130, 100, 200)), (O.BF16, (300, 264, 520)), (O.F16, (64, 72, 40)),
                                      (O.BF16, (1024, 512, 768))], ids=["f32-ragged", "bf16-ragged", "f16-small", "bf16-large"])
def test_bwd_shapes_and_weight_layouts(client, dt, shape, layout):
    m, n, k = shape
    _case(client, dt, m, n, k, O.ACT_GELU, layout=layout, seed=m)


def test_bwd_identities(client):
    """activation None: d_a = grad @ b^T, d_b = a^T @ grad, d_bias = column sums of grad, whatever the bias."""
    rng = np.random.default_rng(5)
    dt = O.F32
    a, b = random_operand(rng, (50, 40), dt), random_operand(rng, (40, 30), dt)
    grad, bias = random_operand(rng, (50, 30), dt), random_operand(rng, (30,), dt)
    ta, tb, tg = to_torch(a, dt, DEV), to_torch(b, dt, DEV), to_torch(grad, dt, DEV)
    d_a, d_b, d_bias = client.matmul_bias_activation_bwd(tg, ta, tb, to_torch(bias, dt, DEV), GemmActivation.NONE)
    assert torch.allclose(d_a, client.matmul(tg, tb.t()), rtol=1e-5, atol=1e-5)
    assert torch.allclose(d_b, client.matmul(ta.t(), tg), rtol=1e-5, atol=1e-5)
    assert torch.allclose(d_bias, tg.sum(0), rtol=1e-5, atol=1e-5)
    again = client.matmul_bias_activation_bwd(tg, ta, tb, to_torch(bias, dt, DEV), GemmActivation.NONE)
    assert all(torch.equal(x, y) for x, y in zip((d_a, d_b, d_bias), again))


def test_bwd_empty_and_errors(client):
    z = lambda *s: torch.zeros(s, device=DEV)
    d_a, d_b, d_bias = client.matmul_bias_activation_bwd(z(0, 6), z(0, 8), z(8, 6), z(6), GemmActivation.RELU)
    assert tuple(d_a.shape) == (0, 8) and not d_b.any() and not d_bias.any()
    with pytest.raises(DTypeMismatch):
        client.matmul_bias_activation_bwd(z(4, 6).bfloat16(), z(4, 8), z(8, 6), z(6), GemmActivation.RELU)
    with pytest.raises(UnsupportedDType):
        i8 = torch.zeros((4, 8), dtype=torch.int8, device=DEV)
        client.matmul_bias_activation_bwd(torch.zeros((4, 8), dtype=torch.int32, device=DEV), i8, i8.t().contiguous().t(),
                                          torch.zeros(8, dtype=torch.int32, device=DEV), GemmActivation.RELU)


@pytest.mark.parametrize("dt", [O.F32, O.BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shared_b", [True, False], ids=["one-weight", "weight-per-batch"])
def test_bwd_batched(client, dt, shared_b):
    """a and grad with leading batch dimensions (src/ops/cuda/gemm_epilogue.rs:293-300). One 2-D weight
    for all batches: d_b and d_bias sum over the batches (the same as folding them into the rows). One
    weight per batch: d_b[i] = a[i]^T @ grad_pre[i] per batch, d_bias over all of them."""
    lead, m, n, k = (2, 3), 70, 96, 56
    act = O.ACT_SILU
    rng = np.random.default_rng(31)
    a = random_operand(rng, lead + (m, k), dt, 1.0)
    b = random_operand(rng, ((k, n) if shared_b else lead + (k, n)), dt, 1.0 / np.sqrt(k))
    bias = random_operand(rng, (n,), dt, 0.5)
    grad = random_operand(rng, lead + (m, n), dt, 1.0)
    d_a, d_b, d_bias = client.matmul_bias_activation_bwd(to_torch(grad, dt, DEV), to_torch(a, dt, DEV),
                                                         to_torch(b, dt, DEV), to_torch(bias, dt, DEV),
                                                         GemmActivation(act))
    assert tuple(d_a.shape) == a.shape and tuple(d_b.shape) == b.shape and tuple(d_bias.shape) == (n,)
    nb = int(np.prod(lead))
    a2, g2 = a.reshape(nb, m, k), grad.reshape(nb, m, n)
    if shared_b:
        t_a, t_b, t_bias = O.gemm_bias_act_bwd(dt, g2.reshape(nb * m, n), a2.reshape(nb * m, k), b, bias, act,
                                               precision=np.float64)
        t_a = t_a.reshape(a.shape)
    else:
        b2 = b.reshape(nb, k, n)
        parts = [O.gemm_bias_act_bwd(dt, g2[i], a2[i], b2[i], bias, act, precision=np.float64) for i in range(nb)]
        t_a = np.stack([p[0] for p in parts]).reshape(a.shape)
        t_b = np.stack([p[1] for p in parts]).reshape(b.shape)
        t_bias = sum(p[2] for p in parts)
    for name, got, tr in (("d_a", d_a, t_a), ("d_b", d_b, t_b), ("d_bias", d_bias, t_bias)):
        rel = O.rel_frobenius(as_f64(to_numpy(got, dt), dt), tr)
        assert rel <= TOL[dt], f"batched {name} {NAMES[dt]} shared_b={shared_b}: relative Frobenius error {rel:.3e}"
