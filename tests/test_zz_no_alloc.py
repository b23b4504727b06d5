"""The allocation-free GEMM entry point, numr_b200_gemm_static_scratch.

Some callers cannot obtain a workspace: code running inside another framework's stream hook, a
host replaying a captured graph with its allocator frozen, an embedding that owns nothing but its
input and output buffers. For them the library carries a fixed scratch array in its device image.
This test calls that entry point through the raw C ABI, twice in a row (the scratch keeps the
first call's contents, so the second call must not depend on it being clean), and checks each
result against numr_b200_gemm fed the same problem with a caller-allocated workspace.

Collected last (file name) so that a run stopping at the first failure has already run every
other test; it also passes on its own in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

from numr_b200 import _lib

pytestmark = pytest.mark.gpu


def _desc(m, n, k, f32_mode, activation):
    d = _lib.GemmDesc()
    d.a_dtype = d.b_dtype = d.out_dtype = d.bias_dtype = _lib.F32
    d.batch, d.m, d.n, d.k, d.a_batch, d.b_batch = 1, m, n, k, 1, 1
    d.b_layout, d.activation, d.f32_mode = _lib.B_KN, activation, f32_mode
    d.scale_a = d.scale_b = 1.0
    return d


def test_static_scratch_matches_workspace_entry_twice(nb_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    cap = nb_lib.numr_b200_static_scratch_bytes()
    assert cap == 16 << 20
    rng = np.random.default_rng(21)
    # two different problems back to back: the second finds the first one's leftovers in the scratch
    cases = [(300, 200, 260, _lib.F32_EXACT, 2), (129, 515, 77, _lib.F32_TF32, 0)]
    for m, n, k, mode, act in cases:
        a = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32)).to(dev)
        b = torch.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32)).to(dev)
        bias = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).to(dev)
        d = _desc(m, n, k, mode, act)
        need = nb_lib.numr_b200_gemm_workspace_bytes(ctypes.byref(d), a.data_ptr(), b.data_ptr())
        assert 0 < need <= cap
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        want = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
        st = nb_lib.numr_b200_gemm(ctypes.byref(d), a.data_ptr(), b.data_ptr(), bias.data_ptr(), None,
                                   want.data_ptr(), ws.data_ptr(), need, stream, 0)
        assert st == _lib.OK, _lib.last_error()
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
        st = nb_lib.numr_b200_gemm_static_scratch(ctypes.byref(d), a.data_ptr(), b.data_ptr(), bias.data_ptr(),
                                                  None, got.data_ptr(), stream, 0)
        assert st == _lib.OK, _lib.last_error()
        torch.cuda.synchronize()
        # same kernels on the same operand bits: identical, well inside the 1e-5 / 1e-3 parity bounds
        assert torch.equal(got, want)
        truth = a.double().cpu().numpy() @ b.double().cpu().numpy() + bias.double().cpu().numpy()
        if act == 2:
            truth = 0.5 * truth * (1.0 + np.tanh(0.7978845608028654 * (truth + 0.044715 * truth ** 3)))
        rel = np.linalg.norm(got.double().cpu().numpy() - truth) / np.linalg.norm(truth)
        assert rel <= (1e-5 if mode == _lib.F32_EXACT else 1e-3)


def test_static_scratch_rejects_oversized_problem(nb_lib):
    # exact-mode 2048^3 needs 64 MiB of scratch: refused before anything is launched (no pointer is read)
    d = _desc(2048, 2048, 2048, _lib.F32_EXACT, 0)
    st = nb_lib.numr_b200_gemm_static_scratch(ctypes.byref(d), 4096, 8192, None, None, 16384, None, 0)
    assert st == _lib.EWORKSPACE
    msg = _lib.last_error()
    assert "scratch" in msg and str(16 << 20) in msg


def _raw(nb_lib, d, a, b, bias, out, stream, static):
    if static:
        return nb_lib.numr_b200_gemm_static_scratch(ctypes.byref(d), a.data_ptr(), b.data_ptr(),
                                                    bias.data_ptr() if bias is not None else None, None,
                                                    out.data_ptr(), stream, 0)
    need = nb_lib.numr_b200_gemm_workspace_bytes(ctypes.byref(d), a.data_ptr(), b.data_ptr())
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=a.device)
    return nb_lib.numr_b200_gemm(ctypes.byref(d), a.data_ptr(), b.data_ptr(),
                                 bias.data_ptr() if bias is not None else None, None, out.data_ptr(),
                                 ws.data_ptr(), need, stream, 0)


def test_static_scratch_other_uses_of_the_array(nb_lib):
    """The array's other users, each against numr_b200_gemm and the CPU oracle: a BF16 operand with
    odd K (its rows are re-pitched into the scratch), a long-K problem that needs no operand
    preparation but cuts K (partial sums in the scratch), and an integer width that uses no
    scratch at all and passes straight through."""
    from helpers import as_f64, random_operand, to_numpy, to_torch
    from oracle import oracle as O
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(22)

    def desc(dt, out_dt, m, n, k):
        d = _lib.GemmDesc()
        d.a_dtype = d.b_dtype = dt
        d.out_dtype = d.bias_dtype = out_dt
        d.batch, d.m, d.n, d.k, d.a_batch, d.b_batch = 1, m, n, k, 1, 1
        d.b_layout, d.activation, d.f32_mode = _lib.B_KN, 0, _lib.F32_EXACT
        d.scale_a = d.scale_b = 1.0
        return d

    # BF16, K = 77 (rows of 154 bytes: not a multiple of 16) -> pad_rows into the scratch; twice
    for m, n, k in ((130, 96, 77), (64, 200, 131)):
        a, b = random_operand(rng, (m, k), O.BF16), random_operand(rng, (k, n), O.BF16, 0.1)
        ta, tb = to_torch(a, O.BF16, dev), to_torch(b, O.BF16, dev)
        d = desc(_lib.BF16, _lib.BF16, m, n, k)
        assert nb_lib.numr_b200_gemm_workspace_bytes(ctypes.byref(d), ta.data_ptr(), tb.data_ptr()) > 0
        outs = []
        for static in (False, True):
            out = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
            assert _raw(nb_lib, d, ta, tb, None, out, stream, static) == _lib.OK, _lib.last_error()
            outs.append(out)
        torch.cuda.synchronize()
        assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
        truth = O.truth_f64(O.BF16, a, O.BF16, b)
        assert O.rel_frobenius(as_f64(to_numpy(outs[1], O.BF16), O.BF16), truth) <= 1e-2

    # BF16 256 x 256 x 16384: operands are read in place, K is cut over the idle SMs -> only the
    # partial-sum scratch is used
    m, n, k = 256, 256, 16384
    a, b = random_operand(rng, (m, k), O.BF16), random_operand(rng, (k, n), O.BF16, 0.02)
    ta, tb = to_torch(a, O.BF16, dev), to_torch(b, O.BF16, dev)
    d = desc(_lib.BF16, _lib.BF16, m, n, k)
    need = nb_lib.numr_b200_gemm_workspace_bytes(ctypes.byref(d), ta.data_ptr(), tb.data_ptr())
    assert 0 < need <= nb_lib.numr_b200_static_scratch_bytes(), "expected a K cut that fits the built-in scratch"
    outs = []
    for static in (False, True, True):
        out = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
        assert _raw(nb_lib, d, ta, tb, None, out, stream, static) == _lib.OK, _lib.last_error()
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[1].view(torch.int16), outs[2].view(torch.int16))
    truth = O.truth_f64(O.BF16, a, O.BF16, b)
    assert O.rel_frobenius(as_f64(to_numpy(outs[1], O.BF16), O.BF16), truth) <= 1e-2

    # I32 (CUDA cores, 128-bit accumulator): no scratch, same call as numr_b200_gemm
    m, n, k = 50, 70, 90
    a = rng.integers(-1000, 1000, (m, k)).astype(np.int32)
    b = rng.integers(-1000, 1000, (k, n)).astype(np.int32)
    ta, tb = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
    d = desc(_lib.I32, _lib.I32, m, n, k)
    out = torch.zeros((m, n), dtype=torch.int32, device=dev)
    assert _raw(nb_lib, d, ta, tb, None, out, stream, True) == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), O.matmul_wide_int(a, b))


def test_static_scratch_refuses_another_devices_index(nb_lib):
    # the scratch address belongs to the current device: an index naming another one is an error
    torch.cuda.set_device(0)
    d = _desc(64, 64, 64, _lib.F32_EXACT, 0)
    x = torch.zeros((64, 64), dtype=torch.float32, device="cuda:0")
    st = nb_lib.numr_b200_gemm_static_scratch(ctypes.byref(d), x.data_ptr(), x.data_ptr(), None, None,
                                              x.data_ptr(), None, 5)
    assert st == _lib.EINVAL and "current device" in _lib.last_error()
