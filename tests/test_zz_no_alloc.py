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
