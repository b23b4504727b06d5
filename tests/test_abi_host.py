"""CPU-only checks of the C ABI: the library loads without a GPU driver, exports every
symbol include/numr_b200.h declares, and rejects bad arguments with the reference's error
classes before anything would be launched. No compute call is made here.
"""
import ctypes
import re
from pathlib import Path

import pytest

from numr_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "numr_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(numr_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(nb_lib):
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(nb_lib, name), f"{name} is declared in the header but not exported"
    # and the binding knows every one of them
    assert sorted(_lib.SIGNATURES) == declared


def test_version_and_error_text(nb_lib):
    assert b"sm_100a" in nb_lib.numr_b200_version()
    assert isinstance(_lib.last_error(), str)


def _desc(**kw):
    d = _lib.GemmDesc()
    base = dict(a_dtype=_lib.BF16, b_dtype=_lib.BF16, out_dtype=_lib.BF16, bias_dtype=_lib.BF16, batch=1,
                m=128, n=128, k=128, a_batch=1, b_batch=1, b_layout=_lib.B_KN, activation=0, f32_mode=0,
                scale_a=1.0, scale_b=1.0)
    base.update(kw)
    for k, v in base.items():
        setattr(d, k, v)
    return d


def _gemm(nb_lib, d, a=256, b=512, bias=None, res=None, c=1024, ws=None, ws_bytes=0):
    return nb_lib.numr_b200_gemm(ctypes.byref(d), a, b, bias, res, c, ws, ws_bytes, None, 0)


@pytest.mark.parametrize("kw,status,needle", [
    (dict(a_dtype=_lib.BF16, b_dtype=_lib.F16), _lib.EDTYPE, "mismatch"),
    (dict(a_dtype=99, b_dtype=99, out_dtype=99), _lib.EUNSUPPORTED, "dtype"),
    (dict(a_dtype=_lib.I32, b_dtype=_lib.I64, out_dtype=_lib.I32), _lib.EDTYPE, "mismatch"),
    (dict(a_dtype=_lib.I64, b_dtype=_lib.I64, out_dtype=_lib.I32), _lib.EDTYPE, "I64"),
    (dict(a_dtype=_lib.U32, b_dtype=_lib.U32, out_dtype=_lib.U32, activation=1), _lib.EUNSUPPORTED, "U32"),
    (dict(out_dtype=_lib.F32), _lib.EDTYPE, "BF16"),
    (dict(b_layout=7), _lib.EINVAL, "b_layout"),
    (dict(activation=9), _lib.EINVAL, "activation"),
    (dict(a_batch=3), _lib.EINVAL, "batch"),
    (dict(a_dtype=_lib.I8, b_dtype=_lib.I8, out_dtype=_lib.I32, activation=1), _lib.EUNSUPPORTED, "I8"),
    (dict(a_dtype=_lib.I8, b_dtype=_lib.I8, out_dtype=_lib.I8), _lib.EDTYPE, "I32"),
    (dict(a_dtype=_lib.F32, b_dtype=_lib.F32, out_dtype=_lib.F32, f32_mode=5), _lib.EINVAL, "f32_mode"),
    (dict(a_dtype=_lib.FP8E4M3, b_dtype=_lib.FP8E5M2, out_dtype=_lib.F32), _lib.EDTYPE, "mismatch"),
    (dict(a_dtype=_lib.FP8E4M3, b_dtype=_lib.FP8E4M3, out_dtype=_lib.I32), _lib.EUNSUPPORTED, "output dtype"),
])
def test_descriptor_validation(nb_lib, kw, status, needle):
    assert _gemm(nb_lib, _desc(**kw)) == status
    assert needle in _lib.last_error()


def test_pointer_and_workspace_validation(nb_lib):
    assert nb_lib.numr_b200_gemm(None, 256, 512, None, None, 1024, None, 0, None, 0) == _lib.EINVAL
    assert _gemm(nb_lib, _desc(), c=None) == _lib.EINVAL                      # NULL output
    assert _gemm(nb_lib, _desc(), c=1025) == _lib.EINVAL                      # misaligned output
    assert _gemm(nb_lib, _desc(bias_dtype=_lib.F32), bias=64) == _lib.EDTYPE   # bias dtype differs from output
    d8 = _desc(a_dtype=_lib.I8, b_dtype=_lib.I8, out_dtype=_lib.I32, bias_dtype=_lib.I32)
    assert _gemm(nb_lib, d8, res=2048) == _lib.EUNSUPPORTED                    # I8 + residual
    # Empty outputs are a no-op, as the reference's callers return before launching.
    assert _gemm(nb_lib, _desc(m=0)) == _lib.OK
    assert _gemm(nb_lib, _desc(batch=0)) == _lib.OK


def test_workspace_query(nb_lib):
    q = nb_lib.numr_b200_gemm_workspace_bytes
    assert q(ctypes.byref(_desc()), 256, 512) == 0                                   # aligned bf16: in place
    assert q(ctypes.byref(_desc()), 258, 512) >= 128 * 128 * 2                       # misaligned A: re-pitched copy
    assert q(ctypes.byref(_desc(k=100)), 256, 512) >= 128 * 104 * 2                  # K*2 not a multiple of 16
    f32 = _desc(a_dtype=_lib.F32, b_dtype=_lib.F32, out_dtype=_lib.F32, f32_mode=_lib.F32_EXACT)
    exact = q(ctypes.byref(f32), None, None)
    f32.f32_mode = _lib.F32_TF32
    tf32 = q(ctypes.byref(f32), None, None)
    assert tf32 == 2 * 128 * 128 * 4 and exact == 2 * tf32                           # hi (+ lo) parts of A and B
    assert q(ctypes.byref(_desc(k=0)), 256, 512) == 0


def _tensor(shape, dtype, strides=None, ptr=4096):
    d = _lib.TensorDesc()
    d.ptr = ptr
    d.dtype = dtype
    d.ndim = len(shape)
    if strides is None:
        strides, acc = [], 1
        for s in reversed(shape):
            strides.insert(0, acc)
            acc *= s
    for i, (s, t) in enumerate(zip(shape, strides)):
        d.shape[i] = s
        d.strides[i] = t
    return d


def test_op_layer_errors_match_reference_classes(nb_lib):
    """Error classes of src/ops/cuda/matmul.rs, gemm_epilogue.rs, fp8_matmul.rs and
    src/ops/matmul_dtype.rs, raised before any launch (pointers here are never dereferenced)."""
    B = ctypes.byref
    a = _tensor([4, 8], _lib.F32)
    b = _tensor([8, 6], _lib.F32)
    out = _tensor([4, 6], _lib.F32)
    bad_b = _tensor([7, 6], _lib.F32)
    assert nb_lib.numr_b200_matmul(B(a), B(bad_b), B(out), 0, None, 0, None, 0) == _lib.ESHAPE
    b16 = _tensor([8, 6], _lib.BF16)
    assert nb_lib.numr_b200_matmul(B(a), B(b16), B(out), 0, None, 0, None, 0) == _lib.EDTYPE
    # batch dims that do not broadcast
    a3 = _tensor([2, 4, 8], _lib.F32)
    b3 = _tensor([3, 8, 6], _lib.F32)
    assert nb_lib.numr_b200_matmul(B(a3), B(b3), B(out), 0, None, 0, None, 0) == _lib.ESHAPE
    # bias rules
    bias_ok = _tensor([6], _lib.F32)
    bias_2d = _tensor([1, 6], _lib.F32)
    bias_len = _tensor([5], _lib.F32)
    bias_dt = _tensor([6], _lib.BF16)
    f = nb_lib.numr_b200_matmul_bias_activation
    assert f(B(a), B(b), B(bias_2d), 1, B(out), 0, None, 0, None, 0) == _lib.EINVAL
    assert "1-D" in _lib.last_error()
    assert f(B(a), B(b), B(bias_len), 1, B(out), 0, None, 0, None, 0) == _lib.ESHAPE
    assert f(B(a), B(b), B(bias_dt), 1, B(out), 0, None, 0, None, 0) == _lib.EDTYPE
    assert f(B(a), B(b), B(bias_ok), 17, B(out), 0, None, 0, None, 0) == _lib.EINVAL
    # I8: epilogue ops reject it; matmul_bias wants an I32 bias (InvalidArgument, naming I32)
    a8, b8 = _tensor([4, 8], _lib.I8), _tensor([8, 6], _lib.I8)
    out32 = _tensor([4, 6], _lib.I32)
    bias8, bias32 = _tensor([6], _lib.I8), _tensor([6], _lib.I32)
    assert f(B(a8), B(b8), B(bias32), 1, B(out32), 0, None, 0, None, 0) == _lib.EUNSUPPORTED
    assert nb_lib.numr_b200_matmul_bias(B(a8), B(b8), B(bias8), B(out32), 0, None, 0, None, 0) == _lib.EINVAL
    assert "I32" in _lib.last_error()
    # output tensor must match the op's shape and dtype
    wrong_out = _tensor([4, 7], _lib.F32)
    assert nb_lib.numr_b200_matmul(B(a), B(b), B(wrong_out), 0, None, 0, None, 0) == _lib.ESHAPE
    out_bf = _tensor([4, 6], _lib.BF16)
    assert nb_lib.numr_b200_matmul(B(a), B(b), B(out_bf), 0, None, 0, None, 0) == _lib.EDTYPE
    # residual must have the output's shape
    res_bad = _tensor([4, 5], _lib.F32)
    g = nb_lib.numr_b200_matmul_bias_residual
    assert g(B(a), B(b), B(bias_ok), B(res_bad), B(out), 0, None, 0, None, 0) == _lib.ESHAPE
    # fp8_matmul dtype rules
    a_f8, b_f8 = _tensor([4, 8], _lib.FP8E4M3), _tensor([8, 6], _lib.FP8E4M3)
    h = nb_lib.numr_b200_fp8_matmul
    assert h(B(a), B(b_f8), 1.0, 1.0, 0, B(out), None, 0, None, 0) == _lib.EDTYPE
    assert h(B(a_f8), B(b_f8), 1.0, 1.0, 1, B(out), None, 0, None, 0) == _lib.EDTYPE          # e5m2 form wants E5M2 A
    out_i = _tensor([4, 6], _lib.I32)
    assert h(B(a_f8), B(b_f8), 1.0, 1.0, 0, B(out_i), None, 0, None, 0) == _lib.EUNSUPPORTED
    # empty outputs return OK without touching the device
    a0 = _tensor([0, 8], _lib.F32)
    out0 = _tensor([0, 6], _lib.F32)
    assert nb_lib.numr_b200_matmul(B(a0), B(b), B(out0), 0, None, 0, None, 0) == _lib.OK


def test_op_workspace_accounts_for_views(nb_lib):
    B = ctypes.byref
    a = _tensor([64, 128], _lib.BF16)
    b = _tensor([128, 96], _lib.BF16)
    base = nb_lib.numr_b200_op_workspace_bytes(B(a), B(b), _lib.BF16, 0)
    # transposed-B view ([K,N] with strides [1,K]) is read in place: no extra bytes
    bt = _tensor([128, 96], _lib.BF16, strides=[1, 128])
    assert nb_lib.numr_b200_op_workspace_bytes(B(a), B(bt), _lib.BF16, 0) == base
    # a column-sliced A (row stride 256) has to be gathered
    a_view = _tensor([64, 128], _lib.BF16, strides=[256, 1])
    assert nb_lib.numr_b200_op_workspace_bytes(B(a_view), B(b), _lib.BF16, 0) >= base + 64 * 128 * 2
    # middle-dimension broadcast cannot be expressed as bi % count: B is expanded
    a4 = _tensor([2, 4, 64, 128], _lib.BF16)
    b4 = _tensor([2, 1, 128, 96], _lib.BF16)
    need = nb_lib.numr_b200_op_workspace_bytes(B(a4), B(b4), _lib.BF16, 0)
    assert need >= 8 * 128 * 96 * 2


def test_grouped_matmul_validation(nb_lib):
    """validate_grouped (src/ops/cpu/grouped_matmul.rs:13-75), raised before any launch."""
    B = ctypes.byref
    f = nb_lib.numr_b200_grouped_matmul
    a, b = _tensor([8, 32], _lib.F32), _tensor([2, 32, 16], _lib.F32)
    off, out = _tensor([3], _lib.I32), _tensor([8, 16], _lib.F32)
    call = lambda a_, b_, o_, out_, act=0: f(B(a_), B(b_), B(o_), act, B(out_), 0, None, 0, None, 0)
    assert call(_tensor([2, 4, 32], _lib.F32), b, off, out) == _lib.EINVAL and "2-D" in _lib.last_error()
    assert call(a, _tensor([32, 16], _lib.F32), off, out) == _lib.EINVAL and "3-D" in _lib.last_error()
    assert call(a, b, _tensor([3], _lib.I64), out) == _lib.EINVAL and "I32" in _lib.last_error()
    assert call(a, b, _tensor([2], _lib.I32), out) == _lib.EINVAL and "3 entries" in _lib.last_error()
    assert call(a, _tensor([2, 32, 16], _lib.BF16), off, out) == _lib.EINVAL
    assert call(_tensor([8, 32], _lib.I8), _tensor([2, 32, 16], _lib.I8), off, _tensor([8, 16], _lib.I32)) == _lib.EINVAL
    assert "F32/F16/BF16" in _lib.last_error()
    assert call(a, _tensor([2, 31, 16], _lib.F32), off, out) == _lib.ESHAPE
    assert call(a, b, off, _tensor([8, 17], _lib.F32)) == _lib.ESHAPE
    assert call(a, b, off, out, act=9) == _lib.EINVAL
    # workspace is needed (the tile plan lives there) and checked before anything is launched
    assert call(a, b, off, out) in (_lib.EWORKSPACE, _lib.ECUDA)
    d = _desc(a_dtype=_lib.F32, b_dtype=_lib.F32, out_dtype=_lib.F32, m=8, n=16, k=32, batch=1, a_batch=1, b_batch=2)
    assert nb_lib.numr_b200_grouped_gemm_workspace_bytes(ctypes.byref(d), 2, None, None) >= (1 + 2) * 16
    d.batch = 2
    assert nb_lib.numr_b200_grouped_gemm(ctypes.byref(d), 2, 256, 512, 768, 1024, None, 0, None, 0) == _lib.EINVAL


def test_matmul_bias_activation_bwd_validation(nb_lib):
    """Error classes of matmul_bias_activation_bwd (src/ops/cpu/gemm_epilogue.rs:261-281), before any launch."""
    B = ctypes.byref
    f = nb_lib.numr_b200_matmul_bias_activation_bwd
    grad, a, b, bias = _tensor([4, 6], _lib.F32), _tensor([4, 8], _lib.F32), _tensor([8, 6], _lib.F32), _tensor([6], _lib.F32)
    d_a, d_b, d_bias = _tensor([4, 8], _lib.F32), _tensor([8, 6], _lib.F32), _tensor([6], _lib.F32)
    call = lambda g=grad, a_=a, b_=b, bi=bias, act=1, oa=d_a, ob=d_b, obi=d_bias: \
        f(B(g), B(a_), B(b_), B(bi), act, B(oa), B(ob), B(obi), 0, None, 0, None, 0)
    assert call(g=_tensor([4, 6], _lib.BF16)) == _lib.EDTYPE
    assert call(a_=_tensor([4, 8], _lib.I8), b_=_tensor([8, 6], _lib.I8), bi=_tensor([6], _lib.I32)) == _lib.EUNSUPPORTED
    assert call(bi=_tensor([6], _lib.BF16)) == _lib.EDTYPE
    assert call(b_=_tensor([7, 6], _lib.F32)) == _lib.ESHAPE
    assert call(g=_tensor([4, 5], _lib.F32)) == _lib.ESHAPE
    assert call(bi=_tensor([1, 6], _lib.F32)) == _lib.EINVAL
    assert call(act=7) == _lib.EINVAL
    assert call(a_=_tensor([2, 2, 8], _lib.F32)) == _lib.EUNSUPPORTED
    assert call(oa=_tensor([4, 7], _lib.F32)) == _lib.ESHAPE
    assert call() == _lib.EWORKSPACE                       # grad_pre and a^T live in the workspace
    q = nb_lib.numr_b200_matmul_bias_activation_bwd_workspace_bytes
    assert q(B(grad), B(a), B(b), B(bias), 0) >= 4 * 6 * 4 + 8 * 4 * 4
    # the descriptor-level backward epilogue needs the incoming gradient in the residual slot
    d = _desc(activation=1 + 16)
    assert _gemm(nb_lib, d, res=None) in (_lib.EINVAL, _lib.ECUDA)
