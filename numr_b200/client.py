"""Host-side mirror of numr's CUDA client for the dense-GEMM ops.

`CudaClient` exposes the methods numr puts on its client for this path, with the same
names, argument meaning and error classes:

    MatmulOps::matmul, matmul_bias                      src/ops/traits/matmul.rs:12,107
    GemmEpilogueOps::matmul_bias_activation / _residual src/ops/traits/gemm_epilogue.rs:66,105
    Fp8MatmulOps::fp8_matmul / fp8_matmul_e5m2          src/ops/traits/fp8_matmul.rs:57,85

Tensors are torch CUDA tensors (torch is used for device memory and streams only); all
validation, shape logic and compute happen in libnumr_b200 through its C ABI. The output
and the workspace are allocated from torch's stream-ordered caching allocator on the
current stream, the same contract numr's `Tensor::empty` + `CudaAllocator` give its
launchers. There is no fallback: without the library or an sm_100 GPU every op raises.
"""
from __future__ import annotations

import contextlib
import ctypes
from enum import IntEnum

import torch

from . import _lib


class GemmActivation(IntEnum):
    """numr::ops::GemmActivation with its `code()` values."""
    NONE = 0
    RELU = 1
    GELU = 2
    SILU = 3
    SIGMOID = 4
    TANH = 5


class NumrError(Exception):
    """Base of the errors this path can raise (numr::error::Error)."""


class InvalidArgument(NumrError):
    pass


class UnsupportedDType(NumrError):
    pass


class Internal(NumrError):
    pass


class ShapeMismatch(NumrError):
    pass


class DTypeMismatch(NumrError):
    pass


_STATUS_ERRORS = {
    _lib.EINVAL: InvalidArgument,
    _lib.EUNSUPPORTED: UnsupportedDType,
    _lib.ECUDA: Internal,
    _lib.EWORKSPACE: Internal,
    _lib.ETIMEOUT: Internal,
    _lib.ESHAPE: ShapeMismatch,
    _lib.EDTYPE: DTypeMismatch,
}

_TORCH_TO_DTYPE = {
    torch.float32: _lib.F32,
    torch.bfloat16: _lib.BF16,
    torch.float16: _lib.F16,
    torch.float8_e4m3fn: _lib.FP8E4M3,
    torch.float8_e5m2: _lib.FP8E5M2,
    torch.int8: _lib.I8,
    torch.int32: _lib.I32,
    torch.int64: _lib.I64,
    torch.int16: _lib.I16,
    torch.uint8: _lib.U8,
    torch.uint16: _lib.U16,
    torch.uint32: _lib.U32,
    torch.uint64: _lib.U64,
}
_DTYPE_TO_TORCH = {v: k for k, v in _TORCH_TO_DTYPE.items()}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _TORCH_TO_DTYPE[dt]
    except KeyError:
        raise UnsupportedDType(f"dtype {dt} is not on the dense-GEMM path") from None


def _check(status: int) -> None:
    if status != _lib.OK:
        raise _STATUS_ERRORS.get(status, Internal)(_lib.last_error())


def _desc(t: torch.Tensor) -> _lib.TensorDesc:
    d = _lib.TensorDesc()
    d.ptr = t.data_ptr()
    d.dtype = dtype_code(t.dtype)
    d.ndim = t.dim()
    if t.dim() > 8:
        raise InvalidArgument("tensors of more than 8 dimensions are not supported")
    for i, (s, st) in enumerate(zip(t.shape, t.stride())):
        d.shape[i] = s
        d.strides[i] = st
    return d


class CudaClient:
    """The op surface of numr's CUDA client for matmul and its fused epilogues.

    f32_mode: "exact" (three TF32 products per term, <= 1e-5 relative Frobenius error) or
    "tf32" (operands rounded to TF32, <= 1e-3); only F32 inputs read it.
    """

    def __init__(self, device: int = 0, f32_mode: str = "exact"):
        self._lib = _lib.load()
        if not torch.cuda.is_available():
            raise Internal("numr_b200 needs a CUDA device (sm_100); there is no CPU path")
        self.device = torch.device("cuda", device)
        self.device_index = device
        if f32_mode not in ("exact", "tf32"):
            raise InvalidArgument("f32_mode must be 'exact' or 'tf32'")
        self.f32_mode = _lib.F32_EXACT if f32_mode == "exact" else _lib.F32_TF32
        self._workspace = None
        self._cache = {}   # shape / workspace answers per operand signature (host-side only)

    # -- plumbing ---------------------------------------------------------------
    def _stream(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _ws(self, nbytes: int):
        """Workspace of at least nbytes from the caching allocator (kept and regrown)."""
        if nbytes == 0:
            return None, 0
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return ctypes.c_void_p(self._workspace.data_ptr()), self._workspace.numel()

    def _guard(self):
        """Makes the client's device current for a call (free when it already is)."""
        if torch.cuda.current_device() == self.device_index:
            return contextlib.nullcontext()
        return torch.cuda.device(self.device)

    def _check_device(self, *tensors) -> None:
        for t in tensors:
            if t is not None and t.device != self.device:
                raise InvalidArgument(f"tensor lives on {t.device}, the client drives {self.device}")

    @staticmethod
    def _sig(t):
        """What the shape / workspace answers depend on for one tensor."""
        return None if t is None else (tuple(t.shape), t.stride(), t.dtype, t.data_ptr() & 15)

    def _out_shape(self, a, b, bias):
        key = ("shape", self._sig(a), self._sig(b), self._sig(bias))
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        hit = self._out_shape_uncached(a, b, bias)
        self._cache[key] = hit
        return hit

    def _out_shape_uncached(self, a, b, bias):
        shape = (ctypes.c_int64 * 8)()
        ndim = ctypes.c_int32()
        dt = ctypes.c_int32()
        da, db = _desc(a), _desc(b)
        dbias = _desc(bias) if bias is not None else None
        _check(self._lib.numr_b200_matmul_out_shape(
            ctypes.byref(da), ctypes.byref(db), ctypes.byref(dbias) if dbias is not None else None,
            shape, ctypes.byref(ndim), ctypes.byref(dt)))
        return tuple(shape[i] for i in range(ndim.value)), dt.value

    def _workspace_for(self, a, b, out_dtype_code, bias=None, residual=None):
        """Workspace for this very call: operand preparation, plus a gather buffer for a bias or
        residual only when that tensor is there and not contiguous."""
        key = ("ws", self._sig(a), self._sig(b), out_dtype_code, self._sig(bias), self._sig(residual))
        n = self._cache.get(key)
        if n is None:
            da, db = _desc(a), _desc(b)
            dbias = _desc(bias) if bias is not None else None
            dres = _desc(residual) if residual is not None else None
            with self._guard():
                n = int(self._lib.numr_b200_op_workspace_bytes_for(
                    ctypes.byref(da), ctypes.byref(db), ctypes.byref(dbias) if dbias is not None else None,
                    ctypes.byref(dres) if dres is not None else None, out_dtype_code, self.f32_mode))
            self._cache[key] = n
        return self._ws(n)

    def synchronize(self) -> None:
        """cuStreamSynchronize on the compute stream (numr client.rs:415-419)."""
        torch.cuda.current_stream(self.device).synchronize()

    def device_status(self) -> int:
        """Device-side status word (0 = every bounded wait completed); synchronises."""
        v = ctypes.c_int(0)
        with self._guard():
            _check(self._lib.numr_b200_device_status(ctypes.byref(v)))
        return v.value

    # -- ops ----------------------------------------------------------------------
    def matmul(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """C = A @ B with NumPy batch broadcasting; I8 x I8 gives I32."""
        self._check_device(a, b)
        if a.dtype != b.dtype:
            raise DTypeMismatch(f"matmul: {a.dtype} vs {b.dtype}")
        shape, out_dt = self._out_shape(a, b, None)
        out = torch.empty(shape, dtype=_DTYPE_TO_TORCH[out_dt], device=self.device)
        ws, ws_bytes = self._workspace_for(a, b, out_dt)
        da, db, do = _desc(a), _desc(b), _desc(out)
        with self._guard():
            _check(self._lib.numr_b200_matmul(ctypes.byref(da), ctypes.byref(db), ctypes.byref(do),
                                              self.f32_mode, ws, ws_bytes, self._stream(), self.device_index))
        return out

    def matmul_bias(self, a, b, bias) -> torch.Tensor:
        """C = A @ B + bias[N]; for I8 operands the bias is I32 and joins the wide accumulator."""
        self._check_device(a, b, bias)
        self._pre_dtype_check("matmul_bias", a, b, bias, epilogue=False)
        shape, out_dt = self._out_shape(a, b, bias)
        out = torch.empty(shape, dtype=_DTYPE_TO_TORCH[out_dt], device=self.device)
        ws, ws_bytes = self._workspace_for(a, b, out_dt, bias)
        da, db, dbias, do = _desc(a), _desc(b), _desc(bias), _desc(out)
        with self._guard():
            _check(self._lib.numr_b200_matmul_bias(ctypes.byref(da), ctypes.byref(db), ctypes.byref(dbias),
                                                   ctypes.byref(do), self.f32_mode, ws, ws_bytes,
                                                   self._stream(), self.device_index))
        return out

    def matmul_bias_activation(self, a, b, bias, activation: GemmActivation) -> torch.Tensor:
        """C = activation(A @ B + bias)."""
        self._check_device(a, b, bias)
        self._pre_dtype_check("matmul_bias_activation", a, b, bias, epilogue=True)
        if bias.dim() != 1:
            raise InvalidArgument(f"bias must be 1D tensor, got shape {tuple(bias.shape)}")
        shape, out_dt = self._out_shape(a, b, bias)
        out = torch.empty(shape, dtype=_DTYPE_TO_TORCH[out_dt], device=self.device)
        ws, ws_bytes = self._workspace_for(a, b, out_dt, bias)
        da, db, dbias, do = _desc(a), _desc(b), _desc(bias), _desc(out)
        with self._guard():
            _check(self._lib.numr_b200_matmul_bias_activation(
                ctypes.byref(da), ctypes.byref(db), ctypes.byref(dbias), int(activation), ctypes.byref(do),
                self.f32_mode, ws, ws_bytes, self._stream(), self.device_index))
        return out

    def matmul_activation(self, a, b, activation: GemmActivation) -> torch.Tensor:
        """C = activation(A @ B): matmul_bias_activation without the bias term (not in numr's trait;
        its grouped GEMM has the same form). Used by the column-sharded MLP projection."""
        self._check_device(a, b)
        if a.dtype == torch.int8:
            raise UnsupportedDType("matmul_activation: I8 is not supported")
        if a.dtype != b.dtype:
            raise DTypeMismatch(f"matmul_activation: {a.dtype} vs {b.dtype}")
        shape, out_dt = self._out_shape(a, b, None)
        out = torch.empty(shape, dtype=_DTYPE_TO_TORCH[out_dt], device=self.device)
        ws, ws_bytes = self._workspace_for(a, b, out_dt)
        da, db, do = _desc(a), _desc(b), _desc(out)
        with self._guard():
            _check(self._lib.numr_b200_matmul_activation(
                ctypes.byref(da), ctypes.byref(db), int(activation), ctypes.byref(do), self.f32_mode, ws,
                ws_bytes, self._stream(), self.device_index))
        return out

    def matmul_bias_residual(self, a, b, bias, residual) -> torch.Tensor:
        """C = A @ B + bias + residual (residual has the output's shape)."""
        self._check_device(a, b, bias, residual)
        self._pre_dtype_check("matmul_bias_residual", a, b, bias, epilogue=True)
        if bias.dim() != 1:
            raise InvalidArgument(f"bias must be 1D tensor, got shape {tuple(bias.shape)}")
        shape, out_dt = self._out_shape(a, b, bias)
        out = torch.empty(shape, dtype=_DTYPE_TO_TORCH[out_dt], device=self.device)
        ws, ws_bytes = self._workspace_for(a, b, out_dt, bias, residual)
        da, db, dbias, dres, do = _desc(a), _desc(b), _desc(bias), _desc(residual), _desc(out)
        with self._guard():
            _check(self._lib.numr_b200_matmul_bias_residual(
                ctypes.byref(da), ctypes.byref(db), ctypes.byref(dbias), ctypes.byref(dres), ctypes.byref(do),
                self.f32_mode, ws, ws_bytes, self._stream(), self.device_index))
        return out

    def fp8_matmul(self, a, b, scale_a: float, scale_b: float, out_dtype: torch.dtype) -> torch.Tensor:
        """out = scale_a * scale_b * (A_e4m3 @ B_e4m3), f32 accumulation, cast to out_dtype."""
        return self._fp8(a, b, scale_a, scale_b, out_dtype, a_e5m2=False)

    def fp8_matmul_e5m2(self, a, b, scale_a: float, scale_b: float, out_dtype: torch.dtype) -> torch.Tensor:
        """out = scale_a * scale_b * (A_e5m2 @ B_e4m3): the backward-pass form."""
        return self._fp8(a, b, scale_a, scale_b, out_dtype, a_e5m2=True)

    def fp8_matmul_fused(self, a, b, scale_a, scale_b, out_dtype, bias=None,
                         activation: GemmActivation = GemmActivation.NONE, residual=None) -> torch.Tensor:
        """out = cast(activation(scale_a*scale_b*(A@B) + bias) + residual); bias and residual carry
        out_dtype. A superset of numr's fp8_matmul (which has no epilogue operands)."""
        self._check_device(a, b, bias, residual)
        shape, _ = self._out_shape(a, b, bias)
        out_code = dtype_code(out_dtype)
        out = torch.empty(shape, dtype=out_dtype, device=self.device)
        ws, ws_bytes = self._workspace_for(a, b, out_code, bias, residual)
        da, db, do = _desc(a), _desc(b), _desc(out)
        dbias = _desc(bias) if bias is not None else None
        dres = _desc(residual) if residual is not None else None
        with self._guard():
            _check(self._lib.numr_b200_fp8_matmul_fused(
                ctypes.byref(da), ctypes.byref(db), float(scale_a), float(scale_b),
                ctypes.byref(dbias) if dbias is not None else None, int(activation),
                ctypes.byref(dres) if dres is not None else None, ctypes.byref(do), ws, ws_bytes,
                self._stream(), self.device_index))
        return out

    def matmul_bias_activation_bwd(self, grad, a, b, bias, activation: GemmActivation):
        """Gradients of activation(a @ b + bias) (numr GemmEpilogueOps::matmul_bias_activation_bwd):
        returns (d_a like a, d_b like b, d_bias [N]). a and grad may carry leading batch dimensions; b is
        2-D (one weight for all batches: d_b sums over them) or carries the same leading dimensions (one
        weight, and one d_b, per batch). Three tensor-core GEMMs: the first recomputes the
        pre-activation and multiplies its derivative into grad in the epilogue."""
        self._check_device(grad, a, b, bias)
        self._pre_dtype_check("matmul_bias_activation_bwd", a, b, bias, epilogue=True)
        if grad.dtype != a.dtype:
            raise DTypeMismatch(f"matmul_bias_activation_bwd: {a.dtype} vs {grad.dtype}")
        if a.dim() < 2 or b.dim() < 2 or grad.dim() != a.dim() or b.dim() not in (2, a.dim()):
            raise InvalidArgument("matmul_bias_activation_bwd: a and grad need the same rank >= 2; b is 2-D or "
                                  "carries a's leading dimensions")
        d_a = torch.empty(tuple(a.shape), dtype=a.dtype, device=self.device)
        d_b = torch.empty(tuple(b.shape), dtype=a.dtype, device=self.device)
        d_bias = torch.empty((b.shape[-1],), dtype=a.dtype, device=self.device)
        dg, da, db, dbias = _desc(grad), _desc(a), _desc(b), _desc(bias)
        key = ("bwd", self._sig(a), self._sig(b))
        n = self._cache.get(key)
        if n is None:
            with self._guard():
                n = int(self._lib.numr_b200_matmul_bias_activation_bwd_workspace_bytes(
                    ctypes.byref(dg), ctypes.byref(da), ctypes.byref(db), ctypes.byref(dbias), self.f32_mode))
            self._cache[key] = n
        ws, ws_bytes = self._ws(n)
        oa, ob, obias = _desc(d_a), _desc(d_b), _desc(d_bias)
        with self._guard():
            _check(self._lib.numr_b200_matmul_bias_activation_bwd(
                ctypes.byref(dg), ctypes.byref(da), ctypes.byref(db), ctypes.byref(dbias), int(activation),
                ctypes.byref(oa), ctypes.byref(ob), ctypes.byref(obias), self.f32_mode, ws, ws_bytes,
                self._stream(), self.device_index))
        return d_a, d_b, d_bias

    def grouped_matmul(self, a, b, group_offsets) -> torch.Tensor:
        """c[offsets[g]:offsets[g+1]] = a[offsets[g]:offsets[g+1]] @ b[g] with the offsets on the device
        (numr GroupedMatmulOps::grouped_matmul): a [rows, k], b [groups, k, n], group_offsets int32
        [groups + 1]. Nothing is read back to the host."""
        return self.grouped_matmul_activation(a, b, group_offsets, GemmActivation.NONE)

    def grouped_matmul_activation(self, a, b, group_offsets, activation: GemmActivation) -> torch.Tensor:
        """Grouped matmul with the activation fused into the epilogue (numr grouped_matmul_activation)."""
        self._check_device(a, b, group_offsets)
        if a.dim() != 2:
            raise InvalidArgument(f"a: expected 2-D [total_rows, k], got {a.dim()}-D")
        if b.dim() != 3:
            raise InvalidArgument(f"b: expected 3-D [num_groups, k, n], got {b.dim()}-D")
        out = torch.empty((a.shape[0], b.shape[2]), dtype=a.dtype, device=self.device)
        key = ("gws", self._sig(a), self._sig(b))
        n = self._cache.get(key)
        da, db, dofs, do = _desc(a), _desc(b), _desc(group_offsets), _desc(out)
        if n is None:
            with self._guard():
                n = int(self._lib.numr_b200_grouped_matmul_workspace_bytes(ctypes.byref(da), ctypes.byref(db),
                                                                           self.f32_mode))
            self._cache[key] = n
        ws, ws_bytes = self._ws(n)
        with self._guard():
            _check(self._lib.numr_b200_grouped_matmul(ctypes.byref(da), ctypes.byref(db), ctypes.byref(dofs),
                                                      int(activation), ctypes.byref(do), self.f32_mode, ws, ws_bytes,
                                                      self._stream(), self.device_index))
        return out

    def matmul_activation_allgather(self, a, b, activation: GemmActivation, gathered, bias=None) -> torch.Tensor:
        """activation(a @ b (+ bias)) for this rank's column block of a column-sharded GEMM, with the
        all-gather fused into the epilogue: every finished tile is stored into column block `rank` of
        EVERY rank's row-major `[M, world * N]` buffer (`gathered`, a sharding.GatheredOutput) over
        NVLink. a [M, K] and b [K, N] (or the transposed view of a contiguous [N, K]) are 2-D; N * element
        size must be a multiple of 16. Returns this rank's buffer (complete once every rank's kernel
        has finished: `gathered.barrier()` orders that on the stream)."""
        self._check_device(a, b, bias)
        if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
            raise ShapeMismatch(f"matmul_activation_allgather: a {tuple(a.shape)} vs b {tuple(b.shape)}")
        if a.dtype != b.dtype or (bias is not None and bias.dtype != a.dtype):
            raise DTypeMismatch(f"matmul_activation_allgather: {a.dtype} vs {b.dtype}")
        m, k = a.shape
        n = b.shape[1]
        out = gathered.tensor
        if tuple(out.shape) != (m, n * gathered.world) or out.dtype != a.dtype:
            raise ShapeMismatch(f"matmul_activation_allgather: the gathered buffer is {tuple(out.shape)} {out.dtype}, "
                                f"expected {(m, n * gathered.world)} {a.dtype}")
        a = a.contiguous()
        if b.is_contiguous():
            layout = _lib.B_KN
        elif b.t().is_contiguous():
            layout = _lib.B_NK
        else:
            b, layout = b.contiguous(), _lib.B_KN
        d = _lib.GemmDesc()
        d.a_dtype = d.b_dtype = d.out_dtype = d.bias_dtype = dtype_code(a.dtype)
        d.batch = d.a_batch = d.b_batch = 1
        d.m, d.n, d.k = m, n, k
        d.b_layout, d.activation, d.f32_mode = layout, int(activation), self.f32_mode
        d.scale_a = d.scale_b = 1.0
        ptrs = (ctypes.c_uint64 * gathered.world)(*gathered.ptrs)
        with self._guard():
            need = int(self._lib.numr_b200_gemm_workspace_bytes(ctypes.byref(d), a.data_ptr(), b.data_ptr()))
            ws, ws_bytes = self._ws(need)
            _check(self._lib.numr_b200_gemm_allgather(
                ctypes.byref(d), a.data_ptr(), b.data_ptr(), bias.data_ptr() if bias is not None else None, None,
                ptrs, gathered.world, gathered.rank, ws, ws_bytes, self._stream(), self.device_index))
        return out

    # -- convolutions as GEMM ----------------------------------------------------------
    def _conv(self, kind, entry, x, weight, bias, c_out, geom, out_shape_of):
        self._check_device(x, weight, bias)
        if x.dtype != weight.dtype or (bias is not None and bias.dtype != x.dtype):
            raise DTypeMismatch(f"conv: input {x.dtype}, weight {weight.dtype}, bias {None if bias is None else bias.dtype}")
        if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise UnsupportedDType(f"conv as GEMM: dtype {x.dtype} (F32, F16 or BF16 expected)")
        if bias is not None and (bias.dim() != 1 or bias.shape[0] != c_out):
            raise InvalidArgument(f"conv: bias must have {c_out} elements, got shape {tuple(bias.shape)}")
        x, weight = x.contiguous(), weight.contiguous()
        bias = bias.contiguous() if bias is not None else None
        d = _lib.ConvDesc()
        d.dtype = dtype_code(x.dtype)
        d.groups = 1
        d.f32_mode = self.f32_mode
        d.c_out = c_out
        for k, v in geom.items():
            setattr(d, k, v)
        oh, ow = ctypes.c_uint32(), ctypes.c_uint32()
        _check(self._lib.numr_b200_conv_out_shape(ctypes.byref(d), kind, ctypes.byref(oh), ctypes.byref(ow)))
        out = torch.empty(out_shape_of(oh.value, ow.value), dtype=x.dtype, device=self.device)
        with self._guard():
            n = int(self._lib.numr_b200_conv_workspace_bytes(ctypes.byref(d), kind, weight.data_ptr()))
            ws, ws_bytes = self._ws(n)
            _check(entry(ctypes.byref(d), x.data_ptr(), weight.data_ptr(),
                         bias.data_ptr() if bias is not None else None, out.data_ptr(), ws, ws_bytes,
                         self._stream(), self.device_index))
        return out

    def conv1d(self, x, weight, bias=None, stride=1, padding=(0, 0), dilation=1, groups=1) -> torch.Tensor:
        """ConvOps::conv1d through the im2col + GEMM path (src/ops/cuda/conv1d_im2col.rs:100): x [N, C_in, L],
        weight [C_out, C_in, K], padding = resolved (left, right); groups must be 1."""
        if groups != 1:
            raise UnsupportedDType("conv as GEMM: groups != 1 stays on the direct kernel")
        if x.dim() != 3 or weight.dim() != 3 or weight.shape[1] != x.shape[1]:
            raise ShapeMismatch(f"conv1d: input {tuple(x.shape)} vs weight {tuple(weight.shape)}")
        n, c_in, length = x.shape
        geom = dict(batch=n, c_in=c_in, in_h=1, in_w=length, kernel_h=1, kernel_w=weight.shape[2], stride_h=1,
                    stride_w=stride, pad_top=0, pad_bottom=0, pad_left=padding[0], pad_right=padding[1],
                    dilation_h=1, dilation_w=dilation, output_padding=0)
        return self._conv(_lib.CONV1D, self._lib.numr_b200_conv1d, x, weight, bias, weight.shape[0], geom,
                          lambda oh, ow: (n, weight.shape[0], ow))

    def conv2d(self, x, weight, bias=None, stride=(1, 1), padding=(0, 0, 0, 0), dilation=(1, 1), groups=1):
        """ConvOps::conv2d through the im2col + GEMM path (src/ops/cuda/conv2d_im2col.rs:104): x [N, C_in, H, W],
        weight [C_out, C_in, Kh, Kw], padding = resolved (top, bottom, left, right); groups must be 1."""
        if groups != 1:
            raise UnsupportedDType("conv as GEMM: groups != 1 stays on the direct kernel")
        if x.dim() != 4 or weight.dim() != 4 or weight.shape[1] != x.shape[1]:
            raise ShapeMismatch(f"conv2d: input {tuple(x.shape)} vs weight {tuple(weight.shape)}")
        n, c_in, h, w = x.shape
        geom = dict(batch=n, c_in=c_in, in_h=h, in_w=w, kernel_h=weight.shape[2], kernel_w=weight.shape[3],
                    stride_h=stride[0], stride_w=stride[1], pad_top=padding[0], pad_bottom=padding[1],
                    pad_left=padding[2], pad_right=padding[3], dilation_h=dilation[0], dilation_w=dilation[1],
                    output_padding=0)
        return self._conv(_lib.CONV2D, self._lib.numr_b200_conv2d, x, weight, bias, weight.shape[0], geom,
                          lambda oh, ow: (n, weight.shape[0], oh, ow))

    def conv_transpose1d(self, x, weight, bias=None, stride=1, padding=(0, 0), output_padding=0, dilation=1,
                         groups=1) -> torch.Tensor:
        """ConvOps::conv_transpose1d through the gather + GEMM path (src/ops/cuda/conv_transpose1d_gemm.rs:108):
        x [N, C_in, L], weight [C_in, C_out, K], padding = resolved (left, right); groups must be 1."""
        if groups != 1:
            raise UnsupportedDType("conv as GEMM: groups != 1 stays on the direct kernel")
        if x.dim() != 3 or weight.dim() != 3 or weight.shape[0] != x.shape[1]:
            raise ShapeMismatch(f"conv_transpose1d: input {tuple(x.shape)} vs weight {tuple(weight.shape)}")
        n, c_in, length = x.shape
        geom = dict(batch=n, c_in=c_in, in_h=1, in_w=length, kernel_h=1, kernel_w=weight.shape[2], stride_h=1,
                    stride_w=stride, pad_top=0, pad_bottom=0, pad_left=padding[0], pad_right=padding[1],
                    dilation_h=1, dilation_w=dilation, output_padding=output_padding)
        return self._conv(_lib.CONV_TRANSPOSE1D, self._lib.numr_b200_conv_transpose1d, x, weight, bias,
                          weight.shape[1], geom, lambda oh, ow: (n, weight.shape[1], ow))

    # -- helpers ------------------------------------------------------------------
    def _fp8(self, a, b, scale_a, scale_b, out_dtype, a_e5m2):
        self._check_device(a, b)
        shape, _ = self._out_shape(a, b, None)
        if out_dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise UnsupportedDType(f"fp8_matmul: output dtype {out_dtype} (F32, F16 or BF16 expected)")
        out_code = dtype_code(out_dtype)
        out = torch.empty(shape, dtype=out_dtype, device=self.device)
        ws, ws_bytes = self._workspace_for(a, b, out_code)
        da, db, do = _desc(a), _desc(b), _desc(out)
        with self._guard():
            _check(self._lib.numr_b200_fp8_matmul(ctypes.byref(da), ctypes.byref(db), float(scale_a),
                                                  float(scale_b), int(a_e5m2), ctypes.byref(do), ws, ws_bytes,
                                                  self._stream(), self.device_index))
        return out

    @staticmethod
    def _pre_dtype_check(op, a, b, bias, epilogue):
        """validate_matmul_bias_dtypes / validate_gemm_epilogue_dtypes (src/ops/matmul_dtype.rs:44-100);
        done here too so the error surfaces before the output is allocated."""
        if epilogue and a.dtype == torch.int8:
            raise UnsupportedDType(f"{op}: I8 is not supported")
        if a.dtype != b.dtype:
            raise DTypeMismatch(f"{op}: {a.dtype} vs {b.dtype}")
        want = torch.int32 if a.dtype == torch.int8 else a.dtype
        if bias.dtype != want:
            if a.dtype == torch.int8:
                raise InvalidArgument(f"{op} on I8 operands accumulates into I32, so the bias must be I32, "
                                      f"got {bias.dtype}")
            raise DTypeMismatch(f"{op}: {a.dtype} vs bias {bias.dtype}")
