//! Blackwell (sm_100a) back end of numr's dense-GEMM launchers: the Rust side of libnumr_b200.
//!
//! NOT COMPILED in this repository (its build image has no Rust toolchain); written against
//! numr 0.7.0 and `include/numr_b200.h`, to be dropped in as `src/runtime/cuda/kernels/b200.rs`.
//! Every `pub unsafe fn` below keeps the name, argument order and `Result<()>` of the numr launcher
//! it stands in for; the existing launchers call it first and fall through to their own body when
//! it returns `Ok(false)` (not a Blackwell device, or a dtype this library does not serve):
//!
//! ```ignore
//! // loader/matmul.rs:64, first lines of launch_matmul_kernel
//! if b200::launch_matmul_kernel(context, stream, device_index, dtype, a_ptr, b_ptr, c_ptr, m, n, k)? {
//!     return Ok(());
//! }
//! ```
//!
//! Contract with the library: the caller's context is current on this thread (numr binds it,
//! client.rs:128-131), `device_index` names that device, everything is enqueued on `stream` and
//! nothing synchronises or allocates inside the library. The workspace some problems need (F32
//! operand parts, re-pitched copies of misaligned operands, partial sums of a K cut) is allocated
//! here, stream-ordered, and freed stream-ordered right after the launch is enqueued.
#![allow(clippy::too_many_arguments)]

use std::ffi::{c_void, CStr};
use std::os::raw::{c_char, c_int};
use std::sync::Arc;

use cudarc::driver::{CudaContext, CudaStream};

use crate::dtype::DType;
use crate::error::{Error, Result};
use crate::ops::GemmActivation;

// ------------------------------------------------------------------------------------------------
// C ABI (include/numr_b200.h), one declaration per exported symbol
// ------------------------------------------------------------------------------------------------

/// `numr_b200_gemm_desc`
#[repr(C)]
#[derive(Clone, Copy)]
pub struct GemmDesc {
    pub a_dtype: i32,
    pub b_dtype: i32,
    pub out_dtype: i32,
    pub bias_dtype: i32,
    pub batch: u32,
    pub m: u32,
    pub n: u32,
    pub k: u32,
    pub a_batch: u32,
    pub b_batch: u32,
    pub b_layout: i32,   // 0: B is [K,N] (the launchers' contract), 1: B is [N,K] (transposed view, read in place)
    pub activation: i32, // GemmActivation::code(); + 16 for the backward epilogue
    pub f32_mode: i32,   // 0 exact (three TF32 products), 1 TF32
    pub scale_a: f32,
    pub scale_b: f32,
}

/// `numr_b200_tensor`
#[repr(C)]
#[derive(Clone, Copy)]
pub struct TensorDesc {
    pub ptr: u64,
    pub dtype: i32,
    pub ndim: i32,
    pub shape: [i64; 8],
    pub strides: [i64; 8], // in elements
}

type Stream = *mut c_void;
type Ws = *mut c_void;
type T = *const TensorDesc;

#[link(name = "numr_b200", kind = "static")]
extern "C" {
    pub fn numr_b200_version() -> *const c_char;
    pub fn numr_b200_last_error() -> *const c_char;
    pub fn numr_b200_init(device_index: c_int) -> c_int;
    pub fn numr_b200_reload_tuning();
    pub fn numr_b200_device_status(kernel_status: *mut c_int) -> c_int;

    pub fn numr_b200_gemm_workspace_bytes(desc: *const GemmDesc, a: *const c_void, b: *const c_void) -> usize;
    pub fn numr_b200_gemm(desc: *const GemmDesc, a: *const c_void, b: *const c_void, bias: *const c_void,
        residual: *const c_void, c: *mut c_void, ws: Ws, ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_static_scratch_bytes() -> usize;
    pub fn numr_b200_gemm_static_scratch(desc: *const GemmDesc, a: *const c_void, b: *const c_void,
        bias: *const c_void, residual: *const c_void, c: *mut c_void, stream: Stream, device: c_int) -> c_int;

    pub fn numr_b200_launch_matmul_kernel(stream: Stream, device: c_int, dtype: i32, a: u64, b: u64, c: u64,
        m: usize, n: usize, k: usize, ws: Ws, ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_matmul_batched_kernel(stream: Stream, device: c_int, dtype: i32, a: u64, b: u64,
        c: u64, batch: usize, m: usize, n: usize, k: usize, a_batch: usize, b_batch: usize, ws: Ws,
        ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_matmul_bias_kernel(stream: Stream, device: c_int, dtype: i32, a: u64, b: u64,
        bias: u64, c: u64, m: usize, n: usize, k: usize, ws: Ws, ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_matmul_bias_batched_kernel(stream: Stream, device: c_int, dtype: i32, a: u64,
        b: u64, bias: u64, c: u64, batch: usize, m: usize, n: usize, k: usize, a_batch: usize, b_batch: usize,
        ws: Ws, ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_gemm_bias_act_kernel(stream: Stream, device: c_int, dtype: i32, a: u64, b: u64,
        bias: u64, c: u64, m: usize, n: usize, k: usize, activation: i32, ws: Ws, ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_gemm_bias_act_batched_kernel(stream: Stream, device: c_int, dtype: i32, a: u64,
        b: u64, bias: u64, c: u64, batch: usize, m: usize, n: usize, k: usize, activation: i32, ws: Ws,
        ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_gemm_bias_residual_kernel(stream: Stream, device: c_int, dtype: i32, a: u64,
        b: u64, bias: u64, residual: u64, c: u64, m: usize, n: usize, k: usize, ws: Ws, ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_gemm_bias_residual_batched_kernel(stream: Stream, device: c_int, dtype: i32,
        a: u64, b: u64, bias: u64, residual: u64, c: u64, batch: usize, m: usize, n: usize, k: usize, ws: Ws,
        ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_fp8_matmul_e4m3(stream: Stream, device: c_int, out_dtype: i32, a: u64, b: u64,
        out: u64, scale_a: f32, scale_b: f32, batch: usize, m: usize, n: usize, k: usize, ws: Ws,
        ws_bytes: usize) -> c_int;
    pub fn numr_b200_launch_fp8_matmul_e5m2(stream: Stream, device: c_int, out_dtype: i32, a: u64, b: u64,
        out: u64, scale_a: f32, scale_b: f32, batch: usize, m: usize, n: usize, k: usize, ws: Ws,
        ws_bytes: usize) -> c_int;

    pub fn numr_b200_matmul_out_shape(a: T, b: T, bias: T, out_shape: *mut i64, out_ndim: *mut i32,
        out_dtype: *mut i32) -> c_int;
    pub fn numr_b200_op_workspace_bytes(a: T, b: T, out_dtype: i32, f32_mode: i32) -> usize;
    pub fn numr_b200_op_workspace_bytes_for(a: T, b: T, bias: T, residual: T, out_dtype: i32, f32_mode: i32) -> usize;
    pub fn numr_b200_matmul(a: T, b: T, out: T, f32_mode: i32, ws: Ws, ws_bytes: usize, stream: Stream,
        device: c_int) -> c_int;
    pub fn numr_b200_matmul_bias(a: T, b: T, bias: T, out: T, f32_mode: i32, ws: Ws, ws_bytes: usize,
        stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_matmul_bias_activation(a: T, b: T, bias: T, activation: i32, out: T, f32_mode: i32, ws: Ws,
        ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_matmul_activation(a: T, b: T, activation: i32, out: T, f32_mode: i32, ws: Ws,
        ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_matmul_bias_residual(a: T, b: T, bias: T, residual: T, out: T, f32_mode: i32, ws: Ws,
        ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_fp8_matmul(a: T, b: T, scale_a: f32, scale_b: f32, a_e5m2: i32, out: T, ws: Ws,
        ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_fp8_matmul_fused(a: T, b: T, scale_a: f32, scale_b: f32, bias: T, activation: i32,
        residual: T, out: T, ws: Ws, ws_bytes: usize, stream: Stream, device: c_int) -> c_int;

    pub fn numr_b200_grouped_gemm_workspace_bytes(desc: *const GemmDesc, groups: u32, a: *const c_void,
        b: *const c_void) -> usize;
    pub fn numr_b200_grouped_gemm(desc: *const GemmDesc, groups: u32, a: *const c_void, b: *const c_void,
        group_offsets: *const i32, c: *mut c_void, ws: Ws, ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_grouped_matmul_workspace_bytes(a: T, b: T, f32_mode: i32) -> usize;
    pub fn numr_b200_grouped_matmul(a: T, b: T, group_offsets: T, activation: i32, out: T, f32_mode: i32, ws: Ws,
        ws_bytes: usize, stream: Stream, device: c_int) -> c_int;

    pub fn numr_b200_matmul_bias_activation_bwd_workspace_bytes(grad: T, a: T, b: T, bias: T, f32_mode: i32) -> usize;
    pub fn numr_b200_matmul_bias_activation_bwd(grad: T, a: T, b: T, bias: T, activation: i32, d_a: T, d_b: T,
        d_bias: T, f32_mode: i32, ws: Ws, ws_bytes: usize, stream: Stream, device: c_int) -> c_int;

    pub fn numr_b200_conv_out_shape(desc: *const ConvDesc, kind: i32, out_h: *mut u32, out_w: *mut u32) -> c_int;
    pub fn numr_b200_conv_workspace_bytes(desc: *const ConvDesc, kind: i32, weight: *const c_void) -> usize;
    pub fn numr_b200_conv1d(desc: *const ConvDesc, input: *const c_void, weight: *const c_void,
        bias: *const c_void, out: *mut c_void, ws: Ws, ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_conv2d(desc: *const ConvDesc, input: *const c_void, weight: *const c_void,
        bias: *const c_void, out: *mut c_void, ws: Ws, ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
    pub fn numr_b200_conv_transpose1d(desc: *const ConvDesc, input: *const c_void, weight: *const c_void,
        bias: *const c_void, out: *mut c_void, ws: Ws, ws_bytes: usize, stream: Stream, device: c_int) -> c_int;
}

/// `numr_b200_conv_kind`
pub const CONV1D: i32 = 0;
pub const CONV2D: i32 = 1;
pub const CONV_TRANSPOSE1D: i32 = 2;

/// `numr_b200_conv_desc`: the im2col + GEMM convolutions (conv1d_im2col.rs, conv2d_im2col.rs,
/// conv_transpose1d_gemm.rs). The 1-D forms use the `_w` fields and leave the `_h` fields neutral
/// (in_h = kernel_h = stride_h = dilation_h = 1, pad_top = pad_bottom = 0). Field order and types are
/// those of the C struct.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct ConvDesc {
    pub dtype: i32,
    pub batch: u32,
    pub c_in: u32,
    pub c_out: u32,
    pub groups: u32, // must be 1 (numr keeps grouped convolutions on its direct kernels)
    pub in_h: u32,   // 1 for the 1-D forms
    pub in_w: u32,   // length for the 1-D forms
    pub kernel_h: u32,
    pub kernel_w: u32,
    pub stride_h: u32,
    pub stride_w: u32,
    pub pad_top: u32,
    pub pad_bottom: u32,
    pub pad_left: u32,
    pub pad_right: u32,
    pub dilation_h: u32,
    pub dilation_w: u32,
    pub output_padding: u32, // conv_transpose1d only
    pub f32_mode: i32,
}

// ------------------------------------------------------------------------------------------------
// helpers
// ------------------------------------------------------------------------------------------------

/// `numr_b200_dtype` code of a numr dtype, or None for the dtypes that stay on numr's own kernels.
pub fn dtype_code(d: DType) -> Option<i32> {
    Some(match d {
        DType::F32 => 0,
        DType::BF16 => 1,
        DType::F16 => 2,
        DType::FP8E4M3 => 3,
        DType::FP8E5M2 => 4,
        DType::I8 => 5,
        DType::I32 => 6,
        DType::I64 => 7,
        DType::I16 => 8,
        DType::U8 => 9,
        DType::U16 => 10,
        DType::U32 => 11,
        DType::U64 => 12,
        _ => return None, // F64, Bool, complex
    })
}

/// True when `device_index` is an sm_100 device (the library has no kernels for anything else).
/// numr caches the device profile per index (device.rs:184-191); this reads it.
fn on_blackwell(device_index: usize) -> bool {
    crate::runtime::cuda::device::profile(device_index)
        .map(|p| p.compute_capability_major == 10)
        .unwrap_or(false)
}

fn status_to_result(st: c_int, dtype: DType, op: &'static str) -> Result<()> {
    if st == 0 {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(numr_b200_last_error()) }.to_string_lossy().into_owned();
    Err(match st {
        1 => Error::InvalidArgument { arg: "gemm", reason: msg },
        2 => Error::UnsupportedDType { dtype, op },
        6 => Error::ShapeMismatch { expected: vec![], got: vec![] },
        7 => Error::DTypeMismatch { lhs: dtype, rhs: dtype },
        _ => Error::Internal(msg), // 3 ECUDA, 4 EWORKSPACE, 5 ETIMEOUT
    })
}

/// A stream-ordered scratch buffer that lives until the stream has passed the launch: allocated with
/// the stream's pool right before the launch, freed (stream-ordered) right after it is enqueued.
struct Workspace {
    ptr: u64,
    bytes: usize,
    stream: Stream,
}

impl Workspace {
    fn new(stream: &CudaStream, bytes: usize) -> Result<Self> {
        let raw = stream.cu_stream() as Stream;
        if bytes == 0 {
            return Ok(Self { ptr: 0, bytes: 0, stream: raw });
        }
        // cuMemAllocAsync: 256-byte aligned, usable by work enqueued on `stream` after this call
        let ptr = unsafe { cudarc::driver::result::malloc_async(stream.cu_stream(), bytes) }
            .map_err(|e| Error::Internal(format!("b200 workspace of {bytes} bytes: {e}")))?;
        Ok(Self { ptr, bytes, stream: raw })
    }
    fn ptr(&self) -> Ws {
        self.ptr as Ws
    }
}

impl Drop for Workspace {
    fn drop(&mut self) {
        if self.ptr != 0 {
            // stream-ordered: the memory is released only after the GEMM that uses it
            unsafe {
                let _ = cudarc::driver::result::free_async(self.ptr, self.stream as _);
            }
        }
    }
}

fn plain_desc(dtype: i32, batch: usize, m: usize, n: usize, k: usize, a_batch: usize, b_batch: usize) -> GemmDesc {
    let out = if dtype == 5 { 6 } else { dtype }; // I8 x I8 -> I32
    GemmDesc {
        a_dtype: dtype, b_dtype: dtype, out_dtype: out, bias_dtype: out,
        batch: batch as u32, m: m as u32, n: n as u32, k: k as u32, a_batch: a_batch as u32, b_batch: b_batch as u32,
        b_layout: 0, activation: 0, f32_mode: 0, scale_a: 1.0, scale_b: 1.0,
    }
}

/// Workspace for a launcher-level call (contiguous operands at the given addresses).
fn launcher_workspace(stream: &CudaStream, desc: &GemmDesc, a: u64, b: u64) -> Result<Workspace> {
    let bytes = unsafe { numr_b200_gemm_workspace_bytes(desc, a as *const c_void, b as *const c_void) };
    Workspace::new(stream, bytes)
}

macro_rules! guard {
    ($device_index:expr, $dtype:expr) => {{
        if !on_blackwell($device_index) {
            return Ok(false);
        }
        match dtype_code($dtype) {
            Some(c) => c,
            None => return Ok(false),
        }
    }};
}

// ------------------------------------------------------------------------------------------------
// launcher bodies: same names and argument order as the numr launchers; Ok(true) = launched here
// ------------------------------------------------------------------------------------------------

/// loader/matmul.rs:64
pub unsafe fn launch_matmul_kernel(_ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    dtype: DType, a_ptr: u64, b_ptr: u64, c_ptr: u64, m: usize, n: usize, k: usize) -> Result<bool> {
    let code = guard!(device_index, dtype);
    let ws = launcher_workspace(stream, &plain_desc(code, 1, m, n, k, 1, 1), a_ptr, b_ptr)?;
    let st = numr_b200_launch_matmul_kernel(stream.cu_stream() as Stream, device_index as c_int, code, a_ptr,
        b_ptr, c_ptr, m, n, k, ws.ptr(), ws.bytes);
    status_to_result(st, dtype, "matmul").map(|_| true)
}

/// loader/matmul.rs:284
pub unsafe fn launch_matmul_batched_kernel(_ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    dtype: DType, a_ptr: u64, b_ptr: u64, c_ptr: u64, batch: usize, m: usize, n: usize, k: usize,
    a_batch: usize, b_batch: usize) -> Result<bool> {
    let code = guard!(device_index, dtype);
    let ws = launcher_workspace(stream, &plain_desc(code, batch, m, n, k, a_batch, b_batch), a_ptr, b_ptr)?;
    let st = numr_b200_launch_matmul_batched_kernel(stream.cu_stream() as Stream, device_index as c_int, code,
        a_ptr, b_ptr, c_ptr, batch, m, n, k, a_batch, b_batch, ws.ptr(), ws.bytes);
    status_to_result(st, dtype, "matmul").map(|_| true)
}

/// loader/matmul_bias.rs:46
pub unsafe fn launch_matmul_bias_kernel(_ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    dtype: DType, a_ptr: u64, b_ptr: u64, bias_ptr: u64, c_ptr: u64, m: usize, n: usize, k: usize) -> Result<bool> {
    let code = guard!(device_index, dtype);
    let ws = launcher_workspace(stream, &plain_desc(code, 1, m, n, k, 1, 1), a_ptr, b_ptr)?;
    let st = numr_b200_launch_matmul_bias_kernel(stream.cu_stream() as Stream, device_index as c_int, code, a_ptr,
        b_ptr, bias_ptr, c_ptr, m, n, k, ws.ptr(), ws.bytes);
    status_to_result(st, dtype, "matmul_bias").map(|_| true)
}

/// loader/matmul_bias.rs:254
pub unsafe fn launch_matmul_bias_batched_kernel(_ctx: &Arc<CudaContext>, stream: &CudaStream,
    device_index: usize, dtype: DType, a_ptr: u64, b_ptr: u64, bias_ptr: u64, c_ptr: u64, batch: usize, m: usize,
    n: usize, k: usize, a_batch: usize, b_batch: usize) -> Result<bool> {
    let code = guard!(device_index, dtype);
    let ws = launcher_workspace(stream, &plain_desc(code, batch, m, n, k, a_batch, b_batch), a_ptr, b_ptr)?;
    let st = numr_b200_launch_matmul_bias_batched_kernel(stream.cu_stream() as Stream, device_index as c_int,
        code, a_ptr, b_ptr, bias_ptr, c_ptr, batch, m, n, k, a_batch, b_batch, ws.ptr(), ws.bytes);
    status_to_result(st, dtype, "matmul_bias").map(|_| true)
}

/// kernels/gemm_epilogue/launcher.rs:35
pub unsafe fn launch_gemm_bias_act_kernel(ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    dtype: DType, a_ptr: u64, b_ptr: u64, bias_ptr: u64, c_ptr: u64, m: usize, n: usize, k: usize,
    activation: GemmActivation) -> Result<bool> {
    launch_gemm_bias_act_batched_kernel(ctx, stream, device_index, dtype, a_ptr, b_ptr, bias_ptr, c_ptr, 1, m, n,
        k, activation)
}

/// kernels/gemm_epilogue/launcher.rs:153 (A, B and C advance one full matrix per batch)
pub unsafe fn launch_gemm_bias_act_batched_kernel(_ctx: &Arc<CudaContext>, stream: &CudaStream,
    device_index: usize, dtype: DType, a_ptr: u64, b_ptr: u64, bias_ptr: u64, c_ptr: u64, batch: usize, m: usize,
    n: usize, k: usize, activation: GemmActivation) -> Result<bool> {
    let code = guard!(device_index, dtype);
    let ws = launcher_workspace(stream, &plain_desc(code, batch, m, n, k, batch, batch), a_ptr, b_ptr)?;
    let st = numr_b200_launch_gemm_bias_act_batched_kernel(stream.cu_stream() as Stream, device_index as c_int,
        code, a_ptr, b_ptr, bias_ptr, c_ptr, batch, m, n, k, activation.code() as i32, ws.ptr(), ws.bytes);
    status_to_result(st, dtype, "matmul_bias_activation").map(|_| true)
}

/// kernels/gemm_epilogue/launcher.rs:278
pub unsafe fn launch_gemm_bias_residual_kernel(ctx: &Arc<CudaContext>, stream: &CudaStream,
    device_index: usize, dtype: DType, a_ptr: u64, b_ptr: u64, bias_ptr: u64, residual_ptr: u64, c_ptr: u64,
    m: usize, n: usize, k: usize) -> Result<bool> {
    launch_gemm_bias_residual_batched_kernel(ctx, stream, device_index, dtype, a_ptr, b_ptr, bias_ptr,
        residual_ptr, c_ptr, 1, m, n, k)
}

/// kernels/gemm_epilogue/launcher.rs:398
pub unsafe fn launch_gemm_bias_residual_batched_kernel(_ctx: &Arc<CudaContext>, stream: &CudaStream,
    device_index: usize, dtype: DType, a_ptr: u64, b_ptr: u64, bias_ptr: u64, residual_ptr: u64, c_ptr: u64,
    batch: usize, m: usize, n: usize, k: usize) -> Result<bool> {
    let code = guard!(device_index, dtype);
    let ws = launcher_workspace(stream, &plain_desc(code, batch, m, n, k, batch, batch), a_ptr, b_ptr)?;
    let st = numr_b200_launch_gemm_bias_residual_batched_kernel(stream.cu_stream() as Stream,
        device_index as c_int, code, a_ptr, b_ptr, bias_ptr, residual_ptr, c_ptr, batch, m, n, k, ws.ptr(), ws.bytes);
    status_to_result(st, dtype, "matmul_bias_residual").map(|_| true)
}

unsafe fn fp8(stream: &CudaStream, device_index: usize, e5m2: bool, out_dtype: DType, a: u64, b: u64, c: u64,
    scale_a: f32, scale_b: f32, batch: usize, m: usize, n: usize, k: usize) -> Result<bool> {
    let out = guard!(device_index, out_dtype);
    // aligned FP8 operands need no workspace; a misaligned address (a sliced view) does
    let mut d = plain_desc(3, batch, m, n, k, batch, batch);
    d.a_dtype = if e5m2 { 4 } else { 3 };
    d.out_dtype = out;
    d.bias_dtype = out;
    let ws = launcher_workspace(stream, &d, a, b)?;
    let s = stream.cu_stream() as Stream;
    let st = if e5m2 {
        numr_b200_launch_fp8_matmul_e5m2(s, device_index as c_int, out, a, b, c, scale_a, scale_b, batch, m, n, k,
            ws.ptr(), ws.bytes)
    } else {
        numr_b200_launch_fp8_matmul_e4m3(s, device_index as c_int, out, a, b, c, scale_a, scale_b, batch, m, n, k,
            ws.ptr(), ws.bytes)
    };
    status_to_result(st, out_dtype, "fp8_matmul").map(|_| true)
}

/// kernels/fp8_matmul.rs:51
pub unsafe fn launch_fp8_matmul_e4m3(_ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    out_dtype: DType, a_ptr: u64, b_ptr: u64, c_ptr: u64, scale_a: f32, scale_b: f32, m: usize, n: usize,
    k: usize) -> Result<bool> {
    fp8(stream, device_index, false, out_dtype, a_ptr, b_ptr, c_ptr, scale_a, scale_b, 1, m, n, k)
}

/// kernels/fp8_matmul.rs:101
pub unsafe fn launch_fp8_matmul_e5m2(_ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    out_dtype: DType, a_ptr: u64, b_ptr: u64, c_ptr: u64, scale_a: f32, scale_b: f32, m: usize, n: usize,
    k: usize) -> Result<bool> {
    fp8(stream, device_index, true, out_dtype, a_ptr, b_ptr, c_ptr, scale_a, scale_b, 1, m, n, k)
}

/// kernels/fp8_matmul.rs:151
pub unsafe fn launch_fp8_matmul_e4m3_batched(_ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    out_dtype: DType, a_ptr: u64, b_ptr: u64, c_ptr: u64, scale_a: f32, scale_b: f32, batch: usize, m: usize,
    n: usize, k: usize) -> Result<bool> {
    fp8(stream, device_index, false, out_dtype, a_ptr, b_ptr, c_ptr, scale_a, scale_b, batch, m, n, k)
}

/// kernels/fp8_matmul.rs:204
pub unsafe fn launch_fp8_matmul_e5m2_batched(_ctx: &Arc<CudaContext>, stream: &CudaStream, device_index: usize,
    out_dtype: DType, a_ptr: u64, b_ptr: u64, c_ptr: u64, scale_a: f32, scale_b: f32, batch: usize, m: usize,
    n: usize, k: usize) -> Result<bool> {
    fp8(stream, device_index, true, out_dtype, a_ptr, b_ptr, c_ptr, scale_a, scale_b, batch, m, n, k)
}

/// The transposed-B fast path above the launchers (helpers/matmul.rs:66-92): instead of materialising
/// a `[N,K]` weight viewed as `[K,N]` with a strided copy, or routing small M to the gemv kernels, pass
/// the weight as it lies. `w_ptr` is the contiguous `[b_batch, N, K]` buffer behind the view.
pub unsafe fn launch_matmul_transposed_b(stream: &CudaStream, device_index: usize, dtype: DType, a_ptr: u64,
    w_ptr: u64, c_ptr: u64, batch: usize, m: usize, n: usize, k: usize, a_batch: usize, b_batch: usize)
    -> Result<bool> {
    let code = guard!(device_index, dtype);
    let mut d = plain_desc(code, batch, m, n, k, a_batch, b_batch);
    d.b_layout = 1;
    let ws = launcher_workspace(stream, &d, a_ptr, w_ptr)?;
    let st = numr_b200_gemm(&d, a_ptr as *const c_void, w_ptr as *const c_void, std::ptr::null(),
        std::ptr::null(), c_ptr as *mut c_void, ws.ptr(), ws.bytes, stream.cu_stream() as Stream,
        device_index as c_int);
    status_to_result(st, dtype, "matmul").map(|_| true)
}

/// Once per device, before the first stream capture (numr's graph capture, runtime.rs:427-513):
/// the library's first-use set-up calls runtime functions that are not legal while capturing.
pub fn init_device(device_index: usize) -> Result<()> {
    if !on_blackwell(device_index) {
        return Ok(());
    }
    status_to_result(unsafe { numr_b200_init(device_index as c_int) }, DType::F32, "init")
}
