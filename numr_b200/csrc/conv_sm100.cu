// Convolutions as GEMM on the tcgen05 kernel: conv1d, conv2d (groups = 1) and conv_transpose1d.
//
// numr's CUDA back end turns these into "gather the receptive fields into a column buffer, then one
// batched matmul" (src/ops/cuda/conv1d_im2col.rs:100-157, conv2d_im2col.rs:104-158,
// conv_transpose1d_gemm.rs:108-162; gather kernels src/runtime/cuda/kernels/im2col.cu, im2col2d.cu,
// col_transpose1d.cu). The same formulation here:
//   col[n]   [C_in*Kh*Kw, L_out]   gathered from the input (zero where a tap falls into the padding)
//   out[n]   [C_out, L_out]      = W [C_out, C_in*Kh*Kw] @ col[n]  + bias[C_out] (one value per ROW)
// with three differences that follow from the GEMM kernel underneath:
//   * the column buffer's rows are padded to 16 bytes so TMA can read it in place (the GEMM reads an
//     [K, N] operand directly: no transpose, as in the reference);
//   * for F32 the gather writes the TF32 parts (high, and low in exact mode) the tensor cores consume,
//     so the column buffer is never re-read for a split pass;
//   * the bias is added in the GEMM's epilogue (a per-row bias) instead of by a broadcast add
//     afterwards (conv1d_im2col.rs:147-156).
// The weight is used in place when it is a TMA-readable [C_out, contraction] matrix; otherwise one
// small kernel re-pitches it, splits it (F32) or swaps its leading axes (conv_transpose1d's weight is
// [C_in, C_out, K], conv_transpose1d_gemm.rs:141-149).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstring>

#include "gemm_internal.h"

namespace nb {
namespace {

constexpr int kThreads = 256;

struct ConvGeom {
  uint32_t batch, c_in, in_h, in_w, kh, kw, out_h, out_w;
  uint32_t stride_h, stride_w, pad_top, pad_left, dil_h, dil_w;
  uint32_t transposed;   // 1: conv_transpose1d gather (1-D: the _h fields are neutral)
  uint32_t ld;           // row pitch of the column buffer in elements
};

__device__ __forceinline__ float round_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// High TF32 part of x: round to nearest, except that a finite x within half a TF32 ulp of FLT_MAX,
// which would round to infinity, is truncated instead (its low part then carries the rest), so a
// product the reference's F32 kernels keep finite stays finite.
__device__ __forceinline__ float tf32_high(float x) {
  const float h = round_tf32(x);
  return (isinf(h) && isfinite(x)) ? __uint_as_float(__float_as_uint(x) & 0xFFFFE000u) : h;
}

// One thread per column-buffer element, consecutive threads on consecutive output positions.
// Forward: row r = (ic, ky, kx) meets input (ic, oy*stride_h + ky*dil_h - pad_top, ox*stride_w + kx*dil_w - pad_left).
// Transposed 1-D: output position ot and tap k are fed by input l = (ot + pad_left - k*dil) / stride when
// that is a non-negative multiple of the stride inside the input (col_transpose1d.cu:25-45,
// src/runtime/cpu/kernels/conv_transpose.rs:85-98).
template <typename T, bool F32_PARTS>
__global__ void conv_gather_kernel(const T* __restrict__ in, T* __restrict__ col, T* __restrict__ col_lo, ConvGeom g) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMM after this may begin its set-up
  const uint32_t spatial = g.out_h * g.out_w;
  const uint32_t rows = g.c_in * g.kh * g.kw;
  const size_t total = (size_t)g.batch * rows * g.ld;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t p = (uint32_t)(i % g.ld);
    const size_t rn = i / g.ld;
    const uint32_t r = (uint32_t)(rn % rows);
    const uint32_t n = (uint32_t)(rn / rows);
    T v = T(0.0f);
    if (p < spatial) {
      const uint32_t kx = r % g.kw;
      const uint32_t ky = (r / g.kw) % g.kh;
      const uint32_t ic = r / (g.kw * g.kh);
      const uint32_t oy = p / g.out_w, ox = p - oy * g.out_w;
      if (!g.transposed) {
        const int iy = (int)(oy * g.stride_h + ky * g.dil_h) - (int)g.pad_top;
        const int ix = (int)(ox * g.stride_w + kx * g.dil_w) - (int)g.pad_left;
        if (iy >= 0 && iy < (int)g.in_h && ix >= 0 && ix < (int)g.in_w)
          v = in[(((size_t)n * g.c_in + ic) * g.in_h + iy) * g.in_w + ix];
      } else {
        const int num = (int)ox + (int)g.pad_left - (int)(kx * g.dil_w);
        if (num >= 0 && (uint32_t)num % g.stride_w == 0) {
          const uint32_t l = (uint32_t)num / g.stride_w;
          if (l < g.in_w) v = in[((size_t)n * g.c_in + ic) * g.in_w + l];
        }
      }
    }
    if constexpr (F32_PARTS) {
      const float x = v;
      const float h = tf32_high(x);
      col[i] = h;
      if (col_lo) col_lo[i] = (isfinite(x) && isfinite(h)) ? round_tf32(x - h) : 0.0f;
    } else {
      col[i] = v;
    }
  }
}

// W' [c_out, ld] from the weight: forward weights are [c_out, contraction] already (a re-pitch and/or
// TF32 split); a transposed convolution's weight is [c_in, c_out, k] and row r = ic*k + kx of W'[oc]
// is weight[ic][oc][kx].
template <typename T, bool F32_PARTS>
__global__ void conv_weight_kernel(const T* __restrict__ w, T* __restrict__ out, T* __restrict__ out_lo,
                                   uint32_t c_out, uint32_t contraction, uint32_t k, uint32_t ld, uint32_t transposed) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t total = (size_t)c_out * ld;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t r = (uint32_t)(i % ld);
    const uint32_t oc = (uint32_t)(i / ld);
    T v = T(0.0f);
    if (r < contraction) {
      if (!transposed) v = w[(size_t)oc * contraction + r];
      else v = w[((size_t)(r / k) * c_out + oc) * k + (r % k)];
    }
    if constexpr (F32_PARTS) {
      const float x = v;
      const float h = tf32_high(x);
      out[i] = h;
      if (out_lo) out_lo[i] = (isfinite(x) && isfinite(h)) ? round_tf32(x - h) : 0.0f;
    } else {
      out[i] = v;
    }
  }
}

inline uint32_t grid_for(size_t work) {
  size_t blocks = (work + kThreads - 1) / kThreads;
  blocks = std::min<size_t>(blocks, 148 * 8);   // grid-stride beyond that
  return (uint32_t)std::max<size_t>(blocks, 1);
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

uint32_t out_size(uint32_t in, uint32_t k, uint32_t stride, uint32_t dil, uint32_t pad_a, uint32_t pad_b) {
  // compute_output_size (src/ops/conv_common.rs:146-161)
  const uint64_t eff = (uint64_t)dil * (k - 1) + 1, padded = (uint64_t)in + pad_a + pad_b;
  return padded < eff ? 0u : (uint32_t)((padded - eff) / stride + 1);
}

uint32_t transpose_out_size(uint32_t in, uint32_t k, uint32_t stride, uint32_t dil, uint32_t pad_a, uint32_t pad_b,
                            uint32_t output_padding) {
  // compute_transpose_output_size (src/ops/conv_transpose_common.rs:52-67)
  if (in == 0) return 0;
  const uint64_t grown = (uint64_t)(in - 1) * stride + (uint64_t)dil * (k - 1) + 1 + output_padding;
  const uint64_t pads = (uint64_t)pad_a + pad_b;
  return grown > pads ? (uint32_t)(grown - pads) : 0u;
}

struct ConvPlan {
  ConvGeom g;
  uint32_t elt, c_out, contraction, spatial, lda;
  bool f32, exact, weight_prep;
  size_t off_w, w_bytes, off_col, col_bytes, off_split, split_bytes, total;
};

enum ConvKind { CONV1D = 0, CONV2D = 1, CONV_T1D = 2 };

int make_conv_plan(const numr_b200_conv_desc* d, int kind, const void* weight, ConvPlan* p, int device) {
  if (!d) return fail(NUMR_B200_EINVAL, "conv descriptor is NULL");
  switch (d->dtype) {
    case NUMR_B200_F32: p->elt = 4; break;
    case NUMR_B200_BF16: case NUMR_B200_F16: p->elt = 2; break;
    default:
      return fail(NUMR_B200_EUNSUPPORTED, "conv as GEMM: dtype %d (F32, F16 or BF16 expected)", d->dtype);
  }
  if (d->groups != 1)
    return fail(NUMR_B200_EUNSUPPORTED, "conv as GEMM: groups = %u stays on the direct kernel (groups must be 1)", d->groups);
  if (d->stride_h == 0 || d->stride_w == 0 || d->dilation_h == 0 || d->dilation_w == 0 || d->kernel_h == 0 || d->kernel_w == 0)
    return fail(NUMR_B200_EINVAL, "conv: stride, dilation and kernel extents must be at least 1");
  if (kind != CONV2D && (d->in_h != 1 || d->kernel_h != 1 || d->stride_h != 1 || d->dilation_h != 1 || d->pad_top || d->pad_bottom))
    return fail(NUMR_B200_EINVAL, "conv1d / conv_transpose1d: the height fields must be neutral (in_h = kernel_h = stride_h = dilation_h = 1, no vertical padding)");
  if (kind != CONV_T1D && d->output_padding)
    return fail(NUMR_B200_EINVAL, "output_padding belongs to conv_transpose1d only");
  if (d->f32_mode != NUMR_B200_F32_EXACT && d->f32_mode != NUMR_B200_F32_TF32)
    return fail(NUMR_B200_EINVAL, "f32_mode %d is not 0 (exact) or 1 (tf32)", d->f32_mode);
  ConvGeom& g = p->g;
  memset(&g, 0, sizeof(g));
  g.batch = d->batch; g.c_in = d->c_in; g.in_h = d->in_h; g.in_w = d->in_w; g.kh = d->kernel_h; g.kw = d->kernel_w;
  g.stride_h = d->stride_h; g.stride_w = d->stride_w; g.pad_top = d->pad_top; g.pad_left = d->pad_left;
  g.dil_h = d->dilation_h; g.dil_w = d->dilation_w;
  g.transposed = kind == CONV_T1D ? 1u : 0u;
  if (kind == CONV_T1D) {
    g.out_h = 1;
    g.out_w = transpose_out_size(d->in_w, d->kernel_w, d->stride_w, d->dilation_w, d->pad_left, d->pad_right, d->output_padding);
  } else {
    g.out_h = out_size(d->in_h, d->kernel_h, d->stride_h, d->dilation_h, d->pad_top, d->pad_bottom);
    g.out_w = out_size(d->in_w, d->kernel_w, d->stride_w, d->dilation_w, d->pad_left, d->pad_right);
  }
  const uint64_t contraction = (uint64_t)d->c_in * d->kernel_h * d->kernel_w;
  const uint64_t spatial = (uint64_t)g.out_h * g.out_w;
  if (contraction > 0x7FFFFFFFull || spatial > 0x7FFFFFFFull)
    return fail(NUMR_B200_EINVAL, "conv: contraction or output extent exceeds 2^31-1");
  p->c_out = d->c_out;
  p->contraction = (uint32_t)contraction;
  p->spatial = (uint32_t)spatial;
  p->f32 = d->dtype == NUMR_B200_F32;
  p->exact = p->f32 && d->f32_mode == NUMR_B200_F32_EXACT;
  const uint32_t per16 = 16 / p->elt;
  g.ld = (uint32_t)align_up(p->spatial, per16);
  const uint32_t parts = p->exact ? 2u : 1u;
  // The weight is read in place when TMA can: forward layout, 16-byte aligned base and row pitch, not F32.
  const bool aligned = (reinterpret_cast<uintptr_t>(weight) & 15) == 0 && p->contraction % per16 == 0;
  p->weight_prep = p->f32 || kind == CONV_T1D || !aligned;
  p->lda = p->weight_prep ? (uint32_t)align_up(p->contraction, per16) : p->contraction;
  size_t off = 0;
  p->off_w = off;
  p->w_bytes = p->weight_prep ? (size_t)parts * d->c_out * p->lda * p->elt : 0;
  off = align_up(off + p->w_bytes, 256);
  p->off_col = off;
  p->col_bytes = (size_t)parts * d->batch * p->contraction * g.ld * p->elt;
  off = align_up(off + p->col_bytes, 256);
  p->off_split = off;
  p->split_bytes = 0;
  if (device >= 0 && d->batch && d->c_out && p->spatial && p->contraction) {
    GemmLaunch gl;
    memset(&gl, 0, sizeof(gl));
    gl.kind = p->f32 ? 1 : 0;
    gl.out_kind = p->f32 ? OUT_F32 : (d->dtype == NUMR_B200_BF16 ? OUT_BF16 : OUT_F16);
    gl.elt_bytes = p->elt;
    gl.a_lo = p->exact ? reinterpret_cast<const void*>(1) : nullptr;
    gl.b_layout = NUMR_B200_B_KN;
    gl.batch = d->batch; gl.a_batch = 1; gl.b_batch = d->batch;
    gl.m = d->c_out; gl.n = p->spatial; gl.k = p->contraction;
    gl.device_index = device;
    p->split_bytes = gemm_split_workspace_bytes(gl);
    off = align_up(off + p->split_bytes, 256);
  }
  p->total = off;
  return NUMR_B200_OK;
}

template <typename T>
cudaError_t launch_gather(const ConvPlan& p, const void* in, char* col, cudaStream_t stream) {
  const size_t total = (size_t)p.g.batch * p.contraction * p.g.ld;
  conv_gather_kernel<T, false><<<grid_for(total), kThreads, 0, stream>>>(static_cast<const T*>(in),
                                                                        reinterpret_cast<T*>(col), nullptr, p.g);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_weight(const ConvPlan& p, const void* w, char* out, uint32_t k, cudaStream_t stream) {
  conv_weight_kernel<T, false><<<grid_for((size_t)p.c_out * p.lda), kThreads, 0, stream>>>(
      static_cast<const T*>(w), reinterpret_cast<T*>(out), nullptr, p.c_out, p.contraction, k, p.lda, p.g.transposed);
  return cudaGetLastError();
}

int run_conv(const numr_b200_conv_desc* d, int kind, const void* input, const void* weight, const void* bias,
             void* out, void* ws, size_t ws_bytes, void* cu_stream, int device_index) {
  int dev = 0;
  {
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) {
      cudaGetLastError();
      cur = -1;
    }
    if (cur >= 0 && device_index >= 0 && device_index != cur)
      return fail(NUMR_B200_EINVAL, "device_index %d is not the calling thread's current device (%d): make it current first",
                  device_index, cur);
    dev = cur;
  }
  ConvPlan p;
  int st = make_conv_plan(d, kind, weight, &p, dev);
  if (st != NUMR_B200_OK) return st;
  if (d->batch == 0 || d->c_out == 0 || p.spatial == 0) return NUMR_B200_OK;   // empty output
  if (p.contraction == 0) return fail(NUMR_B200_EINVAL, "conv: c_in is 0");
  if (!input || !weight || !out) return fail(NUMR_B200_EINVAL, "conv: input, weight or output pointer is NULL");
  if ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(bias)) % p.elt)
    return fail(NUMR_B200_EINVAL, "conv: a pointer is not aligned to its element size %u", p.elt);
  if (dev < 0) return fail(NUMR_B200_ECUDA, "no CUDA device is available; this library has no CPU path");
  const size_t required = p.off_split;   // the K-split scratch behind it is optional
  if (!ws || ws_bytes < required)
    return fail(NUMR_B200_EWORKSPACE, "conv: workspace of %zu bytes needed, %zu given", required, ws ? ws_bytes : (size_t)0);
  if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(NUMR_B200_EWORKSPACE, "conv: workspace %p is not 256-byte aligned", ws);
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  char* w = static_cast<char*>(ws);
  const uint32_t parts = p.exact ? 2u : 1u;
  (void)parts;

  // column buffer (and, for F32, its TF32 parts)
  char* col = w + p.off_col;
  cudaError_t e;
  const size_t col_part = (size_t)d->batch * p.contraction * p.g.ld * p.elt;
  if (p.f32) {
    float* lo = p.exact ? reinterpret_cast<float*>(col + col_part) : nullptr;
    conv_gather_kernel<float, true><<<grid_for(col_part / 4), kThreads, 0, stream>>>(
        static_cast<const float*>(input), reinterpret_cast<float*>(col), lo, p.g);
    e = cudaGetLastError();
  } else if (d->dtype == NUMR_B200_BF16) {
    e = launch_gather<__nv_bfloat16>(p, input, col, stream);
  } else {
    e = launch_gather<__half>(p, input, col, stream);
  }
  if (e != cudaSuccess) return fail(NUMR_B200_ECUDA, "conv gather kernel launch failed: %s", cudaGetErrorString(e));

  // weight as the GEMM's A operand
  const void* a_ptr = weight;
  const void* a_lo = nullptr;
  if (p.weight_prep) {
    char* wp = w + p.off_w;
    const size_t w_part = (size_t)d->c_out * p.lda * p.elt;
    const uint32_t k = d->kernel_w;   // (only read for the transposed, 1-D, layout)
    if (p.f32) {
      float* lo = p.exact ? reinterpret_cast<float*>(wp + w_part) : nullptr;
      conv_weight_kernel<float, true><<<grid_for(w_part / 4), kThreads, 0, stream>>>(
          static_cast<const float*>(weight), reinterpret_cast<float*>(wp), lo, p.c_out, p.contraction, k, p.lda, p.g.transposed);
      e = cudaGetLastError();
      a_lo = lo;
    } else if (d->dtype == NUMR_B200_BF16) {
      e = launch_weight<__nv_bfloat16>(p, weight, wp, k, stream);
    } else {
      e = launch_weight<__half>(p, weight, wp, k, stream);
    }
    if (e != cudaSuccess) return fail(NUMR_B200_ECUDA, "conv weight kernel launch failed: %s", cudaGetErrorString(e));
    a_ptr = wp;
  }

  GemmLaunch g;
  memset(&g, 0, sizeof(g));
  g.kind = p.f32 ? 1 : 0;                                   // TF32 / F16 MMA kind
  g.out_kind = p.f32 ? OUT_F32 : (d->dtype == NUMR_B200_BF16 ? OUT_BF16 : OUT_F16);
  g.elt_bytes = p.elt;
  g.a_fmt = g.b_fmt = p.f32 ? 2u : (d->dtype == NUMR_B200_BF16 ? 1u : 0u);
  g.a = a_ptr; g.lda = p.lda; g.a_lo = a_lo;
  g.b = col; g.ldb = p.g.ld; g.b_lo = p.exact ? col + col_part : nullptr;
  g.b_layout = NUMR_B200_B_KN;
  g.batch = d->batch; g.a_batch = 1; g.b_batch = d->batch;
  g.m = d->c_out; g.n = p.spatial; g.k = p.contraction;
  g.bias = bias; g.bias_per_row = bias ? 1 : 0;
  g.out = out;
  g.scale = 1.0f;
  g.activation = NUMR_B200_ACT_NONE;
  g.stream = stream;
  g.device_index = dev;
  g.f32_exact = p.exact ? 1 : 0;
  if (p.split_bytes && ws_bytes >= p.total) {
    g.split_ws = w + p.off_split;
    g.split_ws_bytes = p.split_bytes;
  }
  return launch_gemm_sm100(g);
}

}  // namespace
}  // namespace nb

using namespace nb;

extern "C" {

numr_b200_status numr_b200_conv_out_shape(const numr_b200_conv_desc* d, int32_t kind, uint32_t* out_h, uint32_t* out_w) {
  ConvPlan p;
  int st = make_conv_plan(d, kind, nullptr, &p, -1);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (out_h) *out_h = p.g.out_h;
  if (out_w) *out_w = p.g.out_w;
  return NUMR_B200_OK;
}

size_t numr_b200_conv_workspace_bytes(const numr_b200_conv_desc* d, int32_t kind, const void* weight) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    dev = -1;
  }
  ConvPlan p;
  if (make_conv_plan(d, kind, weight, &p, dev) != NUMR_B200_OK) return 0;
  if (d->batch == 0 || d->c_out == 0 || p.spatial == 0) return 0;
  return p.total;
}

numr_b200_status numr_b200_conv1d(const numr_b200_conv_desc* d, const void* input, const void* weight, const void* bias,
                                  void* out, void* ws, size_t ws_bytes, void* cu_stream, int device_index) {
  return (numr_b200_status)run_conv(d, CONV1D, input, weight, bias, out, ws, ws_bytes, cu_stream, device_index);
}

numr_b200_status numr_b200_conv2d(const numr_b200_conv_desc* d, const void* input, const void* weight, const void* bias,
                                  void* out, void* ws, size_t ws_bytes, void* cu_stream, int device_index) {
  return (numr_b200_status)run_conv(d, CONV2D, input, weight, bias, out, ws, ws_bytes, cu_stream, device_index);
}

numr_b200_status numr_b200_conv_transpose1d(const numr_b200_conv_desc* d, const void* input, const void* weight,
                                            const void* bias, void* out, void* ws, size_t ws_bytes, void* cu_stream,
                                            int device_index) {
  return (numr_b200_status)run_conv(d, CONV_T1D, input, weight, bias, out, ws, ws_bytes, cu_stream, device_index);
}

}  // extern "C"
