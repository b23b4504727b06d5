// Op layer: the validation, shape, broadcast and dispatch rules numr applies above its
// CUDA launchers, restated over plain tensor descriptors so that a caller holding
// Tensor<CudaRuntime>-like views (pointer, shape, strides, dtype) gets the reference's
// behaviour and error classes:
//   shapes      src/ops/matmul.rs:73-255 (1-D promotion, NumPy batch broadcast, bias [N])
//   dtypes      src/ops/matmul_dtype.rs:19-100 (I8 -> I32, I32 bias, I8 rejected by epilogue ops)
//   dispatch    src/ops/cuda/matmul.rs:17-288, src/ops/cuda/gemm_epilogue.rs:25-256,
//               src/ops/cuda/fp8_matmul.rs:81-214
//   layouts     transposed-B views are read in place (is_transposed_b, src/ops/matmul.rs:193-211);
//               any other non-contiguous view is gathered first (ensure_contiguous,
//               src/runtime/cuda/ops/helpers/matmul.rs:91-92)
// Unlike the reference, unaligned F16/BF16 shapes are not padded and sliced here: the
// kernel handles ragged tiles itself.
#include <algorithm>
#include <cstring>
#include <vector>

#include "gemm_internal.h"

namespace nb {
namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

uint32_t dtype_bytes(int dt) {
  switch (dt) {
    case NUMR_B200_I64: case NUMR_B200_U64: return 8;
    case NUMR_B200_F32: case NUMR_B200_I32: case NUMR_B200_U32: return 4;
    case NUMR_B200_BF16: case NUMR_B200_F16: case NUMR_B200_I16: case NUMR_B200_U16: return 2;
    case NUMR_B200_FP8E4M3: case NUMR_B200_FP8E5M2: case NUMR_B200_I8: case NUMR_B200_U8: return 1;
    default: return 0;
  }
}

int matmul_output_dtype(int dt) { return dt == NUMR_B200_I8 ? NUMR_B200_I32 : dt; }

bool tensor_ok(const numr_b200_tensor* t, const char* name) {
  if (!t) { set_error("%s tensor is NULL", name); return false; }
  if (t->ndim < 0 || t->ndim > 8) { set_error("%s: ndim %d out of range 0..8", name, t->ndim); return false; }
  for (int i = 0; i < t->ndim; ++i)
    if (t->shape[i] < 0) { set_error("%s: negative extent", name); return false; }
  return true;
}

bool is_contiguous(const numr_b200_tensor& t) {
  int64_t expect = 1;
  for (int i = t.ndim - 1; i >= 0; --i) {
    if (t.shape[i] != 1 && t.strides[i] != expect) return false;
    expect *= t.shape[i];
  }
  return true;
}

// Shapes of one matmul after 1-D promotion and batch broadcast.
struct Shapes {
  int64_t m = 0, k = 0, n = 0;
  std::vector<int64_t> a_batch, b_batch, out_batch;
  std::vector<int64_t> out;    // full output shape
  int64_t batch = 1;           // product of out_batch
};

bool broadcast(const std::vector<int64_t>& x, const std::vector<int64_t>& y, std::vector<int64_t>* out) {
  const size_t nd = std::max(x.size(), y.size());
  out->assign(nd, 1);
  for (size_t i = 0; i < nd; ++i) {
    const int64_t dx = i < nd - x.size() ? 1 : x[i - (nd - x.size())];
    const int64_t dy = i < nd - y.size() ? 1 : y[i - (nd - y.size())];
    if (dx == dy) (*out)[i] = dx;
    else if (dx == 1) (*out)[i] = dy;
    else if (dy == 1) (*out)[i] = dx;
    else return false;
  }
  return true;
}

// validate_matmul_shapes + matmul_output_shape.
int resolve_shapes(const numr_b200_tensor& a, const numr_b200_tensor& b, Shapes* s) {
  if (a.ndim == 0 || b.ndim == 0)
    return fail(NUMR_B200_ESHAPE, "matmul: 0-dimensional operand");
  int64_t a_rows, a_cols, b_rows, b_cols;
  if (a.ndim == 1) { a_rows = 1; a_cols = a.shape[0]; }
  else { a_rows = a.shape[a.ndim - 2]; a_cols = a.shape[a.ndim - 1]; }
  if (b.ndim == 1) { b_rows = b.shape[0]; b_cols = 1; }
  else { b_rows = b.shape[b.ndim - 2]; b_cols = b.shape[b.ndim - 1]; }
  if (a_cols != b_rows)
    return fail(NUMR_B200_ESHAPE, "matmul: inner dimensions differ (A has K=%lld, B has K=%lld)",
                (long long)a_cols, (long long)b_rows);
  s->m = a_rows; s->k = a_cols; s->n = b_cols;
  s->a_batch.assign(a.shape, a.shape + (a.ndim > 2 ? a.ndim - 2 : 0));
  s->b_batch.assign(b.shape, b.shape + (b.ndim > 2 ? b.ndim - 2 : 0));
  if (!broadcast(s->a_batch, s->b_batch, &s->out_batch))
    return fail(NUMR_B200_ESHAPE, "matmul: batch dimensions do not broadcast");
  s->out = s->out_batch;
  s->out.push_back(s->m);
  s->out.push_back(s->n);
  s->batch = 1;
  for (int64_t d : s->out_batch) s->batch *= d;
  return NUMR_B200_OK;
}

// matmul_batch_indices for one operand: which operand batch each output batch reads.
std::vector<int64_t> batch_indices(const std::vector<int64_t>& out_batch, const std::vector<int64_t>& op_batch) {
  int64_t total = 1;
  for (int64_t d : out_batch) total *= d;
  std::vector<int64_t> idx((size_t)total);
  std::vector<int64_t> coord(out_batch.size());
  const size_t offset = out_batch.size() - op_batch.size();
  for (int64_t flat = 0; flat < total; ++flat) {
    int64_t rem = flat;
    for (int d = (int)out_batch.size() - 1; d >= 0; --d) { coord[d] = rem % out_batch[d]; rem /= out_batch[d]; }
    int64_t v = 0;
    for (size_t d = 0; d < op_batch.size(); ++d) {
      const int64_t c = op_batch[d] == 1 ? 0 : coord[offset + d];
      v = v * op_batch[d] + c;
    }
    idx[(size_t)flat] = v;
  }
  return idx;
}

// How one matrix operand is handed to the GEMM.
struct OperandView {
  bool gather = false;          // materialise into the workspace first
  bool broadcast_gather = false;  // gathered copy is expanded to the full output batch
  int layout = NUMR_B200_B_KN;  // for B
  uint32_t batch_count = 1;     // operand batch count the kernel indexes with bi % count
  size_t gather_bytes = 0;
};

bool is_transposed_b(const numr_b200_tensor& b, int64_t k, int64_t n) {
  if (b.ndim < 2 || k == 0 || n == 0) return false;
  if (b.strides[b.ndim - 2] != 1 || b.strides[b.ndim - 1] != k) return false;
  int64_t expect = n * k;
  for (int d = b.ndim - 3; d >= 0; --d) {
    if (b.shape[d] != 1 && b.strides[d] != expect) return false;
    expect *= b.shape[d];
  }
  return true;
}

// Decides whether `t` (matrix dims rows x cols, batch dims op_batch) can be read in place.
OperandView plan_operand(const numr_b200_tensor& t, const std::vector<int64_t>& op_batch,
                         const std::vector<int64_t>& out_batch, int64_t rows, int64_t cols,
                         int64_t out_batch_count, bool is_b, uint32_t elt) {
  OperandView v;
  int64_t count = 1;
  for (int64_t d : op_batch) count *= d;
  // Can `bi % count` express the broadcast? (count == 1, or indices == bi % count)
  bool modulo_ok = true;
  if (count != 1) {
    const std::vector<int64_t> idx = batch_indices(out_batch, op_batch);
    for (size_t i = 0; i < idx.size(); ++i)
      if (idx[i] != (int64_t)(i % (size_t)count)) { modulo_ok = false; break; }
  }
  bool dense = is_contiguous(t);
  if (is_b && !dense && t.ndim >= 2 && is_transposed_b(t, rows, cols)) {
    v.layout = NUMR_B200_B_NK;
    dense = true;
  }
  if (dense && modulo_ok) {
    v.batch_count = (uint32_t)count;
    return v;
  }
  v.gather = true;
  v.broadcast_gather = !modulo_ok;
  const int64_t copies = modulo_ok ? count : out_batch_count;
  v.batch_count = (uint32_t)copies;
  v.gather_bytes = (size_t)copies * (size_t)rows * (size_t)cols * elt;
  return v;
}

// Gathers `t` into dst as [copies][rows][cols] contiguous.
int gather_operand(const numr_b200_tensor& t, const OperandView& v, const std::vector<int64_t>& op_batch,
                   const std::vector<int64_t>& out_batch, int64_t rows, int64_t cols, bool promote_1d_a,
                   bool promote_1d_b, void* dst, uint32_t elt, cudaStream_t stream) {
  int64_t shape[8], strides[8];
  int nd = 0;
  if (v.broadcast_gather) {
    // Expand to the output batch dims: stride 0 along broadcast dims.
    const size_t offset = out_batch.size() - op_batch.size();
    if (out_batch.size() + 2 > 8) return fail(NUMR_B200_EINVAL, "matmul: too many batch dimensions to gather");
    for (size_t d = 0; d < out_batch.size(); ++d) {
      shape[nd] = out_batch[d];
      if (d < offset) strides[nd] = 0;
      else strides[nd] = op_batch[d - offset] == 1 ? 0 : t.strides[d - offset];
      ++nd;
    }
  } else {
    for (size_t d = 0; d < op_batch.size(); ++d) { shape[nd] = op_batch[d]; strides[nd] = t.strides[d]; ++nd; }
  }
  if (promote_1d_a) { shape[nd] = 1; strides[nd] = 0; ++nd; shape[nd] = cols; strides[nd] = t.strides[0]; ++nd; }
  else if (promote_1d_b) { shape[nd] = rows; strides[nd] = t.strides[0]; ++nd; shape[nd] = 1; strides[nd] = 0; ++nd; }
  else {
    shape[nd] = rows; strides[nd] = t.strides[t.ndim - 2]; ++nd;
    shape[nd] = cols; strides[nd] = t.strides[t.ndim - 1]; ++nd;
  }
  return launch_gather_strided(reinterpret_cast<const void*>(static_cast<uintptr_t>(t.ptr)), dst, nd, shape,
                               strides, elt, stream);
}

struct OpArgs {
  const char* op;
  const numr_b200_tensor* a;
  const numr_b200_tensor* b;
  const numr_b200_tensor* bias;       // nullable
  const numr_b200_tensor* residual;   // nullable
  const numr_b200_tensor* out;
  int out_dtype;
  int activation;
  int f32_mode;
  float scale_a, scale_b;
};

struct OpPlan {
  Shapes s;
  OperandView av, bv;
  bool gather_bias = false, gather_res = false;
  size_t off_a = 0, off_b = 0, off_bias = 0, off_res = 0, off_gemm = 0;
  size_t gemm_ws = 0, total_ws = 0;
  numr_b200_gemm_desc desc;
};

int make_op_plan(const OpArgs& o, OpPlan* p) {
  if (!tensor_ok(o.a, "a") || !tensor_ok(o.b, "b")) return NUMR_B200_EINVAL;
  int st = resolve_shapes(*o.a, *o.b, &p->s);
  if (st != NUMR_B200_OK) return st;
  const Shapes& s = p->s;
  if (s.m > 0x7FFFFFFFll || s.n > 0x7FFFFFFFll || s.k > 0x7FFFFFFFll || s.batch > 0x7FFFFFFFll)
    return fail(NUMR_B200_EINVAL, "%s: dimension exceeds 2^31-1", o.op);
  const uint32_t elt = dtype_bytes(o.a->dtype);
  if (!elt) return fail(NUMR_B200_EUNSUPPORTED, "%s: unsupported dtype %d", o.op, o.a->dtype);

  p->av = plan_operand(*o.a, s.a_batch, s.out_batch, s.m, s.k, s.batch, false, elt);
  p->bv = plan_operand(*o.b, s.b_batch, s.out_batch, s.k, s.n, s.batch, true, dtype_bytes(o.b->dtype));
  if (s.k == 0 || s.batch == 0 || s.m == 0 || s.n == 0) { p->av.gather = p->bv.gather = false; p->av.gather_bytes = p->bv.gather_bytes = 0; }

  if (o.bias) {
    p->gather_bias = o.bias->ndim == 1 && o.bias->shape[0] > 1 && o.bias->strides[0] != 1;
  }
  if (o.residual) p->gather_res = !is_contiguous(*o.residual);

  numr_b200_gemm_desc& d = p->desc;
  memset(&d, 0, sizeof(d));
  d.a_dtype = o.a->dtype;
  d.b_dtype = o.b->dtype;
  d.out_dtype = o.out_dtype;
  d.bias_dtype = o.bias ? o.bias->dtype : o.out_dtype;
  d.batch = (uint32_t)s.batch;
  d.m = (uint32_t)s.m; d.n = (uint32_t)s.n; d.k = (uint32_t)s.k;
  d.a_batch = p->av.batch_count ? p->av.batch_count : 1;
  d.b_batch = p->bv.batch_count ? p->bv.batch_count : 1;
  d.b_layout = p->bv.gather ? NUMR_B200_B_KN : p->bv.layout;
  d.activation = o.activation;
  d.f32_mode = o.f32_mode;
  d.scale_a = o.scale_a;
  d.scale_b = o.scale_b;

  // Workspace: gathered operands first, then what the GEMM itself asks for.
  const uint32_t out_elt = dtype_bytes(o.out_dtype);
  size_t off = 0;
  if (p->av.gather) { p->off_a = off; off = align_up(off + p->av.gather_bytes, 256); }
  if (p->bv.gather) { p->off_b = off; off = align_up(off + p->bv.gather_bytes, 256); }
  if (p->gather_bias) { p->off_bias = off; off = align_up(off + (size_t)s.n * dtype_bytes(o.bias->dtype), 256); }
  if (p->gather_res) { p->off_res = off; off = align_up(off + (size_t)s.batch * s.m * s.n * out_elt, 256); }
  p->off_gemm = off;
  const void* a_ptr = p->av.gather ? nullptr : reinterpret_cast<const void*>(static_cast<uintptr_t>(o.a->ptr));
  const void* b_ptr = p->bv.gather ? nullptr : reinterpret_cast<const void*>(static_cast<uintptr_t>(o.b->ptr));
  p->gemm_ws = numr_b200_gemm_workspace_bytes(&d, a_ptr, b_ptr);
  p->total_ws = off + p->gemm_ws;
  return NUMR_B200_OK;
}

int check_out(const OpArgs& o, const Shapes& s) {
  if (!tensor_ok(o.out, "out")) return NUMR_B200_EINVAL;
  if (o.out->dtype != o.out_dtype)
    return fail(NUMR_B200_EDTYPE, "%s: output tensor has dtype %d, the op writes %d", o.op, o.out->dtype, o.out_dtype);
  if ((size_t)o.out->ndim != s.out.size())
    return fail(NUMR_B200_ESHAPE, "%s: output tensor has %d dims, expected %zu", o.op, o.out->ndim, s.out.size());
  for (int i = 0; i < o.out->ndim; ++i)
    if (o.out->shape[i] != s.out[(size_t)i])
      return fail(NUMR_B200_ESHAPE, "%s: output extent %d is %lld, expected %lld", o.op, i,
                  (long long)o.out->shape[i], (long long)s.out[(size_t)i]);
  if (!is_contiguous(*o.out)) return fail(NUMR_B200_EINVAL, "%s: output tensor must be contiguous", o.op);
  return NUMR_B200_OK;
}

int run_op(const OpArgs& o, void* ws, size_t ws_bytes, void* cu_stream, int device_index) {
  OpPlan p;
  int st = make_op_plan(o, &p);
  if (st != NUMR_B200_OK) return st;
  const Shapes& s = p.s;
  if (o.bias) {
    if (!tensor_ok(o.bias, "bias")) return NUMR_B200_EINVAL;
    if (o.bias->ndim != 1)
      return fail(NUMR_B200_EINVAL, "%s: bias must be a 1-D tensor, got %d dims", o.op, o.bias->ndim);
    if (o.bias->shape[0] != s.n)
      return fail(NUMR_B200_ESHAPE, "%s: bias has %lld elements, output has %lld columns", o.op,
                  (long long)o.bias->shape[0], (long long)s.n);
  }
  if (o.residual) {
    if (!tensor_ok(o.residual, "residual")) return NUMR_B200_EINVAL;
    if (o.residual->dtype != o.out_dtype)
      return fail(NUMR_B200_EDTYPE, "%s: residual dtype %d differs from the output dtype %d", o.op,
                  o.residual->dtype, o.out_dtype);
    bool same = (size_t)o.residual->ndim == s.out.size();
    for (int i = 0; same && i < o.residual->ndim; ++i) same = o.residual->shape[i] == s.out[(size_t)i];
    if (!same) return fail(NUMR_B200_ESHAPE, "%s: residual shape differs from the output shape", o.op);
  }
  st = check_out(o, s);
  if (st != NUMR_B200_OK) return st;
  if (s.batch == 0 || s.m == 0 || s.n == 0) return NUMR_B200_OK;

  if (p.total_ws) {
    if (!ws || ws_bytes < p.total_ws)
      return fail(NUMR_B200_EWORKSPACE, "%s: workspace of %zu bytes needed, %zu given", o.op, p.total_ws,
                  ws ? ws_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(ws) & 255)
      return fail(NUMR_B200_EWORKSPACE, "%s: workspace %p is not 256-byte aligned", o.op, ws);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  char* w = static_cast<char*>(ws);
  const void* a_ptr = reinterpret_cast<const void*>(static_cast<uintptr_t>(o.a->ptr));
  const void* b_ptr = reinterpret_cast<const void*>(static_cast<uintptr_t>(o.b->ptr));
  const void* bias_ptr = o.bias ? reinterpret_cast<const void*>(static_cast<uintptr_t>(o.bias->ptr)) : nullptr;
  const void* res_ptr = o.residual ? reinterpret_cast<const void*>(static_cast<uintptr_t>(o.residual->ptr)) : nullptr;
  const uint32_t elt = dtype_bytes(o.a->dtype);
  if (p.av.gather) {
    st = gather_operand(*o.a, p.av, s.a_batch, s.out_batch, s.m, s.k, o.a->ndim == 1, false, w + p.off_a, elt, stream);
    if (st != NUMR_B200_OK) return st;
    a_ptr = w + p.off_a;
  }
  if (p.bv.gather) {
    st = gather_operand(*o.b, p.bv, s.b_batch, s.out_batch, s.k, s.n, false, o.b->ndim == 1, w + p.off_b,
                        dtype_bytes(o.b->dtype), stream);
    if (st != NUMR_B200_OK) return st;
    b_ptr = w + p.off_b;
  }
  if (p.gather_bias) {
    st = launch_gather_strided(bias_ptr, w + p.off_bias, 1, o.bias->shape, o.bias->strides,
                               dtype_bytes(o.bias->dtype), stream);
    if (st != NUMR_B200_OK) return st;
    bias_ptr = w + p.off_bias;
  }
  if (p.gather_res) {
    st = launch_gather_strided(res_ptr, w + p.off_res, o.residual->ndim, o.residual->shape,
                               o.residual->strides, dtype_bytes(o.out_dtype), stream);
    if (st != NUMR_B200_OK) return st;
    res_ptr = w + p.off_res;
  }
  return numr_b200_gemm(&p.desc, a_ptr, b_ptr, bias_ptr, res_ptr,
                        reinterpret_cast<void*>(static_cast<uintptr_t>(o.out->ptr)),
                        p.gemm_ws ? w + p.off_gemm : nullptr, p.gemm_ws, cu_stream, device_index);
}

// validate_binary_dtypes / validate_matmul_bias_dtypes / validate_gemm_epilogue_dtypes.
int check_dtypes(const char* op, const numr_b200_tensor* a, const numr_b200_tensor* b,
                 const numr_b200_tensor* bias, bool epilogue_op) {
  if (!tensor_ok(a, "a") || !tensor_ok(b, "b")) return NUMR_B200_EINVAL;
  if (epilogue_op && matmul_output_dtype(a->dtype) != a->dtype)
    return fail(NUMR_B200_EUNSUPPORTED, "%s: unsupported dtype I8", op);
  if (a->dtype != b->dtype)
    return fail(NUMR_B200_EDTYPE, "%s: dtype mismatch between A (%d) and B (%d)", op, a->dtype, b->dtype);
  if (bias) {
    if (!tensor_ok(bias, "bias")) return NUMR_B200_EINVAL;
    const int out_dt = matmul_output_dtype(a->dtype);
    if (bias->dtype != out_dt) {
      if (out_dt != a->dtype)
        return fail(NUMR_B200_EINVAL,
                    "%s on I8 operands accumulates into I32, so the bias must be I32, got dtype %d", op,
                    bias->dtype);
      return fail(NUMR_B200_EDTYPE, "%s: dtype mismatch between A (%d) and bias (%d)", op, a->dtype, bias->dtype);
    }
  }
  return NUMR_B200_OK;
}

}  // namespace
}  // namespace nb

using namespace nb;

extern "C" {

numr_b200_status numr_b200_matmul_out_shape(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                            const numr_b200_tensor* bias, int64_t out_shape[8],
                                            int32_t* out_ndim, int32_t* out_dtype) {
  if (!tensor_ok(a, "a") || !tensor_ok(b, "b")) return NUMR_B200_EINVAL;
  Shapes s;
  int st = resolve_shapes(*a, *b, &s);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (bias) {
    if (!tensor_ok(bias, "bias")) return NUMR_B200_EINVAL;
    if (bias->ndim != 1 || bias->shape[0] != s.n)
      return (numr_b200_status)fail(NUMR_B200_ESHAPE, "matmul_bias: bias must be 1-D with %lld elements", (long long)s.n);
  }
  if (s.out.size() > 8) return (numr_b200_status)fail(NUMR_B200_EINVAL, "matmul: more than 8 output dimensions");
  for (size_t i = 0; i < s.out.size(); ++i) out_shape[i] = s.out[i];
  if (out_ndim) *out_ndim = (int32_t)s.out.size();
  if (out_dtype) *out_dtype = matmul_output_dtype(a->dtype);
  return NUMR_B200_OK;
}

size_t numr_b200_op_workspace_bytes(const numr_b200_tensor* a, const numr_b200_tensor* b, int32_t out_dtype,
                                    int32_t f32_mode) {
  OpArgs o{"workspace", a, b, nullptr, nullptr, nullptr, out_dtype, 0, f32_mode, 1.0f, 1.0f};
  OpPlan p;
  if (make_op_plan(o, &p) != NUMR_B200_OK) return 0;
  // Bias / residual gathers are only needed for non-contiguous epilogue operands; budget
  // for them so one query serves every op on these operands.
  const size_t extra = align_up((size_t)p.s.n * 8, 256) +
                       align_up((size_t)p.s.batch * p.s.m * p.s.n * dtype_bytes(out_dtype), 256);
  return p.total_ws + extra;
}

size_t numr_b200_op_workspace_bytes_for(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                        const numr_b200_tensor* bias, const numr_b200_tensor* residual,
                                        int32_t out_dtype, int32_t f32_mode) {
  OpArgs o{"workspace", a, b, bias, residual, nullptr, out_dtype, 0, f32_mode, 1.0f, 1.0f};
  OpPlan p;
  if (make_op_plan(o, &p) != NUMR_B200_OK) return 0;
  return p.total_ws;
}

numr_b200_status numr_b200_matmul(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                  const numr_b200_tensor* out, int32_t f32_mode, void* ws, size_t ws_bytes,
                                  void* cu_stream, int device_index) {
  int st = check_dtypes("matmul", a, b, nullptr, false);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  OpArgs o{"matmul", a, b, nullptr, nullptr, out, matmul_output_dtype(a->dtype), 0, f32_mode, 1.0f, 1.0f};
  return (numr_b200_status)run_op(o, ws, ws_bytes, cu_stream, device_index);
}

numr_b200_status numr_b200_matmul_bias(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                       const numr_b200_tensor* bias, const numr_b200_tensor* out,
                                       int32_t f32_mode, void* ws, size_t ws_bytes, void* cu_stream,
                                       int device_index) {
  if (!bias) return (numr_b200_status)fail(NUMR_B200_EINVAL, "matmul_bias: bias tensor is NULL");
  int st = check_dtypes("matmul_bias", a, b, bias, false);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  OpArgs o{"matmul_bias", a, b, bias, nullptr, out, matmul_output_dtype(a->dtype), 0, f32_mode, 1.0f, 1.0f};
  return (numr_b200_status)run_op(o, ws, ws_bytes, cu_stream, device_index);
}

numr_b200_status numr_b200_matmul_bias_activation(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                                  const numr_b200_tensor* bias, int32_t activation,
                                                  const numr_b200_tensor* out, int32_t f32_mode, void* ws,
                                                  size_t ws_bytes, void* cu_stream, int device_index) {
  if (!bias) return (numr_b200_status)fail(NUMR_B200_EINVAL, "matmul_bias_activation: bias tensor is NULL");
  int st = check_dtypes("matmul_bias_activation", a, b, bias, true);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (activation < 0 || activation > 5)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "matmul_bias_activation: activation code %d", activation);
  OpArgs o{"matmul_bias_activation", a, b, bias, nullptr, out, a->dtype, activation, f32_mode, 1.0f, 1.0f};
  return (numr_b200_status)run_op(o, ws, ws_bytes, cu_stream, device_index);
}

numr_b200_status numr_b200_matmul_activation(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                             int32_t activation, const numr_b200_tensor* out,
                                             int32_t f32_mode, void* ws, size_t ws_bytes, void* cu_stream,
                                             int device_index) {
  int st = check_dtypes("matmul_activation", a, b, nullptr, true);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (activation < 0 || activation > 5)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "matmul_activation: activation code %d", activation);
  OpArgs o{"matmul_activation", a, b, nullptr, nullptr, out, a->dtype, activation, f32_mode, 1.0f, 1.0f};
  return (numr_b200_status)run_op(o, ws, ws_bytes, cu_stream, device_index);
}

numr_b200_status numr_b200_matmul_bias_residual(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                                const numr_b200_tensor* bias,
                                                const numr_b200_tensor* residual,
                                                const numr_b200_tensor* out, int32_t f32_mode, void* ws,
                                                size_t ws_bytes, void* cu_stream, int device_index) {
  if (!bias || !residual)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "matmul_bias_residual: bias or residual tensor is NULL");
  int st = check_dtypes("matmul_bias_residual", a, b, bias, true);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  OpArgs o{"matmul_bias_residual", a, b, bias, residual, out, a->dtype, 0, f32_mode, 1.0f, 1.0f};
  return (numr_b200_status)run_op(o, ws, ws_bytes, cu_stream, device_index);
}

static int check_fp8(const char* op, const numr_b200_tensor* a, const numr_b200_tensor* b, int a_e5m2,
                     const numr_b200_tensor* out) {
  if (!tensor_ok(a, "a") || !tensor_ok(b, "b") || !tensor_ok(out, "out")) return NUMR_B200_EINVAL;
  const int want_a = a_e5m2 ? NUMR_B200_FP8E5M2 : NUMR_B200_FP8E4M3;
  if (a->dtype != want_a)
    return fail(NUMR_B200_EDTYPE, "%s: A must be %s, got dtype %d", op, a_e5m2 ? "FP8E5M2" : "FP8E4M3", a->dtype);
  if (b->dtype != NUMR_B200_FP8E4M3)
    return fail(NUMR_B200_EDTYPE, "%s: B must be FP8E4M3, got dtype %d", op, b->dtype);
  if (out->dtype != NUMR_B200_F32 && out->dtype != NUMR_B200_F16 && out->dtype != NUMR_B200_BF16)
    return fail(NUMR_B200_EUNSUPPORTED, "%s: output dtype must be F32, F16 or BF16, got %d", op, out->dtype);
  return NUMR_B200_OK;
}

numr_b200_status numr_b200_fp8_matmul(const numr_b200_tensor* a, const numr_b200_tensor* b, float scale_a,
                                      float scale_b, int32_t a_e5m2, const numr_b200_tensor* out, void* ws,
                                      size_t ws_bytes, void* cu_stream, int device_index) {
  int st = check_fp8(a_e5m2 ? "fp8_matmul_e5m2" : "fp8_matmul", a, b, a_e5m2, out);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  OpArgs o{a_e5m2 ? "fp8_matmul_e5m2" : "fp8_matmul", a, b, nullptr, nullptr, out, out->dtype, 0, 0, scale_a, scale_b};
  return (numr_b200_status)run_op(o, ws, ws_bytes, cu_stream, device_index);
}

numr_b200_status numr_b200_fp8_matmul_fused(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                            float scale_a, float scale_b, const numr_b200_tensor* bias,
                                            int32_t activation, const numr_b200_tensor* residual,
                                            const numr_b200_tensor* out, void* ws, size_t ws_bytes,
                                            void* cu_stream, int device_index) {
  int st = check_fp8("fp8_matmul_fused", a, b, 0, out);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (activation < 0 || activation > 5)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "fp8_matmul_fused: activation code %d", activation);
  if (bias && bias->dtype != out->dtype)
    return (numr_b200_status)fail(NUMR_B200_EDTYPE, "fp8_matmul_fused: bias dtype %d differs from the output dtype %d",
                                  bias->dtype, out->dtype);
  OpArgs o{"fp8_matmul_fused", a, b, bias, residual, out, out->dtype, activation, 0, scale_a, scale_b};
  return (numr_b200_status)run_op(o, ws, ws_bytes, cu_stream, device_index);
}


// ---- GroupedMatmulOps (src/ops/traits/grouped_matmul.rs:31-52); validation after
// validate_grouped (src/ops/cpu/grouped_matmul.rs:13-75).
static int grouped_desc(const numr_b200_tensor* a, const numr_b200_tensor* b, const numr_b200_tensor* offsets,
                        int32_t activation, int32_t f32_mode, numr_b200_gemm_desc* d, uint32_t* groups) {
  if (!tensor_ok(a, "a") || !tensor_ok(b, "b")) return NUMR_B200_EINVAL;
  if (a->ndim != 2) return fail(NUMR_B200_EINVAL, "grouped_matmul: a: expected 2-D [total_rows, k], got %d-D", a->ndim);
  if (b->ndim != 3) return fail(NUMR_B200_EINVAL, "grouped_matmul: b: expected 3-D [num_groups, k, n], got %d-D", b->ndim);
  if (offsets) {
    if (!tensor_ok(offsets, "group_offsets")) return NUMR_B200_EINVAL;
    if (offsets->ndim != 1)
      return fail(NUMR_B200_EINVAL, "grouped_matmul: group_offsets: expected 1-D [num_groups + 1], got %d-D", offsets->ndim);
    if (offsets->dtype != NUMR_B200_I32)
      return fail(NUMR_B200_EINVAL, "grouped_matmul: group_offsets: expected I32, got dtype %d", offsets->dtype);
  }
  if (a->dtype != b->dtype)
    return fail(NUMR_B200_EINVAL, "grouped_matmul: dtype: a is %d but b is %d", a->dtype, b->dtype);
  if (a->dtype != NUMR_B200_F32 && a->dtype != NUMR_B200_F16 && a->dtype != NUMR_B200_BF16)
    return fail(NUMR_B200_EINVAL, "grouped_matmul: dtype: supports F32/F16/BF16, got dtype %d", a->dtype);
  if (a->shape[1] != b->shape[1])
    return fail(NUMR_B200_ESHAPE, "grouped_matmul: a has k = %lld, b has k = %lld", (long long)a->shape[1], (long long)b->shape[1]);
  if (offsets && offsets->shape[0] != b->shape[0] + 1)
    return fail(NUMR_B200_EINVAL, "grouped_matmul: group_offsets: expected %lld entries, got %lld",
                (long long)b->shape[0] + 1, (long long)offsets->shape[0]);
  if (activation < 0 || activation > NUMR_B200_ACT_TANH)
    return fail(NUMR_B200_EINVAL, "grouped_matmul: activation code %d", activation);
  if (!is_contiguous(*a) || !is_contiguous(*b) || (offsets && offsets->shape[0] > 1 && offsets->strides[0] != 1))
    return fail(NUMR_B200_EINVAL, "grouped_matmul: a, b and group_offsets must be contiguous");
  for (int i = 0; i < 3; ++i)
    if (b->shape[i] > 0x7FFFFFFFll || (i < 2 && a->shape[i] > 0x7FFFFFFFll))
      return fail(NUMR_B200_EINVAL, "grouped_matmul: dimension exceeds 2^31-1");
  memset(d, 0, sizeof(*d));
  d->a_dtype = d->b_dtype = d->out_dtype = d->bias_dtype = a->dtype;
  d->batch = 1; d->a_batch = 1; d->b_batch = (uint32_t)b->shape[0];
  d->m = (uint32_t)a->shape[0]; d->k = (uint32_t)a->shape[1]; d->n = (uint32_t)b->shape[2];
  d->b_layout = NUMR_B200_B_KN;
  d->activation = activation;
  d->f32_mode = f32_mode;
  d->scale_a = d->scale_b = 1.0f;
  *groups = (uint32_t)b->shape[0];
  return NUMR_B200_OK;
}

size_t numr_b200_grouped_matmul_workspace_bytes(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                                int32_t f32_mode) {
  numr_b200_gemm_desc d;
  uint32_t groups = 0;
  if (grouped_desc(a, b, nullptr, 0, f32_mode, &d, &groups) != NUMR_B200_OK) return 0;
  return numr_b200_grouped_gemm_workspace_bytes(&d, groups, reinterpret_cast<const void*>(static_cast<uintptr_t>(a->ptr)),
                                                reinterpret_cast<const void*>(static_cast<uintptr_t>(b->ptr)));
}

numr_b200_status numr_b200_grouped_matmul(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                          const numr_b200_tensor* group_offsets, int32_t activation,
                                          const numr_b200_tensor* out, int32_t f32_mode, void* ws,
                                          size_t ws_bytes, void* cu_stream, int device_index) {
  if (!group_offsets) return (numr_b200_status)fail(NUMR_B200_EINVAL, "grouped_matmul: group_offsets is NULL");
  numr_b200_gemm_desc d;
  uint32_t groups = 0;
  int st = grouped_desc(a, b, group_offsets, activation, f32_mode, &d, &groups);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (!tensor_ok(out, "out")) return NUMR_B200_EINVAL;
  if (out->dtype != a->dtype)
    return (numr_b200_status)fail(NUMR_B200_EDTYPE, "grouped_matmul: output tensor has dtype %d, the op writes %d", out->dtype, a->dtype);
  if (out->ndim != 2 || out->shape[0] != a->shape[0] || out->shape[1] != b->shape[2])
    return (numr_b200_status)fail(NUMR_B200_ESHAPE, "grouped_matmul: output must be [%lld, %lld]", (long long)a->shape[0], (long long)b->shape[2]);
  if (!is_contiguous(*out)) return (numr_b200_status)fail(NUMR_B200_EINVAL, "grouped_matmul: output tensor must be contiguous");
  return numr_b200_grouped_gemm(&d, groups, reinterpret_cast<const void*>(static_cast<uintptr_t>(a->ptr)),
                                reinterpret_cast<const void*>(static_cast<uintptr_t>(b->ptr)),
                                reinterpret_cast<const int32_t*>(static_cast<uintptr_t>(group_offsets->ptr)),
                                reinterpret_cast<void*>(static_cast<uintptr_t>(out->ptr)), ws, ws_bytes, cu_stream, device_index);
}


// ---- GemmEpilogueOps::matmul_bias_activation_bwd (src/ops/traits/gemm_epilogue.rs:107-140; CPU
// kernel src/runtime/cpu/kernels/gemm_epilogue/backward.rs:136-245; CUDA src/ops/cuda/gemm_epilogue.rs:258-366)
//   grad_pre = grad * activation'(a @ b + bias)      one GEMM with the backward epilogue
//   d_bias   = column sums of grad_pre
//   d_a      = grad_pre @ b^T                         b read in place as the transposed operand
//   d_b      = a^T @ grad_pre                         a^T materialised once (strided copy)
// a [..., M, K] and grad [..., M, N] may carry leading batch dimensions (product B):
//   * b 2-D ([K,N], or the transposed view of a contiguous [N,K]): one weight for all batches. The
//     batch folds into the rows (M' = B*M): d_b and d_bias sum over every batch, d_a keeps a's shape.
//   * b with the same leading dimensions as a: one weight per batch, d_b[i] = a[i]^T @ grad_pre[i]
//     (the reference's batched kernels add every batch's product into the first [K,N] block of d_b
//     and leave the others zero, src/ops/cpu/gemm_epilogue.rs:347-386; this returns the per-batch
//     gradient instead), d_bias still sums over all batches.
namespace {
struct BwdPlan {
  numr_b200_gemm_desc pre, da, db;
  size_t off_gp = 0, off_at = 0, off_ws = 0, gemm_ws = 0, total = 0;
  bool b_nk = false;
  int64_t batch = 1, m = 0, n = 0, k = 0;   // per-batch extents (batch = 1 when folded)
  int64_t rows = 0;                         // all rows of grad_pre: batch * m
  bool per_batch_b = false;
};

int bwd_plan(const numr_b200_tensor* grad, const numr_b200_tensor* a, const numr_b200_tensor* b,
             const numr_b200_tensor* bias, int32_t activation, int32_t f32_mode, BwdPlan* p) {
  const char* op = "matmul_bias_activation_bwd";
  int st = check_dtypes(op, a, b, bias, true);
  if (st != NUMR_B200_OK) return st;
  if (!tensor_ok(grad, "grad")) return NUMR_B200_EINVAL;
  if (a->dtype != NUMR_B200_F32 && a->dtype != NUMR_B200_F16 && a->dtype != NUMR_B200_BF16)
    return fail(NUMR_B200_EUNSUPPORTED, "%s: unsupported dtype %d (F32, F16, BF16)", op, a->dtype);
  if (grad->dtype != a->dtype)
    return fail(NUMR_B200_EDTYPE, "%s: dtype mismatch between A (%d) and grad (%d)", op, a->dtype, grad->dtype);
  if (activation < 0 || activation > NUMR_B200_ACT_TANH) return fail(NUMR_B200_EINVAL, "%s: activation code %d", op, activation);
  if (a->ndim < 2 || b->ndim < 2 || grad->ndim != a->ndim || (b->ndim != 2 && b->ndim != a->ndim))
    return fail(NUMR_B200_EUNSUPPORTED,
                "%s: a and grad need the same rank >= 2; b is 2-D (shared) or carries a's leading dimensions", op);
  if (bias->ndim != 1) return fail(NUMR_B200_EINVAL, "%s: bias must be a 1-D tensor, got %d dims", op, bias->ndim);
  const int lead = a->ndim - 2;
  int64_t batch = 1;
  for (int i = 0; i < lead; ++i) {
    if (grad->shape[i] != a->shape[i]) return fail(NUMR_B200_ESHAPE, "%s: grad and a differ in batch dimension %d", op, i);
    batch *= a->shape[i];
  }
  p->per_batch_b = b->ndim != 2;
  if (p->per_batch_b)
    for (int i = 0; i < lead; ++i)
      if (b->shape[i] != a->shape[i]) return fail(NUMR_B200_ESHAPE, "%s: b and a differ in batch dimension %d", op, i);
  const int64_t m1 = a->shape[lead], k = a->shape[lead + 1], n = b->shape[b->ndim - 1];
  if (b->shape[b->ndim - 2] != k) return fail(NUMR_B200_ESHAPE, "%s: a is [.., %lld, %lld], b has %lld rows", op, (long long)m1, (long long)k, (long long)b->shape[b->ndim - 2]);
  if (bias->shape[0] != n) return fail(NUMR_B200_ESHAPE, "%s: bias has %lld elements, b has %lld columns", op, (long long)bias->shape[0], (long long)n);
  if (grad->shape[lead] != m1 || grad->shape[lead + 1] != n) return fail(NUMR_B200_ESHAPE, "%s: grad must be [.., %lld, %lld]", op, (long long)m1, (long long)n);
  // one weight for all batches: the batch folds into the rows
  const int64_t gb = p->per_batch_b ? batch : 1;
  const int64_t m = p->per_batch_b ? m1 : batch * m1;
  if (m > 0x7FFFFFFFll || n > 0x7FFFFFFFll || k > 0x7FFFFFFFll || gb > 0x7FFFFFFFll) return fail(NUMR_B200_EINVAL, "%s: dimension exceeds 2^31-1", op);
  p->batch = gb; p->m = m; p->n = n; p->k = k; p->rows = gb * m;
  p->b_nk = !p->per_batch_b && !is_contiguous(*b) && is_transposed_b(*b, k, n);
  if (!is_contiguous(*a) || !is_contiguous(*grad) || !(is_contiguous(*b) || p->b_nk) ||
      (bias->shape[0] > 1 && bias->strides[0] != 1))
    return fail(NUMR_B200_EINVAL, "%s: a, grad and bias must be contiguous, b contiguous or (2-D) the transposed view of a contiguous [N,K]", op);
  const uint32_t elt = dtype_bytes(a->dtype);
  auto desc = [&](uint32_t mm, uint32_t nn, uint32_t kk, int layout, int act) {
    numr_b200_gemm_desc d;
    memset(&d, 0, sizeof(d));
    d.a_dtype = d.b_dtype = d.out_dtype = d.bias_dtype = a->dtype;
    d.batch = d.a_batch = d.b_batch = (uint32_t)std::max<int64_t>(gb, 1);
    d.m = mm; d.n = nn; d.k = kk;
    d.b_layout = layout;
    d.activation = act;
    d.f32_mode = f32_mode;
    d.scale_a = d.scale_b = 1.0f;
    return d;
  };
  // grad_pre [M,N]: b as given. d_a [M,K] = grad_pre [M,N] x (b^T as the [N,K] operand): a contiguous
  // [K,N] b is that operand in [N', K'] = [K, N] form; a transposed view of W[N,K] is it in [K', N'] form.
  p->pre = desc((uint32_t)m, (uint32_t)n, (uint32_t)k, p->b_nk ? NUMR_B200_B_NK : NUMR_B200_B_KN, activation | NUMR_B200_ACT_BWD);
  p->da = desc((uint32_t)m, (uint32_t)k, (uint32_t)n, p->b_nk ? NUMR_B200_B_KN : NUMR_B200_B_NK, NUMR_B200_ACT_NONE);
  p->db = desc((uint32_t)k, (uint32_t)n, (uint32_t)m, NUMR_B200_B_KN, NUMR_B200_ACT_NONE);
  size_t off = 0;
  p->off_gp = off; off = align_up(off + (size_t)gb * m * n * elt, 256);
  p->off_at = off; off = align_up(off + (size_t)gb * k * m * elt, 256);
  p->off_ws = off;
  size_t w = numr_b200_gemm_workspace_bytes(&p->pre, nullptr, nullptr);
  w = std::max(w, numr_b200_gemm_workspace_bytes(&p->da, nullptr, nullptr));
  w = std::max(w, numr_b200_gemm_workspace_bytes(&p->db, nullptr, nullptr));
  p->gemm_ws = w;
  p->total = off + w;
  return NUMR_B200_OK;
}
}  // namespace

size_t numr_b200_matmul_bias_activation_bwd_workspace_bytes(const numr_b200_tensor* grad, const numr_b200_tensor* a,
                                                            const numr_b200_tensor* b, const numr_b200_tensor* bias,
                                                            int32_t f32_mode) {
  BwdPlan p;
  if (bwd_plan(grad, a, b, bias, 0, f32_mode, &p) != NUMR_B200_OK) return 0;
  return p.total;
}

numr_b200_status numr_b200_matmul_bias_activation_bwd(const numr_b200_tensor* grad, const numr_b200_tensor* a,
                                                      const numr_b200_tensor* b, const numr_b200_tensor* bias,
                                                      int32_t activation, const numr_b200_tensor* d_a,
                                                      const numr_b200_tensor* d_b, const numr_b200_tensor* d_bias,
                                                      int32_t f32_mode, void* ws, size_t ws_bytes, void* cu_stream,
                                                      int device_index) {
  const char* op = "matmul_bias_activation_bwd";
  BwdPlan p;
  int st = bwd_plan(grad, a, b, bias, activation, f32_mode, &p);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  const int64_t m = p.m, k = p.k, n = p.n, gb = p.batch;
  // d_a has a's shape, d_b has b's shape, d_bias is [N]
  const numr_b200_tensor* outs[3] = {d_a, d_b, d_bias};
  const numr_b200_tensor* like[3] = {a, b, nullptr};
  const char* names[3] = {"d_a", "d_b", "d_bias"};
  for (int i = 0; i < 3; ++i) {
    if (!tensor_ok(outs[i], names[i])) return NUMR_B200_EINVAL;
    if (outs[i]->dtype != a->dtype)
      return (numr_b200_status)fail(NUMR_B200_EDTYPE, "%s: %s has dtype %d, the op writes %d", op, names[i], outs[i]->dtype, a->dtype);
    bool ok;
    if (like[i]) {
      ok = outs[i]->ndim == like[i]->ndim;
      for (int j = 0; ok && j < like[i]->ndim; ++j) ok = outs[i]->shape[j] == like[i]->shape[j];
    } else {
      ok = outs[i]->ndim == 1 && outs[i]->shape[0] == n;
    }
    if (!ok) return (numr_b200_status)fail(NUMR_B200_ESHAPE, "%s: %s has the wrong shape", op, names[i]);
    if (!is_contiguous(*outs[i])) return (numr_b200_status)fail(NUMR_B200_EINVAL, "%s: %s must be contiguous", op, names[i]);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  const uint32_t elt = dtype_bytes(a->dtype);
  auto ptr = [](const numr_b200_tensor* t) { return reinterpret_cast<void*>(static_cast<uintptr_t>(t->ptr)); };
  size_t b_elems = 1;
  for (int j = 0; j < b->ndim; ++j) b_elems *= (size_t)b->shape[j];
  if (gb == 0 || m == 0 || n == 0 || k == 0) {
    // sums over nothing: the additive identity (backward.rs and src/ops/cpu/gemm_epilogue.rs:305-315);
    // with k == 0 and rows present, d_bias still sums grad * activation'(bias): not offered here
    if (k == 0 && gb > 0 && m > 0 && n > 0) return (numr_b200_status)fail(NUMR_B200_EUNSUPPORTED, "%s: K = 0 with a non-empty output", op);
    cudaError_t e = cudaSuccess;
    if (gb * m * k) e = cudaMemsetAsync(ptr(d_a), 0, (size_t)gb * m * k * elt, stream);
    if (e == cudaSuccess && b_elems) e = cudaMemsetAsync(ptr(d_b), 0, b_elems * elt, stream);
    if (e == cudaSuccess && n) e = cudaMemsetAsync(ptr(d_bias), 0, (size_t)n * elt, stream);
    if (e != cudaSuccess) return (numr_b200_status)fail(NUMR_B200_ECUDA, "%s: clearing the gradients failed: %s", op, cudaGetErrorString(e));
    return NUMR_B200_OK;
  }
  if (!ws || ws_bytes < p.total)
    return (numr_b200_status)fail(NUMR_B200_EWORKSPACE, "%s: workspace of %zu bytes needed, %zu given", op, p.total, ws ? ws_bytes : (size_t)0);
  if (reinterpret_cast<uintptr_t>(ws) & 255) return (numr_b200_status)fail(NUMR_B200_EWORKSPACE, "%s: workspace %p is not 256-byte aligned", op, ws);
  char* w = static_cast<char*>(ws);
  void* gp = w + p.off_gp;
  void* at = w + p.off_at;
  void* gws = p.gemm_ws ? w + p.off_ws : nullptr;
  // 1. grad_pre = grad * activation'(a @ b + bias)
  numr_b200_status rs = numr_b200_gemm(&p.pre, ptr(a), ptr(b), ptr(bias), ptr(grad), gp, gws, p.gemm_ws, cu_stream, device_index);
  if (rs != NUMR_B200_OK) return rs;
  // 2. d_bias: column sums over every row of every batch
  const int out_kind = a->dtype == NUMR_B200_F32 ? OUT_F32 : (a->dtype == NUMR_B200_BF16 ? OUT_BF16 : OUT_F16);
  st = launch_column_sums(out_kind, gp, ptr(d_bias), (size_t)p.rows, (uint32_t)n, stream);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  // 3. d_a = grad_pre @ b^T
  rs = numr_b200_gemm(&p.da, gp, ptr(b), nullptr, nullptr, ptr(d_a), gws, p.gemm_ws, cu_stream, device_index);
  if (rs != NUMR_B200_OK) return rs;
  // 4. d_b = a^T @ grad_pre (per batch when b is per batch)
  const int64_t t_shape[3] = {gb, k, m}, t_strides[3] = {m * k, 1, k};
  st = launch_gather_strided(ptr(a), at, 3, t_shape, t_strides, elt, stream);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  return numr_b200_gemm(&p.db, at, gp, nullptr, nullptr, ptr(d_b), gws, p.gemm_ws, cu_stream, device_index);
}

}  // extern "C"
