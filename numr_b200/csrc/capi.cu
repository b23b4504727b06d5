// C ABI of the library: argument validation, workspace planning and the launcher
// mirrors. Nothing here allocates, frees or synchronises (numr_b200_device_status
// excepted, which exists for tests and health checks).
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "gemm_internal.h"
#include "sm100_ptx.cuh"

namespace nb {

// ------------------------------------------------------------------ errors
namespace {
thread_local char t_error[512] = "";
__device__ int g_kernel_status = 0;

// Scratch for numr_b200_gemm_static_scratch: lives in the library's device image, so every
// GPU that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = NUMR_B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return status;
}

int* device_status_ptr() {
  // One address per device; resolved on first use with that device current.
  static int* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kernel_status) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

int read_and_clear_device_status(int* out) {
  int v = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(int));
  if (e == cudaSuccess && v != 0) {
    int zero = 0;
    e = cudaMemcpyToSymbol(g_kernel_status, &zero, sizeof(int));
  }
  if (e != cudaSuccess) return fail(NUMR_B200_ECUDA, "reading the device status failed: %s", cudaGetErrorString(e));
  if (out) *out = v;
  return NUMR_B200_OK;
}

// Device address of g_static_scratch on the calling thread's current device. In host code the
// array's name is only a handle for the runtime, not an address a kernel can use; the address
// is looked up once per device (with that device current) and cached.
static void* static_scratch_address() {
  static void* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    set_error("static scratch: no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      set_error("static scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

// ------------------------------------------------------------------ planning
namespace {

uint32_t dtype_bytes(int dt) {
  switch (dt) {
    case NUMR_B200_I64: case NUMR_B200_U64: return 8;
    case NUMR_B200_F32: case NUMR_B200_I32: case NUMR_B200_U32: return 4;
    case NUMR_B200_BF16: case NUMR_B200_F16: case NUMR_B200_I16: case NUMR_B200_U16: return 2;
    case NUMR_B200_FP8E4M3: case NUMR_B200_FP8E5M2: case NUMR_B200_I8: case NUMR_B200_U8: return 1;
    default: return 0;
  }
}

const char* dtype_name(int dt) {
  static const char* names[] = {"F32", "BF16", "F16", "FP8E4M3", "FP8E5M2", "I8", "I32",
                                "I64", "I16", "U8", "U16", "U32", "U64"};
  return (dt >= 0 && dt <= 12) ? names[dt] : "?";
}

// Integer widths served by the CUDA-core kernel (everything integer except I8).
bool is_wide_int(int dt) {
  return dt == NUMR_B200_I32 || (dt >= NUMR_B200_I64 && dt <= NUMR_B200_U64);
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// How one operand reaches the kernel.
struct OperandPlan {
  bool repack = false;     // copy into the workspace (pad, or TF32 split for F32)
  uint32_t ld = 0;         // row pitch in elements as the kernel sees it
  size_t rows = 0;         // rows per batch
  uint32_t cols = 0;       // valid elements per row
  size_t bytes = 0;        // workspace bytes (all parts)
  size_t offset = 0;       // workspace offset
};

struct Plan {
  int kind = 0, out_kind = 0;
  uint32_t elt = 0, a_fmt = 0, b_fmt = 0;
  bool f32 = false, split3 = false;
  OperandPlan a, b;
  size_t split_off = 0, split_bytes = 0;   // scratch for the kernel's K split of its last wave
  size_t required_bytes = 0;   // operand preparation: without it the GEMM cannot run
  size_t ws_bytes = 0;         // required + the optional K-split scratch (what the query reports)
};

// Validates the descriptor and decides, per operand, whether it can be read in place.
int make_plan(const numr_b200_gemm_desc* d, const void* a, const void* b, Plan* p, int device = -1,
              bool grouped = false) {
  if (!d) return fail(NUMR_B200_EINVAL, "descriptor is NULL");
  const uint32_t ea = dtype_bytes(d->a_dtype), eb = dtype_bytes(d->b_dtype);
  if (!ea || !eb || is_wide_int(d->a_dtype) || is_wide_int(d->b_dtype))
    return fail(NUMR_B200_EUNSUPPORTED, "matmul: operand dtype %s x %s has no tensor-core kernel",
                dtype_name(d->a_dtype), dtype_name(d->b_dtype));
  if (d->a_dtype != d->b_dtype &&
      !(d->a_dtype == NUMR_B200_FP8E5M2 && d->b_dtype == NUMR_B200_FP8E4M3))
    return fail(NUMR_B200_EDTYPE, "matmul: dtype mismatch %s vs %s", dtype_name(d->a_dtype),
                dtype_name(d->b_dtype));
  if (d->b_layout != NUMR_B200_B_KN && d->b_layout != NUMR_B200_B_NK)
    return fail(NUMR_B200_EINVAL, "b_layout %d is not 0 ([K,N]) or 1 ([N,K])", d->b_layout);
  if (d->activation < 0 || (d->activation & ~NUMR_B200_ACT_BWD) > 5)
    return fail(NUMR_B200_EINVAL, "activation code %d is not in 0..5 (optionally + NUMR_B200_ACT_BWD)", d->activation);
  if (d->m > 0x7FFFFFFFu || d->n > 0x7FFFFFFFu || d->k > 0x7FFFFFFFu)
    return fail(NUMR_B200_EINVAL, "dimension exceeds 2^31-1");
  if (!grouped && d->batch > 0 && (d->a_batch == 0 || d->b_batch == 0 || d->a_batch > d->batch || d->b_batch > d->batch))
    return fail(NUMR_B200_EINVAL, "operand batch counts (%u, %u) must be in 1..batch (%u)", d->a_batch,
                d->b_batch, d->batch);

  p->elt = ea;
  p->split3 = false;
  p->f32 = false;
  switch (d->a_dtype) {
    case NUMR_B200_F32:
      if (d->f32_mode != NUMR_B200_F32_EXACT && d->f32_mode != NUMR_B200_F32_TF32)
        return fail(NUMR_B200_EINVAL, "f32_mode %d is not 0 (exact) or 1 (tf32)", d->f32_mode);
      p->kind = KIND_TF32; p->a_fmt = p->b_fmt = 2; p->f32 = true;
      p->split3 = d->f32_mode == NUMR_B200_F32_EXACT;
      if (d->out_dtype != NUMR_B200_F32)
        return fail(NUMR_B200_EDTYPE, "F32 matmul writes F32, not %s", dtype_name(d->out_dtype));
      p->out_kind = OUT_F32;
      break;
    case NUMR_B200_BF16:
      p->kind = KIND_F16; p->a_fmt = p->b_fmt = 1;
      if (d->out_dtype != NUMR_B200_BF16)
        return fail(NUMR_B200_EDTYPE, "BF16 matmul writes BF16, not %s", dtype_name(d->out_dtype));
      p->out_kind = OUT_BF16;
      break;
    case NUMR_B200_F16:
      p->kind = KIND_F16; p->a_fmt = p->b_fmt = 0;
      if (d->out_dtype != NUMR_B200_F16)
        return fail(NUMR_B200_EDTYPE, "F16 matmul writes F16, not %s", dtype_name(d->out_dtype));
      p->out_kind = OUT_F16;
      break;
    case NUMR_B200_FP8E4M3:
    case NUMR_B200_FP8E5M2:
      p->kind = KIND_F8F6F4;
      p->a_fmt = d->a_dtype == NUMR_B200_FP8E4M3 ? 0u : 1u;
      p->b_fmt = d->b_dtype == NUMR_B200_FP8E4M3 ? 0u : 1u;
      switch (d->out_dtype) {
        case NUMR_B200_F32: p->out_kind = OUT_F32; break;
        case NUMR_B200_BF16: p->out_kind = OUT_BF16; break;
        case NUMR_B200_F16: p->out_kind = OUT_F16; break;
        case NUMR_B200_FP8E4M3: p->out_kind = OUT_E4M3; break;
        case NUMR_B200_FP8E5M2: p->out_kind = OUT_E5M2; break;
        default:
          return fail(NUMR_B200_EUNSUPPORTED, "fp8_matmul: output dtype %s (F32, F16, BF16 or FP8 expected)",
                      dtype_name(d->out_dtype));
      }
      break;
    case NUMR_B200_I8:
      p->kind = KIND_I8; p->a_fmt = p->b_fmt = 1;
      if (d->out_dtype != NUMR_B200_I32)
        return fail(NUMR_B200_EDTYPE, "I8 x I8 matmul writes I32, not %s", dtype_name(d->out_dtype));
      p->out_kind = OUT_I32;
      if (d->activation != NUMR_B200_ACT_NONE)
        return fail(NUMR_B200_EUNSUPPORTED, "gemm epilogue: I8 is not supported with an activation");
      // (K > 131071, past the exact range of one s32 accumulator, is summed in 64 bits by the epilogue.)
      break;
    default:
      return fail(NUMR_B200_EUNSUPPORTED, "matmul: dtype %s", dtype_name(d->a_dtype));
  }

  // A: [a_batch][M][K]; B: [b_batch][K][N] or [b_batch][N][K].
  p->a.rows = d->m; p->a.cols = d->k;
  if (d->b_layout == NUMR_B200_B_KN) { p->b.rows = d->k; p->b.cols = d->n; }
  else { p->b.rows = d->n; p->b.cols = d->k; }

  size_t off = 0;
  const uint32_t parts = p->split3 ? 2u : 1u;
  const void* ptrs[2] = {a, b};
  OperandPlan* ops[2] = {&p->a, &p->b};
  const uint32_t batches[2] = {d->a_batch, d->b_batch};
  for (int i = 0; i < 2; ++i) {
    OperandPlan& o = *ops[i];
    const uint32_t per16 = 16 / p->elt;
    const bool aligned = (reinterpret_cast<uintptr_t>(ptrs[i]) & 15) == 0 && o.cols % per16 == 0;
    o.repack = p->f32 || !aligned;
    o.ld = o.repack ? (uint32_t)align_up(o.cols, per16) : o.cols;
    if (o.repack) {
      o.offset = off;
      o.bytes = (size_t)parts * batches[i] * o.rows * o.ld * p->elt;
      off = align_up(off + o.bytes, 256);
    }
  }
  p->required_bytes = off;
  // What the kernel itself wants for cutting the tiles of its last wave along K (device dependent:
  // it is a function of the SM count). Without a usable device this is 0.
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    device = -1;
  }
  if (!grouped && device >= 0 && d->batch && d->m && d->n && d->k) {
    GemmLaunch g;
    memset(&g, 0, sizeof(g));
    g.kind = p->kind; g.out_kind = p->out_kind; g.elt_bytes = p->elt;
    g.a_lo = p->split3 ? reinterpret_cast<const void*>(1) : nullptr;   // only "is exact mode" is read
    g.b_layout = d->b_layout;
    g.batch = d->batch; g.a_batch = d->a_batch; g.b_batch = d->b_batch;
    g.m = d->m; g.n = d->n; g.k = d->k;
    g.device_index = device;
    p->split_bytes = gemm_split_workspace_bytes(g);
    if (p->split_bytes) {
      p->split_off = off;
      off = align_up(off + p->split_bytes, 256);
    }
  }
  p->ws_bytes = off;
  return NUMR_B200_OK;
}

}  // namespace

// The device a call runs on: the calling thread's current device, which `device_index` (when not
// negative) must name. Every per-device cache (status word, scratch address, SM count, kernel
// attributes) is filled from the current device, so a mismatch would mix two GPUs' state.
int resolve_device(int device_index, int* dev_out) {
  int cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) {
    cudaGetLastError();
    return fail(NUMR_B200_ECUDA, "no CUDA device is available; this library has no CPU path");
  }
  if (device_index >= 0 && device_index != cur)
    return fail(NUMR_B200_EINVAL, "device_index %d is not the calling thread's current device (%d): make it current first",
                device_index, cur);
  *dev_out = cur;
  return NUMR_B200_OK;
}

}  // namespace nb

using namespace nb;

extern "C" {

const char* numr_b200_version(void) { return "numr_b200 0.1.0 (sm_100a)"; }

const char* numr_b200_last_error(void) { return t_error; }

// numr_b200_gemm for I16/I32/I64/U8/U16/U32/U64: validation, then the CUDA-core kernel.
static numr_b200_status gemm_wide_int(const numr_b200_gemm_desc* d, const void* a, const void* b,
                                      const void* bias, const void* residual, void* c, void* cu_stream,
                                      int device_index) {
  if (d->b_dtype != d->a_dtype)
    return (numr_b200_status)fail(NUMR_B200_EDTYPE, "matmul: dtype mismatch %s vs %s", dtype_name(d->a_dtype), dtype_name(d->b_dtype));
  if (d->out_dtype != d->a_dtype)
    return (numr_b200_status)fail(NUMR_B200_EDTYPE, "%s matmul writes %s, not %s", dtype_name(d->a_dtype), dtype_name(d->a_dtype), dtype_name(d->out_dtype));
  if (d->activation != NUMR_B200_ACT_NONE || residual)
    return (numr_b200_status)fail(NUMR_B200_EUNSUPPORTED, "gemm epilogue: %s has no activation / residual form", dtype_name(d->a_dtype));
  if (d->b_layout != NUMR_B200_B_KN && d->b_layout != NUMR_B200_B_NK)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "b_layout %d is not 0 ([K,N]) or 1 ([N,K])", d->b_layout);
  if (d->batch > 0 && (d->a_batch == 0 || d->b_batch == 0 || d->a_batch > d->batch || d->b_batch > d->batch))
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "operand batch counts (%u, %u) must be in 1..batch (%u)", d->a_batch, d->b_batch, d->batch);
  if (d->batch == 0 || d->m == 0 || d->n == 0) return NUMR_B200_OK;
  const uint32_t e = dtype_bytes(d->a_dtype);
  if (!c || reinterpret_cast<uintptr_t>(c) % e) return (numr_b200_status)fail(NUMR_B200_EINVAL, "output pointer is NULL or misaligned");
  if (d->k && (!a || !b || reinterpret_cast<uintptr_t>(a) % e || reinterpret_cast<uintptr_t>(b) % e))
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "operand pointer is NULL or not aligned to its element size %u", e);
  if (bias) {
    if (d->bias_dtype != d->a_dtype)
      return (numr_b200_status)fail(NUMR_B200_EDTYPE, "bias dtype %s, expected %s", dtype_name(d->bias_dtype), dtype_name(d->a_dtype));
    if (reinterpret_cast<uintptr_t>(bias) % e) return (numr_b200_status)fail(NUMR_B200_EINVAL, "bias pointer is misaligned");
  }
  int dev = 0;
  int dst = resolve_device(device_index, &dev);
  if (dst != NUMR_B200_OK) return (numr_b200_status)dst;
  return (numr_b200_status)launch_matmul_int(d->a_dtype, a, b, bias, c, d->batch, d->m, d->n, d->k, d->a_batch,
                                             d->b_batch, d->b_layout == NUMR_B200_B_NK,
                                             static_cast<cudaStream_t>(cu_stream));
}

size_t numr_b200_gemm_workspace_bytes(const numr_b200_gemm_desc* desc, const void* a, const void* b) {
  if (desc && is_wide_int(desc->a_dtype)) return 0;
  Plan p;
  if (make_plan(desc, a, b, &p) != NUMR_B200_OK) return 0;
  if (desc->k == 0 || desc->m == 0 || desc->n == 0 || desc->batch == 0) return 0;
  return p.ws_bytes;
}

// Row tiles a grouped problem can have at most: every group adds at most one partly filled tile.
static uint32_t group_plan_tiles(uint32_t total_rows, uint32_t groups) {
  return (total_rows + kTileM - 1) / kTileM + groups;
}
static size_t group_plan_bytes(uint32_t total_rows, uint32_t groups) {
  return align_up((size_t)group_plan_tiles(total_rows, groups) * sizeof(int4), 256);
}

// numr_b200_gemm, and (group_offsets != NULL) the grouped form: d->m = total rows of A, d->batch = 1,
// d->a_batch = 1, d->b_batch = groups; the plan sits at the front of the workspace.
struct GatherTarget {   // fused all-gather: every rank's [batch][M][world * N] buffer, and who we are
  const uint64_t* c_ptrs;
  uint32_t world, rank;
};

static numr_b200_status gemm_impl(const numr_b200_gemm_desc* d, const void* a, const void* b,
                                  const void* bias, const void* residual, void* c, void* workspace,
                                  size_t workspace_bytes, void* cu_stream, int device_index,
                                  const int32_t* group_offsets, const GatherTarget* gather = nullptr) {
  const bool grouped = group_offsets != nullptr;
  if (gather && d && is_wide_int(d->a_dtype))
    return (numr_b200_status)fail(NUMR_B200_EUNSUPPORTED, "gemm_allgather: dtype %s has no tensor-core kernel", dtype_name(d->a_dtype));
  if (d && is_wide_int(d->a_dtype)) {
    if (grouped) return (numr_b200_status)fail(NUMR_B200_EINVAL, "grouped matmul supports F32/F16/BF16, got %s", dtype_name(d->a_dtype));
    return gemm_wide_int(d, a, b, bias, residual, c, cu_stream, device_index);
  }
  Plan p;
  int dev = -1;
  int st = NUMR_B200_OK;
  if (d && d->batch && d->m && d->n) {   // (an empty problem launches nothing and needs no device)
    st = resolve_device(device_index, &dev);
    if (st == NUMR_B200_EINVAL) return (numr_b200_status)st;
    if (st != NUMR_B200_OK) dev = -1;    // reported below, after the argument checks
  }
  const int dev_status = st;
  st = make_plan(d, a, b, &p, dev, grouped);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  void* group_plan = nullptr;
  if (grouped && d->m && d->n && d->k) {
    const size_t pb = group_plan_bytes(d->m, d->b_batch);
    if (!workspace || workspace_bytes < pb + p.required_bytes)
      return (numr_b200_status)fail(NUMR_B200_EWORKSPACE, "workspace of %zu bytes needed, %zu given",
                                    pb + p.required_bytes, workspace ? workspace_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
      return (numr_b200_status)fail(NUMR_B200_EWORKSPACE, "workspace %p is not 256-byte aligned", workspace);
    group_plan = workspace;
    workspace = static_cast<char*>(workspace) + pb;
    workspace_bytes -= pb;
  }
  if (d->batch == 0 || d->m == 0 || d->n == 0) return NUMR_B200_OK;   // empty output: nothing to write
  if (!c) return (numr_b200_status)fail(NUMR_B200_EINVAL, "output pointer is NULL");

  static const uint32_t out_bytes[6] = {4, 2, 2, 1, 1, 4};
  const uint32_t ob = out_bytes[p.out_kind];
  if (reinterpret_cast<uintptr_t>(c) % ob)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "output pointer %p is not aligned to its element size %u", c, ob);
  if (bias) {
    const int want = d->a_dtype == NUMR_B200_I8 ? NUMR_B200_I32 : d->out_dtype;
    if (d->bias_dtype != want)
      return (numr_b200_status)fail(NUMR_B200_EDTYPE, "bias dtype %s, expected %s", dtype_name(d->bias_dtype), dtype_name(want));
    if (reinterpret_cast<uintptr_t>(bias) % ob)
      return (numr_b200_status)fail(NUMR_B200_EINVAL, "bias pointer %p is not aligned to its element size", bias);
  }
  if (residual) {
    if (d->a_dtype == NUMR_B200_I8)
      return (numr_b200_status)fail(NUMR_B200_EUNSUPPORTED, "gemm epilogue: I8 is not supported with a residual");
    if (reinterpret_cast<uintptr_t>(residual) % ob)
      return (numr_b200_status)fail(NUMR_B200_EINVAL, "residual pointer %p is not aligned to its element size", residual);
  }

  if (dev_status != NUMR_B200_OK)
    return (numr_b200_status)fail(NUMR_B200_ECUDA, "no CUDA device is available; this library has no CPU path");

  GemmLaunch g;
  memset(&g, 0, sizeof(g));
  g.kind = p.kind;
  g.out_kind = p.out_kind;
  g.elt_bytes = p.elt;
  g.a_fmt = p.a_fmt;
  g.b_fmt = p.b_fmt;
  g.b_layout = d->b_layout;
  g.batch = d->batch; g.a_batch = d->a_batch; g.b_batch = d->b_batch;
  g.m = d->m; g.n = d->n; g.k = d->k;
  g.bias = bias; g.residual = residual; g.out = c;
  g.scale = (p.kind == KIND_F8F6F4) ? d->scale_a * d->scale_b : 1.0f;
  g.activation = d->activation & ~NUMR_B200_ACT_BWD;
  g.epilogue_bwd = (d->activation & NUMR_B200_ACT_BWD) ? 1 : 0;
  if (g.epilogue_bwd && !residual)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "the backward epilogue multiplies by the incoming gradient: residual must not be NULL");
  g.stream = static_cast<cudaStream_t>(cu_stream);
  g.device_index = dev;

  if (gather) {
    // This rank's column block [rank * N, (rank + 1) * N) of every rank's [batch][M][world * N] buffer.
    if (d->k == 0) return (numr_b200_status)fail(NUMR_B200_EUNSUPPORTED, "gemm_allgather: K = 0");
    const size_t col_off = (size_t)gather->rank * d->n * ob;
    g.ldc = gather->world * d->n;
    uint32_t np = 0;
    for (uint32_t r = 0; r < gather->world; ++r) {
      char* base = reinterpret_cast<char*>(static_cast<uintptr_t>(gather->c_ptrs[r]));
      if (!base) return (numr_b200_status)fail(NUMR_B200_EINVAL, "gemm_allgather: buffer pointer of rank %u is NULL", r);
      if (r == gather->rank) g.out = base + col_off;
      else g.peer_out[np++] = base + col_off;
    }
    g.n_peer_out = np;
  }
  if (d->k == 0) return (numr_b200_status)launch_epilogue_only(g);   // (grouped: zeros / act(0) everywhere)

  if (!a || !b) return (numr_b200_status)fail(NUMR_B200_EINVAL, "operand pointer is NULL");
  if (reinterpret_cast<uintptr_t>(a) % p.elt || reinterpret_cast<uintptr_t>(b) % p.elt)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "operand pointer is not aligned to its element size %u", p.elt);

  // Small M against a transposed-B operand: bound by reading B once, served by a streaming kernel
  // (no operand preparation, no workspace).
  {
    g.a = a; g.b = b; g.lda = d->k; g.ldb = d->k;
    g.f32_exact = p.split3 ? 1 : 0;
    if (!grouped && !gather && !g.epilogue_bwd && !tuning().no_gemv && gemv_bt_applicable(g)) {
      const int r = launch_gemv_bt(g);
      if (r != -1) return (numr_b200_status)r;
    }
  }
  if (p.required_bytes) {
    if (!workspace || workspace_bytes < p.required_bytes)
      return (numr_b200_status)fail(NUMR_B200_EWORKSPACE, "workspace of %zu bytes needed, %zu given", p.required_bytes,
                  workspace ? workspace_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
      return (numr_b200_status)fail(NUMR_B200_EWORKSPACE, "workspace %p is not 256-byte aligned", workspace);
  }

  // Operand preparation (stream-ordered, into the caller's workspace).
  const void* srcs[2] = {a, b};
  OperandPlan* ops[2] = {&p.a, &p.b};
  const uint32_t batches[2] = {d->a_batch, d->b_batch};
  const void* use[2] = {a, b};
  const void* use_lo[2] = {nullptr, nullptr};
  if (p.f32 && p.a.repack && p.b.repack) {
    // both F32 operands in one launch
    char* da = static_cast<char*>(workspace) + p.a.offset;
    char* db = static_cast<char*>(workspace) + p.b.offset;
    const size_t ra = (size_t)d->a_batch * p.a.rows, rb = (size_t)d->b_batch * p.b.rows;
    float* a_hi = reinterpret_cast<float*>(da);
    float* b_hi = reinterpret_cast<float*>(db);
    float* a_lo = p.split3 ? a_hi + ra * p.a.ld : nullptr;
    float* b_lo = p.split3 ? b_hi + rb * p.b.ld : nullptr;
    st = launch_split_tf32_pair(static_cast<const float*>(a), a_hi, a_lo, ra, p.a.cols, p.a.ld,
                                static_cast<const float*>(b), b_hi, b_lo, rb, p.b.cols, p.b.ld, g.stream);
    if (st != NUMR_B200_OK) return (numr_b200_status)st;
    use[0] = da; use[1] = db;
    use_lo[0] = a_lo; use_lo[1] = b_lo;
  } else {
  for (int i = 0; i < 2; ++i) {
    OperandPlan& o = *ops[i];
    if (!o.repack) continue;
    char* dst = static_cast<char*>(workspace) + o.offset;
    const size_t rows = (size_t)batches[i] * o.rows;
    if (p.f32) {
      float* hi = reinterpret_cast<float*>(dst);
      float* lo = p.split3 ? hi + rows * o.ld : nullptr;
      st = launch_split_tf32(static_cast<const float*>(srcs[i]), hi, lo, rows, o.cols, o.cols, o.ld, g.stream);
      use_lo[i] = lo;
    } else {
      st = launch_pad_rows(srcs[i], dst, rows, o.cols * p.elt, (size_t)o.cols * p.elt, o.ld * p.elt, g.stream);
    }
    if (st != NUMR_B200_OK) return (numr_b200_status)st;
    use[i] = dst;
  }
  }
  g.a = use[0]; g.b = use[1];
  g.a_lo = use_lo[0]; g.b_lo = use_lo[1];
  g.lda = p.a.ld; g.ldb = p.b.ld;
  // The K-split scratch is optional: without room for it the last wave runs whole tiles.
  if (p.split_bytes && workspace && workspace_bytes >= p.ws_bytes && !(reinterpret_cast<uintptr_t>(workspace) & 255)) {
    g.split_ws = static_cast<char*>(workspace) + p.split_off;
    g.split_ws_bytes = p.split_bytes;
  }
  if (grouped) {   // the launcher builds the tile plan once it has chosen the tile height
    g.group_offsets = group_offsets;
    g.groups = d->b_batch;
    g.group_plan = group_plan;
  }
  return (numr_b200_status)launch_gemm_sm100(g);
}

numr_b200_status numr_b200_gemm(const numr_b200_gemm_desc* d, const void* a, const void* b,
                                const void* bias, const void* residual, void* c, void* workspace,
                                size_t workspace_bytes, void* cu_stream, int device_index) {
  return gemm_impl(d, a, b, bias, residual, c, workspace, workspace_bytes, cu_stream, device_index, nullptr);
}

numr_b200_status numr_b200_gemm_allgather(const numr_b200_gemm_desc* d, const void* a, const void* b,
                                          const void* bias, const void* residual, const uint64_t* c_ptrs,
                                          uint32_t world, uint32_t rank, void* workspace, size_t workspace_bytes,
                                          void* cu_stream, int device_index) {
  if (!c_ptrs) return (numr_b200_status)fail(NUMR_B200_EINVAL, "gemm_allgather: c_ptrs is NULL");
  if (world == 0 || world > 8 || rank >= world)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "gemm_allgather: rank %u of %u (1 to 8 ranks)", rank, world);
  GatherTarget t{c_ptrs, world, rank};
  void* own = reinterpret_cast<void*>(static_cast<uintptr_t>(c_ptrs[rank]));
  return gemm_impl(d, a, b, bias, residual, own, workspace, workspace_bytes, cu_stream, device_index, nullptr, &t);
}

// Checks shared by the grouped entry points: the descriptor describes A [m, k] and `groups` matrices
// B [k, n] (or [n, k]); F32 / F16 / BF16 only, no bias, no residual (src/ops/cpu/grouped_matmul.rs:13-75).
static int check_grouped(const numr_b200_gemm_desc* d, uint32_t groups) {
  if (!d) return fail(NUMR_B200_EINVAL, "descriptor is NULL");
  if (d->a_dtype != d->b_dtype)
    return fail(NUMR_B200_EINVAL, "grouped matmul: a is %s but b is %s", dtype_name(d->a_dtype), dtype_name(d->b_dtype));
  if (d->a_dtype != NUMR_B200_F32 && d->a_dtype != NUMR_B200_F16 && d->a_dtype != NUMR_B200_BF16)
    return fail(NUMR_B200_EINVAL, "grouped matmul supports F32/F16/BF16, got %s", dtype_name(d->a_dtype));
  if (d->batch != 1 || d->a_batch != 1 || d->b_batch != groups)
    return fail(NUMR_B200_EINVAL, "grouped matmul: descriptor must have batch = 1, a_batch = 1, b_batch = groups (%u)", groups);
  return NUMR_B200_OK;
}

size_t numr_b200_grouped_gemm_workspace_bytes(const numr_b200_gemm_desc* d, uint32_t groups, const void* a,
                                              const void* b) {
  if (check_grouped(d, groups) != NUMR_B200_OK) return 0;
  Plan p;
  if (make_plan(d, a, b, &p, -1, true) != NUMR_B200_OK) return 0;
  if (d->m == 0 || d->n == 0 || d->k == 0) return 0;
  return group_plan_bytes(d->m, groups) + p.required_bytes;
}

numr_b200_status numr_b200_grouped_gemm(const numr_b200_gemm_desc* d, uint32_t groups, const void* a,
                                        const void* b, const int32_t* group_offsets, void* c, void* workspace,
                                        size_t workspace_bytes, void* cu_stream, int device_index) {
  int st = check_grouped(d, groups);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (d->m == 0 || d->n == 0) return NUMR_B200_OK;
  if (groups == 0) {
    // no group, no product: the output is all zeros, as numr's CPU path returns
    // (src/ops/cpu/grouped_matmul.rs:86-92)
    if (!c) return (numr_b200_status)fail(NUMR_B200_EINVAL, "output pointer is NULL");
    cudaError_t e = cudaMemsetAsync(c, 0, (size_t)d->m * d->n * dtype_bytes(d->out_dtype), static_cast<cudaStream_t>(cu_stream));
    if (e != cudaSuccess) return (numr_b200_status)fail(NUMR_B200_ECUDA, "clearing the output failed: %s", cudaGetErrorString(e));
    return NUMR_B200_OK;
  }
  if (!group_offsets) return (numr_b200_status)fail(NUMR_B200_EINVAL, "group_offsets pointer is NULL");
  if (reinterpret_cast<uintptr_t>(group_offsets) & 3)
    return (numr_b200_status)fail(NUMR_B200_EINVAL, "group_offsets pointer is not 4-byte aligned");
  return gemm_impl(d, a, b, nullptr, nullptr, c, workspace, workspace_bytes, cu_stream, device_index, group_offsets);
}

void numr_b200_reload_tuning(void) { reload_tuning(); }

numr_b200_status numr_b200_device_status(int* kernel_status) {
  return (numr_b200_status)read_and_clear_device_status(kernel_status);
}

size_t numr_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

numr_b200_status numr_b200_gemm_static_scratch(const numr_b200_gemm_desc* d, const void* a, const void* b,
                                               const void* bias, const void* residual, void* c,
                                               void* cu_stream, int device_index) {
  // The integer widths served by the CUDA cores use no scratch at all: same call as numr_b200_gemm.
  if (d && is_wide_int(d->a_dtype))
    return numr_b200_gemm(d, a, b, bias, residual, c, nullptr, 0, cu_stream, device_index);
  // The scratch address below belongs to the current device; a device_index naming another one
  // would pair this GPU's scratch with that GPU's launch state.
  int dev = 0;
  if (d && d->batch && d->m && d->n) {
    int dst = resolve_device(device_index, &dev);
    if (dst == NUMR_B200_EINVAL) return (numr_b200_status)dst;
  }
  Plan p;
  int st = make_plan(d, a, b, &p);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  const bool empty = d->batch == 0 || d->m == 0 || d->n == 0 || d->k == 0;
  const size_t need = empty ? 0 : p.required_bytes;
  if (need > kStaticScratchBytes)
    return (numr_b200_status)fail(
        NUMR_B200_EWORKSPACE,
        "gemm_static_scratch: this problem needs %zu bytes of scratch, the built-in scratch holds %zu; "
        "use numr_b200_gemm with a caller-provided workspace",
        need, kStaticScratchBytes);
  void* scratch = nullptr;
  if (need) {
    scratch = static_scratch_address();
    if (!scratch) return NUMR_B200_ECUDA;
  }
  // (The optional K-split scratch is used too when it fits beside the required part.)
  if (!scratch && !empty && p.ws_bytes && p.ws_bytes <= kStaticScratchBytes) scratch = static_scratch_address();
  return numr_b200_gemm(d, a, b, bias, residual, c, scratch, scratch ? kStaticScratchBytes : 0, cu_stream,
                        device_index);
}

numr_b200_status numr_b200_init(int device_index) {
  int dev = 0;
  int st = resolve_device(device_index, &dev);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  (void)tuning();
  st = init_gemm_device(dev);
  if (st != NUMR_B200_OK) return (numr_b200_status)st;
  if (!device_status_ptr()) return (numr_b200_status)fail(NUMR_B200_ECUDA, "cannot resolve the device status word");
  if (!static_scratch_address()) return NUMR_B200_ECUDA;
  return NUMR_B200_OK;
}

// ------------------------------------------------------------------ launcher mirrors
static numr_b200_gemm_desc plain_desc(int32_t dtype, size_t batch, size_t m, size_t n, size_t k,
                                      size_t a_batch, size_t b_batch) {
  numr_b200_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.a_dtype = d.b_dtype = dtype;
  d.out_dtype = (dtype == NUMR_B200_I8) ? NUMR_B200_I32 : dtype;
  d.bias_dtype = d.out_dtype;
  d.batch = (uint32_t)batch; d.m = (uint32_t)m; d.n = (uint32_t)n; d.k = (uint32_t)k;
  d.a_batch = (uint32_t)a_batch; d.b_batch = (uint32_t)b_batch;
  d.b_layout = NUMR_B200_B_KN;
  d.activation = NUMR_B200_ACT_NONE;
  d.f32_mode = NUMR_B200_F32_EXACT;
  d.scale_a = d.scale_b = 1.0f;
  return d;
}

static bool dims_fit(size_t batch, size_t m, size_t n, size_t k) {
  const size_t lim = 0x7FFFFFFFull;
  if (batch > lim || m > lim || n > lim || k > lim) {
    set_error("dimension exceeds 2^31-1");
    return false;
  }
  return true;
}

#define PTR(x) reinterpret_cast<void*>(static_cast<uintptr_t>(x))

numr_b200_status numr_b200_launch_matmul_kernel(void* s, int dev, int32_t dtype, uint64_t a, uint64_t b,
                                                uint64_t c, size_t m, size_t n, size_t k, void* ws,
                                                size_t wsb) {
  if (!dims_fit(1, m, n, k)) return NUMR_B200_EINVAL;
  numr_b200_gemm_desc d = plain_desc(dtype, 1, m, n, k, 1, 1);
  return numr_b200_gemm(&d, PTR(a), PTR(b), nullptr, nullptr, PTR(c), ws, wsb, s, dev);
}

numr_b200_status numr_b200_launch_matmul_batched_kernel(void* s, int dev, int32_t dtype, uint64_t a,
                                                        uint64_t b, uint64_t c, size_t batch, size_t m,
                                                        size_t n, size_t k, size_t a_batch,
                                                        size_t b_batch, void* ws, size_t wsb) {
  if (!dims_fit(batch, m, n, k)) return NUMR_B200_EINVAL;
  numr_b200_gemm_desc d = plain_desc(dtype, batch, m, n, k, a_batch, b_batch);
  return numr_b200_gemm(&d, PTR(a), PTR(b), nullptr, nullptr, PTR(c), ws, wsb, s, dev);
}

numr_b200_status numr_b200_launch_matmul_bias_kernel(void* s, int dev, int32_t dtype, uint64_t a,
                                                     uint64_t b, uint64_t bias, uint64_t c, size_t m,
                                                     size_t n, size_t k, void* ws, size_t wsb) {
  if (!dims_fit(1, m, n, k)) return NUMR_B200_EINVAL;
  if (!bias) { set_error("matmul_bias: bias pointer is NULL"); return NUMR_B200_EINVAL; }
  numr_b200_gemm_desc d = plain_desc(dtype, 1, m, n, k, 1, 1);
  return numr_b200_gemm(&d, PTR(a), PTR(b), PTR(bias), nullptr, PTR(c), ws, wsb, s, dev);
}

numr_b200_status numr_b200_launch_matmul_bias_batched_kernel(void* s, int dev, int32_t dtype, uint64_t a,
                                                             uint64_t b, uint64_t bias, uint64_t c,
                                                             size_t batch, size_t m, size_t n, size_t k,
                                                             size_t a_batch, size_t b_batch, void* ws,
                                                             size_t wsb) {
  if (!dims_fit(batch, m, n, k)) return NUMR_B200_EINVAL;
  if (!bias) { set_error("matmul_bias: bias pointer is NULL"); return NUMR_B200_EINVAL; }
  numr_b200_gemm_desc d = plain_desc(dtype, batch, m, n, k, a_batch, b_batch);
  return numr_b200_gemm(&d, PTR(a), PTR(b), PTR(bias), nullptr, PTR(c), ws, wsb, s, dev);
}

numr_b200_status numr_b200_launch_gemm_bias_act_kernel(void* s, int dev, int32_t dtype, uint64_t a,
                                                       uint64_t b, uint64_t bias, uint64_t c, size_t m,
                                                       size_t n, size_t k, int32_t activation, void* ws,
                                                       size_t wsb) {
  return numr_b200_launch_gemm_bias_act_batched_kernel(s, dev, dtype, a, b, bias, c, 1, m, n, k,
                                                       activation, ws, wsb);
}

numr_b200_status numr_b200_launch_gemm_bias_act_batched_kernel(void* s, int dev, int32_t dtype,
                                                               uint64_t a, uint64_t b, uint64_t bias,
                                                               uint64_t c, size_t batch, size_t m,
                                                               size_t n, size_t k, int32_t activation,
                                                               void* ws, size_t wsb) {
  if (!dims_fit(batch, m, n, k)) return NUMR_B200_EINVAL;
  if (dtype == NUMR_B200_I8) {
    set_error("gemm_bias_act: I8 is not supported (the epilogue ops reject I8)");
    return NUMR_B200_EUNSUPPORTED;
  }
  if (!bias) { set_error("gemm_bias_act: bias pointer is NULL"); return NUMR_B200_EINVAL; }
  numr_b200_gemm_desc d = plain_desc(dtype, batch, m, n, k, batch, batch);
  d.activation = activation;
  return numr_b200_gemm(&d, PTR(a), PTR(b), PTR(bias), nullptr, PTR(c), ws, wsb, s, dev);
}

numr_b200_status numr_b200_launch_gemm_bias_residual_kernel(void* s, int dev, int32_t dtype, uint64_t a,
                                                            uint64_t b, uint64_t bias, uint64_t residual,
                                                            uint64_t c, size_t m, size_t n, size_t k,
                                                            void* ws, size_t wsb) {
  return numr_b200_launch_gemm_bias_residual_batched_kernel(s, dev, dtype, a, b, bias, residual, c, 1, m,
                                                            n, k, ws, wsb);
}

numr_b200_status numr_b200_launch_gemm_bias_residual_batched_kernel(
    void* s, int dev, int32_t dtype, uint64_t a, uint64_t b, uint64_t bias, uint64_t residual, uint64_t c,
    size_t batch, size_t m, size_t n, size_t k, void* ws, size_t wsb) {
  if (!dims_fit(batch, m, n, k)) return NUMR_B200_EINVAL;
  if (dtype == NUMR_B200_I8) {
    set_error("gemm_bias_residual: I8 is not supported (the epilogue ops reject I8)");
    return NUMR_B200_EUNSUPPORTED;
  }
  if (!bias || !residual) { set_error("gemm_bias_residual: bias or residual pointer is NULL"); return NUMR_B200_EINVAL; }
  numr_b200_gemm_desc d = plain_desc(dtype, batch, m, n, k, batch, batch);
  return numr_b200_gemm(&d, PTR(a), PTR(b), PTR(bias), PTR(residual), PTR(c), ws, wsb, s, dev);
}

static numr_b200_status fp8_launch(void* s, int dev, int32_t a_dtype, int32_t out_dtype, uint64_t a,
                                   uint64_t b, uint64_t out, float sa, float sb, size_t batch, size_t m,
                                   size_t n, size_t k, void* ws, size_t wsb) {
  if (!dims_fit(batch, m, n, k)) return NUMR_B200_EINVAL;
  if (out_dtype != NUMR_B200_F32 && out_dtype != NUMR_B200_F16 && out_dtype != NUMR_B200_BF16) {
    set_error("fp8_matmul: output dtype must be F32, F16 or BF16");
    return NUMR_B200_EUNSUPPORTED;
  }
  numr_b200_gemm_desc d = plain_desc(NUMR_B200_FP8E4M3, batch, m, n, k, batch, batch);
  d.a_dtype = a_dtype;
  d.out_dtype = d.bias_dtype = out_dtype;
  d.scale_a = sa;
  d.scale_b = sb;
  return numr_b200_gemm(&d, PTR(a), PTR(b), nullptr, nullptr, PTR(out), ws, wsb, s, dev);
}

numr_b200_status numr_b200_launch_fp8_matmul_e4m3(void* s, int dev, int32_t out_dtype, uint64_t a,
                                                  uint64_t b, uint64_t out, float sa, float sb,
                                                  size_t batch, size_t m, size_t n, size_t k, void* ws,
                                                  size_t wsb) {
  return fp8_launch(s, dev, NUMR_B200_FP8E4M3, out_dtype, a, b, out, sa, sb, batch, m, n, k, ws, wsb);
}

numr_b200_status numr_b200_launch_fp8_matmul_e5m2(void* s, int dev, int32_t out_dtype, uint64_t a,
                                                  uint64_t b, uint64_t out, float sa, float sb,
                                                  size_t batch, size_t m, size_t n, size_t k, void* ws,
                                                  size_t wsb) {
  return fp8_launch(s, dev, NUMR_B200_FP8E5M2, out_dtype, a, b, out, sa, sb, batch, m, n, k, ws, wsb);
}

}  // extern "C"
