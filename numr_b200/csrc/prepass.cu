// HBM-bound helper kernels around the tcgen05 GEMM: operand preparation that TMA and
// the TF32 tensor cores need, and the K == 0 epilogue.
//   split_tf32      f32 -> TF32-rounded high part (+ optional low part) with a padded pitch
//   pad_rows        re-pitch an operand whose address or row pitch is not 16-byte aligned
//   gather_strided  materialise a non-contiguous view (the reference's ensure_contiguous,
//                   src/runtime/cuda/ops/helpers/matmul.rs:91-92)
//   group_plan      grouped GEMM: row tiles of every group from the device-side offsets
//   epilogue_only   out = cast(act(bias) + residual): what the reference kernels write when
//                   K == 0 (matmul_f32_tiled.cuh:261-265, matmul_wmma.cuh:331-334)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "epilogue_math.cuh"
#include "gemm_internal.h"

namespace nb {

namespace {

constexpr int kThreads = 256;

inline uint32_t grid_for(size_t work, int sm_multiple = 148 * 8) {
  size_t blocks = (work + kThreads - 1) / kThreads;
  if (blocks > (size_t)sm_multiple) blocks = sm_multiple;   // grid-stride beyond that
  if (blocks == 0) blocks = 1;
  return (uint32_t)blocks;
}

// Lets the kernel after this one in the stream (a GEMM launched as a programmatic dependent launch)
// begin its set-up; it still waits for this kernel to complete before it reads anything.
__device__ __forceinline__ void let_next_kernel_set_up() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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

__global__ void split_tf32_kernel(const float* __restrict__ in, float* __restrict__ hi,
                                  float* __restrict__ lo, size_t rows, uint32_t cols, size_t ld_in,
                                  uint32_t ld_out) {
  let_next_kernel_set_up();
  const size_t total = rows * ld_out;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / ld_out;
    const uint32_t c = (uint32_t)(i - r * ld_out);
    float x = 0.0f;
    if (c < cols) x = in[r * ld_in + c];
    const float h = tf32_high(x);
    hi[i] = h;
    if (lo) {
      // x - h is exact in f32; for non-finite x the low part carries nothing.
      const float d = x - h;
      lo[i] = (isfinite(x) && isfinite(h)) ? round_tf32(d) : 0.0f;
    }
  }
}

// Both F32 operands of one GEMM in a single launch (the second operand's elements follow the first's
// in the index space): one launch less per F32 matmul.
struct SplitOperand {
  const float* in;
  float* hi;
  float* lo;
  size_t rows, ld_in;
  uint32_t cols, ld_out;
};

__global__ void split_tf32_pair_kernel(SplitOperand a, SplitOperand b) {
  let_next_kernel_set_up();
  const size_t total_a = a.rows * a.ld_out, total = total_a + b.rows * b.ld_out;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const bool first = i < total_a;
    const SplitOperand& o = first ? a : b;
    const size_t j = first ? i : i - total_a;
    const size_t r = j / o.ld_out;
    const uint32_t c = (uint32_t)(j - r * o.ld_out);
    float x = 0.0f;
    if (c < o.cols) x = o.in[r * o.ld_in + c];
    const float h = tf32_high(x);
    o.hi[j] = h;
    if (o.lo) {
      const float d = x - h;
      o.lo[j] = (isfinite(x) && isfinite(h)) ? round_tf32(d) : 0.0f;
    }
  }
}

__global__ void pad_rows_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                size_t rows, uint32_t row_bytes, size_t in_pitch, uint32_t out_pitch) {
  let_next_kernel_set_up();
  const size_t total = rows * out_pitch;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / out_pitch;
    const uint32_t c = (uint32_t)(i - r * out_pitch);
    out[i] = c < row_bytes ? in[r * in_pitch + c] : (uint8_t)0;
  }
}

struct GatherDims {
  int ndim;
  long long shape[8];
  long long strides[8];
};

template <typename T>
__global__ void gather_kernel(const T* __restrict__ in, T* __restrict__ out, GatherDims d, size_t total) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    size_t rem = i;
    long long off = 0;
    for (int k = d.ndim - 1; k >= 0; --k) {
      const long long s = d.shape[k];
      const long long c = (long long)(rem % (size_t)s);
      rem /= (size_t)s;
      off += c * d.strides[k];
    }
    out[i] = in[off];
  }
}

template <int OUT>
__global__ void epilogue_only_kernel(const void* __restrict__ bias_v, const void* __restrict__ res_v,
                                     void* __restrict__ out_v, size_t total, uint32_t n, int act, int bwd) {
  using T = decltype(from_f32<OUT>(0.0f));
  const T* bias = static_cast<const T*>(bias_v);
  const T* res = static_cast<const T*>(res_v);
  T* out = static_cast<T*>(out_v);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t col = (uint32_t)(i % n);
    float x = 0.0f;
    if (bias) x += load_f32<OUT>(bias, col);
    if (bwd) {
      x = (res ? to_f32<OUT>(res[i]) : 0.0f) * apply_activation_derivative(x, act);
    } else {
      x = apply_activation(x, act);
      if (res) x += to_f32<OUT>(res[i]);
    }
    out[i] = from_f32<OUT>(x);
  }
}

__global__ void epilogue_only_i32_kernel(const int32_t* __restrict__ bias, int32_t* __restrict__ out,
                                         size_t total, uint32_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = finish_i32(0u, bias, (uint32_t)(i % n));
}

// One warp walks the groups in order (their row-tile counts are a running sum); lanes write the
// tiles of a group in parallel. Tiles lie on the ABSOLUTE row grid (multiples of tile_rows): a group
// [start, end) gets the grid tiles it overlaps, each with the rows of the group it covers, so a tile
// at a group boundary appears once per group it touches. (With tile origins at arbitrary rows the
// TMA row coordinates are not multiples of the tile height, and that measured 30 - 70 % slower.)
// Entry = {group | band size << 24, first row kept, end of the rows kept, first tile of the band}:
// a band is up to `band_tiles` consecutive row tiles of ONE group; the GEMM walks a band column by
// column before it moves on, so one group's weight and the band's rows of A stay in L2.
__global__ void group_plan_kernel(const int32_t* __restrict__ offsets, uint32_t groups, uint32_t total_rows,
                                  int4* __restrict__ plan, uint32_t plan_tiles, uint32_t tile_rows,
                                  uint32_t band_tiles) {
  let_next_kernel_set_up();
  const uint32_t lane = threadIdx.x;
  uint32_t next = 0;
  for (uint32_t g = 0; g < groups; ++g) {
    const int start = max(offsets[g], 0), end = max(offsets[g + 1], 0);
    if (end <= start || (uint32_t)end > total_rows) continue;
    const uint32_t j0 = (uint32_t)start / tile_rows, j1 = ((uint32_t)end - 1) / tile_rows;
    const uint32_t tiles = j1 - j0 + 1;
    for (uint32_t t = lane; t < tiles; t += 32)
      if (next + t < plan_tiles) {
        const uint32_t b0 = t / band_tiles * band_tiles;
        const uint32_t bs = min(band_tiles, tiles - b0);
        const uint32_t lo = max((uint32_t)start, (j0 + t) * tile_rows);
        const uint32_t hi = min((uint32_t)end, (j0 + t + 1) * tile_rows);
        plan[next + t] = make_int4((int)(g | (bs << 24)), (int)lo, (int)hi, (int)(next + b0));
      }
    next += tiles;
  }
  for (uint32_t t = next + lane; t < plan_tiles; t += 32) plan[t] = make_int4(1 << 24, 0, 0, (int)t);   // unused: a band of its own
}

// Column sums of a row-major [rows, n] matrix in f32, rounded once: block = 32 columns x 8 row
// lanes, fixed summation order (deterministic). d_bias of the backward GEMM epilogue.
template <int OUT>
__global__ void column_sums_kernel(const void* __restrict__ in_v, void* __restrict__ out_v, size_t rows, uint32_t n) {
  using T = decltype(from_f32<OUT>(0.0f));
  const T* in = static_cast<const T*>(in_v);
  T* out = static_cast<T*>(out_v);
  __shared__ float part[8][33];
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const uint32_t col = blockIdx.x * 32 + tx;
  float s = 0.0f;
  if (col < n)
    for (size_t r = ty; r < rows; r += 8) s += to_f32<OUT>(in[r * n + col]);
  part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && col < n) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += part[i][tx];
    out[col] = from_f32<OUT>(t);
  }
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(NUMR_B200_ECUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  return NUMR_B200_OK;
}

}  // namespace

int launch_split_tf32(const float* in, float* hi, float* lo, size_t rows, uint32_t cols, size_t ld_in,
                      uint32_t ld_out, cudaStream_t stream) {
  const size_t total = rows * ld_out;
  if (total == 0) return NUMR_B200_OK;
  split_tf32_kernel<<<grid_for(total), kThreads, 0, stream>>>(in, hi, lo, rows, cols, ld_in, ld_out);
  return check_launch("split_tf32");
}

int launch_split_tf32_pair(const float* a_in, float* a_hi, float* a_lo, size_t a_rows, uint32_t a_cols, uint32_t a_ld,
                           const float* b_in, float* b_hi, float* b_lo, size_t b_rows, uint32_t b_cols, uint32_t b_ld,
                           cudaStream_t stream) {
  const size_t total = a_rows * a_ld + b_rows * b_ld;
  if (total == 0) return NUMR_B200_OK;
  SplitOperand a{a_in, a_hi, a_lo, a_rows, a_cols, a_cols, a_ld};
  SplitOperand b{b_in, b_hi, b_lo, b_rows, b_cols, b_cols, b_ld};
  split_tf32_pair_kernel<<<grid_for(total), kThreads, 0, stream>>>(a, b);
  return check_launch("split_tf32_pair");
}

int launch_pad_rows(const void* in, void* out, size_t rows, uint32_t row_bytes, size_t in_pitch,
                    uint32_t out_pitch, cudaStream_t stream) {
  const size_t total = rows * out_pitch;
  if (total == 0) return NUMR_B200_OK;
  pad_rows_kernel<<<grid_for(total), kThreads, 0, stream>>>(
      static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), rows, row_bytes, in_pitch, out_pitch);
  return check_launch("pad_rows");
}

int launch_gather_strided(const void* in, void* out, int ndim, const int64_t* shape,
                          const int64_t* strides, uint32_t elt_bytes, cudaStream_t stream) {
  if (ndim < 0 || ndim > 8) return fail(NUMR_B200_EINVAL, "gather: ndim %d out of range", ndim);
  GatherDims d;
  d.ndim = ndim;
  size_t total = 1;
  for (int i = 0; i < ndim; ++i) {
    d.shape[i] = shape[i];
    d.strides[i] = strides[i];
    total *= (size_t)shape[i];
  }
  if (total == 0) return NUMR_B200_OK;
  const uint32_t grid = grid_for(total);
  switch (elt_bytes) {
    case 1: gather_kernel<uint8_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), d, total); break;
    case 2: gather_kernel<uint16_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), d, total); break;
    case 4: gather_kernel<uint32_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), d, total); break;
    case 8: gather_kernel<uint64_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out), d, total); break;
    default: return fail(NUMR_B200_EINVAL, "gather: element size %u not supported", elt_bytes);
  }
  return check_launch("gather_strided");
}

int launch_group_plan(const int32_t* offsets, uint32_t groups, uint32_t total_rows, void* plan,
                      uint32_t plan_tiles, uint32_t tile_rows, uint32_t band_tiles, cudaStream_t stream) {
  if (plan_tiles == 0) return NUMR_B200_OK;
  if (groups >= (1u << 24)) return fail(NUMR_B200_EINVAL, "grouped matmul: more than 2^24 - 1 groups");
  band_tiles = band_tiles < 1 ? 1 : (band_tiles > 255 ? 255 : band_tiles);
  group_plan_kernel<<<1, 32, 0, stream>>>(offsets, groups, total_rows, static_cast<int4*>(plan), plan_tiles, tile_rows,
                                          band_tiles);
  return check_launch("group_plan");
}

int launch_column_sums(int out_kind, const void* in, void* out, size_t rows, uint32_t n, cudaStream_t stream) {
  if (n == 0) return NUMR_B200_OK;
  const uint32_t grid = (n + 31) / 32;
  switch (out_kind) {
    case OUT_F32: column_sums_kernel<OUT_F32><<<grid, 256, 0, stream>>>(in, out, rows, n); break;
    case OUT_BF16: column_sums_kernel<OUT_BF16><<<grid, 256, 0, stream>>>(in, out, rows, n); break;
    case OUT_F16: column_sums_kernel<OUT_F16><<<grid, 256, 0, stream>>>(in, out, rows, n); break;
    default: return fail(NUMR_B200_EUNSUPPORTED, "column_sums: output kind %d", out_kind);
  }
  return check_launch("column_sums");
}

int launch_epilogue_only(const GemmLaunch& g) {
  const size_t total = (size_t)g.batch * g.m * g.n;
  if (total == 0) return NUMR_B200_OK;
  const uint32_t grid = grid_for(total);
  switch (g.out_kind) {
    case OUT_F32: epilogue_only_kernel<OUT_F32><<<grid, kThreads, 0, g.stream>>>(g.bias, g.residual, g.out, total, g.n, g.activation, g.epilogue_bwd); break;
    case OUT_BF16: epilogue_only_kernel<OUT_BF16><<<grid, kThreads, 0, g.stream>>>(g.bias, g.residual, g.out, total, g.n, g.activation, g.epilogue_bwd); break;
    case OUT_F16: epilogue_only_kernel<OUT_F16><<<grid, kThreads, 0, g.stream>>>(g.bias, g.residual, g.out, total, g.n, g.activation, g.epilogue_bwd); break;
    case OUT_E4M3: epilogue_only_kernel<OUT_E4M3><<<grid, kThreads, 0, g.stream>>>(g.bias, g.residual, g.out, total, g.n, g.activation, g.epilogue_bwd); break;
    case OUT_E5M2: epilogue_only_kernel<OUT_E5M2><<<grid, kThreads, 0, g.stream>>>(g.bias, g.residual, g.out, total, g.n, g.activation, g.epilogue_bwd); break;
    case OUT_I32: epilogue_only_i32_kernel<<<grid, kThreads, 0, g.stream>>>(static_cast<const int32_t*>(g.bias), static_cast<int32_t*>(g.out), total, g.n); break;
    default: return fail(NUMR_B200_EUNSUPPORTED, "epilogue_only: output kind %d", g.out_kind);
  }
  return check_launch("epilogue_only");
}

}  // namespace nb
