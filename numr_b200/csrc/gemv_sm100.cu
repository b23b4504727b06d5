// Small-M matmul against a transposed-B operand: C[M,N] = A[M,K] . W[N,K]^T (kernels for M <= 16;
// the dispatch below uses them for M = 1, and for exact F32 up to M = 8).
//
// With so few rows the product is bound by reading W once from HBM, not by the tensor cores
// (whose 128-row tiles would be almost empty and whose K loop is a serial chain). This kernel
// streams W with 16-byte loads, keeps all M partial sums of a W row in registers, and reduces
// across the lanes of a warp in a fixed order, so results are bitwise reproducible.
//   - one warp owns 4 rows of W (4 output columns); lanes split K in 16-byte steps
//   - A (at most 16 x K) is re-read by every warp and stays in L1/L2
//   - accumulation in f32 (exact int32 for I8, inside the same K bound as the tensor-core path)
//   - the fused epilogue (scale, bias, activation, residual, one conversion) runs on the
//     reducing lane
// It takes the place of the reference's gemv_bt kernels (src/runtime/cuda/kernels/gemv.cu:27-574,
// routed for m <= 16 with a transposed B at src/runtime/cuda/ops/helpers/matmul.rs:66-89).
#include <algorithm>
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "epilogue_math.cuh"
#include "gemm_internal.h"
#include "sm100_ptx.cuh"

namespace nb {
namespace {

constexpr int kRowsPerWarp = 4;
constexpr int kWarps = 8;

struct GemvParams {
  const void* a;
  const void* w;
  const void* bias;
  const void* residual;
  void* out;
  uint32_t m, n, k;
  uint32_t a_batch, b_batch;
  float scale;
  int act;
};

// Operand element kinds and their widening to f32 (exact for every type here).
enum InKind : int { IN_F32 = 0, IN_BF16 = 1, IN_F16 = 2, IN_E4M3 = 3, IN_E5M2 = 4, IN_I8 = 5 };

template <int IN> struct InBytes { static constexpr int v = IN == IN_F32 ? 4 : (IN == IN_BF16 || IN == IN_F16) ? 2 : 1; };

// Widens the 16 bytes in `v` to VEC f32 values (int32 values, bit-cast, for I8).
template <int IN>
__device__ __forceinline__ void widen16(const uint4& v, float* out) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if constexpr (IN == IN_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = __uint_as_float(w[i]);
  } else if constexpr (IN == IN_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else if constexpr (IN == IN_F16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint8_t byte = (uint8_t)(w[i] >> (8 * b));
        if constexpr (IN == IN_E4M3) out[4 * i + b] = e4m3_to_f32(byte);
        else if constexpr (IN == IN_E5M2) out[4 * i + b] = e5m2_to_f32(byte);
        else out[4 * i + b] = __int_as_float((int)(int8_t)byte);
      }
  }
}

template <int IN_A, int IN_W, int OUT, int MT>
__global__ void __launch_bounds__(kWarps * 32) gemv_bt_kernel(const GemvParams p) {
  constexpr int EB = InBytes<IN_W>::v;
  constexpr int VEC = 16 / EB;
  constexpr bool kInt = OUT == OUT_I32;
  using T = decltype(from_f32<OUT>(0.0f));
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bi = blockIdx.y;
  const uint32_t n_base = (blockIdx.x * kWarps + warp) * kRowsPerWarp;
  if (n_base >= p.n) return;
  const char* a = static_cast<const char*>(p.a) + (size_t)(bi % p.a_batch) * p.m * p.k * EB;
  const char* w = static_cast<const char*>(p.w) + (size_t)(bi % p.b_batch) * p.n * p.k * EB;

  float accf[MT][kRowsPerWarp];
  int acci[MT][kRowsPerWarp];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) { accf[m][r] = 0.0f; acci[m][r] = 0; }

  for (uint32_t k0 = lane * VEC; k0 < p.k; k0 += 32 * VEC) {
    float wv[kRowsPerWarp][VEC];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const uint32_t n = min(n_base + r, p.n - 1);   // rows past N repeat the last row; never stored
      const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(w + ((size_t)n * p.k + k0) * EB));   // streamed once
      widen16<IN_W>(raw, wv[r]);
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < (int)p.m) {
        float av[VEC];
        widen16<IN_A>(__ldg(reinterpret_cast<const uint4*>(a + ((size_t)m * p.k + k0) * EB)), av);
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            if constexpr (kInt) acci[m][r] += __float_as_int(av[e]) * __float_as_int(wv[r][e]);
            else accf[m][r] = fmaf(av[e], wv[r][e], accf[m][r]);
          }
      }
    }
  }

  // Lane reduction in a fixed butterfly order, then the epilogue on lane 0.
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        if constexpr (kInt) acci[m][r] += __shfl_xor_sync(0xFFFFFFFFu, acci[m][r], off);
        else accf[m][r] += __shfl_xor_sync(0xFFFFFFFFu, accf[m][r], off);
      }
    }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m >= (int)p.m) break;
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const uint32_t n = n_base + r;
        if (n >= p.n) break;
        const size_t idx = ((size_t)bi * p.m + m) * p.n + n;
        if constexpr (kInt) {
          static_cast<int32_t*>(p.out)[idx] = finish_i32((uint32_t)acci[m][r], static_cast<const int32_t*>(p.bias), n);
        } else {
          float x = accf[m][r] * p.scale;
          if (p.bias) x += load_f32<OUT>(static_cast<const T*>(p.bias), n);
          x = apply_activation(x, p.act);
          if (p.residual) x += to_f32<OUT>(static_cast<const T*>(p.residual)[idx]);
          static_cast<T*>(p.out)[idx] = from_f32<OUT>(x);
        }
      }
    }
  }
}

template <int IN_A, int IN_W, int OUT>
cudaError_t launch_mt(const GemvParams& p, dim3 grid, cudaStream_t stream) {
  if (p.m <= 1) gemv_bt_kernel<IN_A, IN_W, OUT, 1><<<grid, kWarps * 32, 0, stream>>>(p);
  else if (p.m <= 4) gemv_bt_kernel<IN_A, IN_W, OUT, 4><<<grid, kWarps * 32, 0, stream>>>(p);
  else if (p.m <= 8) gemv_bt_kernel<IN_A, IN_W, OUT, 8><<<grid, kWarps * 32, 0, stream>>>(p);
  else gemv_bt_kernel<IN_A, IN_W, OUT, 16><<<grid, kWarps * 32, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

bool gemv_bt_applicable(const GemmLaunch& g) {
  if (g.b_layout != NUMR_B200_B_NK || g.m == 0 || g.k == 0 || g.n == 0) return false;
  // Measured on B200 (N = K = 4096, weights from HBM): a single row streams at the rate of the
  // vendor library's kernel; from two rows on the tensor-core path (which trims its A tile to the
  // rows that exist) is faster, except for exact F32, whose three-product form pays until M = 8.
  uint32_t m_max = (g.kind == KIND_TF32 && g.f32_exact) ? 8u : 1u;
  const int forced_max = tuning().gemv_max_m;   // tests, experiments
  if (forced_max >= 0) m_max = (uint32_t)std::min(16, forced_max);
  if (g.m > m_max) return false;
  // A warp owns four rows of W and walks K alone: with few rows and a long K too few warps are in flight
  // (1 x 4096 x 14336: 41.7 us here against 25.6 us on the tensor-core path with its K-split clusters; at
  // 1 x 14336 x 4096 this kernel wins, 22.4 against 26.1 us; equal at 4096 x 4096).
  if (forced_max < 0 && !(g.kind == KIND_TF32 && g.f32_exact) && (uint64_t)g.n * 2 < g.k) return false;
  if (g.kind == KIND_I8 && g.k > kI8ExactK) return false;                        // int32 sums: exact range only
  if (((size_t)g.k * g.elt_bytes) % 16 != 0) return false;                       // 16-byte steps along K
  if ((reinterpret_cast<uintptr_t>(g.a) | reinterpret_cast<uintptr_t>(g.b)) & 15) return false;
  if (g.lda != g.k || g.ldb != g.k) return false;                                // dense rows
  return true;
}

int launch_gemv_bt(const GemmLaunch& g) {
  GemvParams p;
  p.a = g.a; p.w = g.b; p.bias = g.bias; p.residual = g.residual; p.out = g.out;
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.a_batch = g.a_batch; p.b_batch = g.b_batch;
  p.scale = g.scale; p.act = g.activation;
  const uint32_t cols_per_block = kWarps * kRowsPerWarp;
  if (g.batch > 65535) return fail(NUMR_B200_EINVAL, "small-M path: more than 65535 batches");
  dim3 grid((g.n + cols_per_block - 1) / cols_per_block, g.batch, 1);
  cudaError_t e = cudaErrorInvalidValue;
  // (operand kinds, output kind): the combinations the tensor-core path offers
  const bool bf16 = g.kind == KIND_F16 && g.a_fmt == 1, f16 = g.kind == KIND_F16 && g.a_fmt == 0;
  if (g.kind == KIND_TF32 && g.out_kind == OUT_F32) e = launch_mt<IN_F32, IN_F32, OUT_F32>(p, grid, g.stream);
  else if (bf16 && g.out_kind == OUT_BF16) e = launch_mt<IN_BF16, IN_BF16, OUT_BF16>(p, grid, g.stream);
  else if (f16 && g.out_kind == OUT_F16) e = launch_mt<IN_F16, IN_F16, OUT_F16>(p, grid, g.stream);
  else if (g.kind == KIND_I8 && g.out_kind == OUT_I32) e = launch_mt<IN_I8, IN_I8, OUT_I32>(p, grid, g.stream);
  else if (g.kind == KIND_F8F6F4 && g.b_fmt == 0) {
    const bool a5 = g.a_fmt == 1;
    switch (g.out_kind) {
      case OUT_F32: e = a5 ? launch_mt<IN_E5M2, IN_E4M3, OUT_F32>(p, grid, g.stream) : launch_mt<IN_E4M3, IN_E4M3, OUT_F32>(p, grid, g.stream); break;
      case OUT_BF16: e = a5 ? launch_mt<IN_E5M2, IN_E4M3, OUT_BF16>(p, grid, g.stream) : launch_mt<IN_E4M3, IN_E4M3, OUT_BF16>(p, grid, g.stream); break;
      case OUT_F16: e = a5 ? launch_mt<IN_E5M2, IN_E4M3, OUT_F16>(p, grid, g.stream) : launch_mt<IN_E4M3, IN_E4M3, OUT_F16>(p, grid, g.stream); break;
      default: return -1;   // FP8 outputs stay on the tensor-core path
    }
  } else {
    return -1;              // not offered here: the caller falls through to the tensor-core path
  }
  if (e != cudaSuccess) return fail(NUMR_B200_ECUDA, "small-M kernel launch failed: %s", cudaGetErrorString(e));
  return NUMR_B200_OK;
}

}  // namespace nb
