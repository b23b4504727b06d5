// Integer GEMM for the widths that have no tensor-core form: I16, I32, I64, U8, U16, U32, U64.
//
// Semantics of the reference (src/runtime/cuda/kernels/matmul_int.cu:1-104, numr128.cuh; CPU
// `matmul_scalar_acc::<T, i128>` in src/runtime/cpu/kernels/matmul/kernel.rs:145-175): every
// product is added, in K order, into a signed 128-bit accumulator, the bias (of the element type)
// seeds that accumulator, and the sum is clamped to the element type once, at the store. The output has the
// operands' type. (I8 is the one width that widens to I32; it runs on the tensor cores.)
//
// Plain CUDA-core kernel: 64 x 64 output tile per block of 256 threads, 4 x 4 outputs per thread,
// K staged through shared memory 16 deep, accumulators as native 128-bit integers. It is bound by
// the software 128-bit multiply-add, as the reference's kernel is.
#include "gemm_internal.h"

namespace nb {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// The accumulator is a SIGNED 128-bit integer for every element type, unsigned ones included, as
// in the reference (`i128` on the CPU, `Numr128` on CUDA). Products of elements up to 32 bits and
// any sum of 2^32 of them stay far inside it, so those widths use the plain multiply-add. The two
// 64-bit widths can leave it: one U64 product reaches 2^128, and two I64 products reach 2^127. For
// them the multiply and the add saturate at the 128-bit bounds, term by term in K order, which is
// what `i128::saturating_mul` / `saturating_add` give on the CPU (wide_acc.rs:109-135).
using acc_t = __int128;
using uacc_t = unsigned __int128;

__device__ __forceinline__ acc_t acc_max() { return (acc_t)(~(uacc_t)0 >> 1); }
__device__ __forceinline__ acc_t acc_min() { return -acc_max() - 1; }

__device__ __forceinline__ acc_t add_sat(acc_t a, acc_t b) {
  const acc_t r = (acc_t)((uacc_t)a + (uacc_t)b);
  const bool overflow = (((a ^ r) & (b ^ r)) >> 127) != 0;
  return overflow ? (a < 0 ? acc_min() : acc_max()) : r;
}

template <typename T>
__device__ __forceinline__ acc_t mul_add(acc_t acc, T a, T b) {
  if constexpr (sizeof(T) < 8) {
    return acc + (acc_t)a * (acc_t)b;
  } else if constexpr (static_cast<T>(-1) < static_cast<T>(0)) {
    return add_sat(acc, (acc_t)a * (acc_t)b);               // |product| <= 2^126
  } else {
    const uacc_t p = (uacc_t)a * (uacc_t)b;                 // < 2^128
    return add_sat(acc, (p >> 127) ? acc_max() : (acc_t)p);
  }
}

template <typename T>
__device__ __forceinline__ T saturate(acc_t v) {
  constexpr bool is_signed = static_cast<T>(-1) < static_cast<T>(0);
  constexpr int bits = sizeof(T) * 8;
  if constexpr (is_signed) {
    const acc_t hi = ((acc_t)1 << (bits - 1)) - 1;
    const acc_t lo = -hi - 1;
    return static_cast<T>(v > hi ? hi : (v < lo ? lo : v));
  } else {
    const acc_t hi = ((acc_t)1 << bits) - 1;
    return static_cast<T>(v > hi ? hi : (v < 0 ? (acc_t)0 : v));
  }
}

struct IntParams {
  const void* a;
  const void* b;
  const void* bias;
  void* out;
  uint32_t m, n, k, a_batch, b_batch;
  int b_nk;   // B stored as [N,K]
};

template <typename T>
__global__ void __launch_bounds__(256) matmul_int_kernel(const IntParams p) {
  using W = acc_t;
  __shared__ T As[BK][BM + 1];
  __shared__ T Bs[BK][BN + 1];
  const uint32_t bi = blockIdx.z;
  const T* a = static_cast<const T*>(p.a) + (size_t)(bi % p.a_batch) * p.m * p.k;
  const T* b = static_cast<const T*>(p.b) + (size_t)(bi % p.b_batch) * p.k * p.n;
  T* out = static_cast<T*>(p.out) + (size_t)bi * p.m * p.n;
  const T* bias = static_cast<const T*>(p.bias);
  const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads

  W acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const uint32_t col = n0 + tx * TN + j;
      acc[i][j] = (bias && col < p.n) ? static_cast<W>(bias[col]) : static_cast<W>(0);
    }

  for (uint32_t k0 = 0; k0 < p.k; k0 += BK) {
    // 64 x 16 elements of A and of B, 4 each per thread; out-of-range elements are zero.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t idx = threadIdx.x + i * 256;
      {
        const uint32_t r = idx / BK, kk = idx % BK;      // A: consecutive threads along K (contiguous)
        const uint32_t row = m0 + r, kg = k0 + kk;
        As[kk][r] = (row < p.m && kg < p.k) ? a[(size_t)row * p.k + kg] : static_cast<T>(0);
      }
      if (p.b_nk) {
        const uint32_t c = idx / BK, kk = idx % BK;      // B as [N,K]: contiguous along K
        const uint32_t col = n0 + c, kg = k0 + kk;
        Bs[kk][c] = (col < p.n && kg < p.k) ? b[(size_t)col * p.k + kg] : static_cast<T>(0);
      } else {
        const uint32_t kk = idx / BN, c = idx % BN;      // B as [K,N]: contiguous along N
        const uint32_t col = n0 + c, kg = k0 + kk;
        Bs[kk][c] = (col < p.n && kg < p.k) ? b[(size_t)kg * p.n + col] : static_cast<T>(0);
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      T av[TM], bv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) bv[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = mul_add<T>(acc[i][j], av[i], bv[j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const uint32_t row = m0 + ty * TM + i;
    if (row >= p.m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const uint32_t col = n0 + tx * TN + j;
      if (col < p.n) out[(size_t)row * p.n + col] = saturate<T>(acc[i][j]);
    }
  }
}

template <typename T>
cudaError_t launch_t(const IntParams& p, dim3 grid, cudaStream_t stream) {
  matmul_int_kernel<T><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

int launch_matmul_int(int dtype, const void* a, const void* b, const void* bias, void* out, uint32_t batch,
                      uint32_t m, uint32_t n, uint32_t k, uint32_t a_batch, uint32_t b_batch, int b_nk,
                      cudaStream_t stream) {
  if (batch == 0 || m == 0 || n == 0) return NUMR_B200_OK;
  if (batch > 65535) return fail(NUMR_B200_EINVAL, "integer matmul: more than 65535 batches");
  IntParams p{a, b, bias, out, m, n, k, a_batch, b_batch, b_nk};
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM, batch);
  if (grid.y > 65535) return fail(NUMR_B200_EINVAL, "integer matmul: M too large for this kernel");
  cudaError_t e;
  switch (dtype) {
    case NUMR_B200_I16: e = launch_t<int16_t>(p, grid, stream); break;
    case NUMR_B200_I32: e = launch_t<int32_t>(p, grid, stream); break;
    case NUMR_B200_I64: e = launch_t<int64_t>(p, grid, stream); break;
    case NUMR_B200_U8: e = launch_t<uint8_t>(p, grid, stream); break;
    case NUMR_B200_U16: e = launch_t<uint16_t>(p, grid, stream); break;
    case NUMR_B200_U32: e = launch_t<uint32_t>(p, grid, stream); break;
    case NUMR_B200_U64: e = launch_t<uint64_t>(p, grid, stream); break;
    default: return fail(NUMR_B200_EUNSUPPORTED, "integer matmul: dtype %d", dtype);
  }
  if (e != cudaSuccess) return fail(NUMR_B200_ECUDA, "integer matmul launch failed: %s", cudaGetErrorString(e));
  return NUMR_B200_OK;
}

}  // namespace nb
