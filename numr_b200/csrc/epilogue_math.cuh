// Epilogue arithmetic shared by the GEMM kernel and the K == 0 kernel: activation
// functions, element conversions (one rounding per output) and the I8 -> I32 finish.
//
// Semantics follow the reference: the activation formulas of apply_activation_f32
// (src/runtime/cuda/kernels/gemm_activation.cuh:14-35);
// bf16/f16 narrowing is round-to-nearest-even (half crate 2.7.1 `from_f32`);
// FP8 narrowing follows src/dtype/fp8.rs:503-667 (E4M3: RNE, saturate to +-448, NaN
// 0x7F|sign; E5M2: RNE, overflow to +-inf, NaN 0x7F|sign); the I8 path adds the I32
// bias to the wide accumulator and saturates once (matmul_int.cu:87-103).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

#include "gemm_internal.h"

namespace nb {

// The transcendental forms use the hardware exp2 / reciprocal approximations (relative error
// about 2e-6 here, well inside the tightest bound on this path, 1e-5); the reference builds its
// own kernels with --use_fast_math (build.rs:340). GELU is written as x * sigmoid(2u), which is
// 0.5 x (1 + tanh(u)) without the cancellation of 1 + tanh near -1.
//
// The forward formulas work on PAIRS of values with the packed f32x2 instructions of sm_100 (half
// the issue slots of the scalar forms; the epilogue warps are bound by instruction issue), the two
// special-function results of a pair being the only scalar steps. The scalar forms below are the
// packed ones on a duplicated value, so every kernel of the library rounds alike.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float2 pair_of(float v) { return make_float2(v, v); }

// x * sigmoid(-a / log2(e)) given a = the exponent argument of 2^a: x / (1 + 2^a)
__device__ __forceinline__ float2 times_sigmoid_of_exp2_arg(float2 x, float2 a) {
  const float2 d = __fadd2_rn(make_float2(ex2_approx(a.x), ex2_approx(a.y)), pair_of(1.0f));
  return __fmul2_rn(x, make_float2(rcp_approx(d.x), rcp_approx(d.y)));
}

template <int ACT>
__device__ __forceinline__ float2 activation2(float2 x) {
  constexpr float kLog2e = 1.4426950408889634f;
  if constexpr (ACT == NUMR_B200_ACT_RELU) return make_float2(fmaxf(x.x, 0.0f), fmaxf(x.y, 0.0f));
  else if constexpr (ACT == NUMR_B200_ACT_GELU) {
    // u = c (x + k x^3); the argument of 2^. is -2 u log2(e) = x (A + B x^2)
    constexpr float A = -2.0f * 0.7978845608f * kLog2e, B = A * 0.044715f;
    const float2 t = __ffma2_rn(__fmul2_rn(x, x), pair_of(B), pair_of(A));
    return times_sigmoid_of_exp2_arg(x, __fmul2_rn(x, t));
  }
  else if constexpr (ACT == NUMR_B200_ACT_SILU) return times_sigmoid_of_exp2_arg(x, __fmul2_rn(x, pair_of(-kLog2e)));
  else if constexpr (ACT == NUMR_B200_ACT_SIGMOID)
    return times_sigmoid_of_exp2_arg(pair_of(1.0f), __fmul2_rn(x, pair_of(-kLog2e)));
  else if constexpr (ACT == NUMR_B200_ACT_TANH) return make_float2(tanhf(x.x), tanhf(x.y));
  else return x;
}

__device__ __forceinline__ float fast_sigmoid(float x) {
  return activation2<NUMR_B200_ACT_SIGMOID>(pair_of(x)).x;
}

// Activation selected at compile time.
template <int ACT>
__device__ __forceinline__ float activation(float x) {
  return activation2<ACT>(pair_of(x)).x;
}

// d activation / d x at the pre-activation value x, the formulas of numr's backward kernel
// (src/runtime/cpu/kernels/gemm_epilogue/backward.rs:247-281); a non-finite derivative counts as 0
// there (backward.rs:201-202) and here.
template <int ACT>
__device__ __forceinline__ float activation_derivative(float x) {
  float d;
  if constexpr (ACT == NUMR_B200_ACT_RELU) d = x > 0.0f ? 1.0f : 0.0f;
  else if constexpr (ACT == NUMR_B200_ACT_GELU) {
    const float c = 0.7978845608f, k = 0.044715f;
    const float inner = c * (x + k * x * x * x);
    const float t = 2.0f * fast_sigmoid(2.0f * inner) - 1.0f;          // tanh(inner)
    const float sech2 = 1.0f - t * t;
    d = 0.5f * (1.0f + t) + 0.5f * x * sech2 * c * (1.0f + 3.0f * k * x * x);
  }
  else if constexpr (ACT == NUMR_B200_ACT_SILU) { const float s = fast_sigmoid(x); d = s + x * s * (1.0f - s); }
  else if constexpr (ACT == NUMR_B200_ACT_SIGMOID) { const float s = fast_sigmoid(x); d = s * (1.0f - s); }
  else if constexpr (ACT == NUMR_B200_ACT_TANH) { const float t = tanhf(x); d = 1.0f - t * t; }
  else d = 1.0f;
  return isfinite(d) ? d : 0.0f;
}

__device__ __forceinline__ float apply_activation_derivative(float x, int act) {
  switch (act) {
    case NUMR_B200_ACT_RELU: return activation_derivative<NUMR_B200_ACT_RELU>(x);
    case NUMR_B200_ACT_GELU: return activation_derivative<NUMR_B200_ACT_GELU>(x);
    case NUMR_B200_ACT_SILU: return activation_derivative<NUMR_B200_ACT_SILU>(x);
    case NUMR_B200_ACT_SIGMOID: return activation_derivative<NUMR_B200_ACT_SIGMOID>(x);
    case NUMR_B200_ACT_TANH: return activation_derivative<NUMR_B200_ACT_TANH>(x);
    default: return 1.0f;
  }
}

// Runtime-selected form for code that is not performance critical.
__device__ __forceinline__ float apply_activation(float x, int act) {
  switch (act) {
    case NUMR_B200_ACT_RELU: return activation<NUMR_B200_ACT_RELU>(x);
    case NUMR_B200_ACT_GELU: return activation<NUMR_B200_ACT_GELU>(x);
    case NUMR_B200_ACT_SILU: return activation<NUMR_B200_ACT_SILU>(x);
    case NUMR_B200_ACT_SIGMOID: return activation<NUMR_B200_ACT_SIGMOID>(x);
    case NUMR_B200_ACT_TANH: return activation<NUMR_B200_ACT_TANH>(x);
    default: return x;
  }
}

// ---- FP8 codecs on raw bytes -------------------------------------------------
__device__ __forceinline__ float e4m3_to_f32(uint8_t v) {
  const uint32_t sign = (uint32_t)(v & 0x80) << 24;
  const uint32_t exp = (v >> 3) & 0xF;
  const uint32_t man = v & 7;
  if (exp == 15 && man == 7) return __uint_as_float(sign | 0x7FC00000u);
  if (exp == 0) {
    const float f = (float)man * 0.001953125f;   // man * 2^-9
    return __uint_as_float(__float_as_uint(f) | sign);
  }
  return __uint_as_float(sign | ((exp + 120u) << 23) | (man << 20));
}

__device__ __forceinline__ float e5m2_to_f32(uint8_t v) {
  // E5M2 is the upper byte of an IEEE half.
  return __half2float(__ushort_as_half((unsigned short)((unsigned short)v << 8)));
}

// Round-to-nearest-even narrowing of |x| to a format with `MAN` mantissa bits, exponent
// bias `BIAS`; returns the magnitude bits (without sign) before range handling.
template <int MAN, int BIAS>
__device__ __forceinline__ uint32_t fp8_round_magnitude(uint32_t abs_bits) {
  const int exp = (int)(abs_bits >> 23) - 127;
  const uint32_t sig = (abs_bits & 0x7FFFFFu) | 0x800000u;   // 1.m, 24 bits
  int shift = 23 - MAN;                                       // bits dropped for a normal result
  int e_out = exp + BIAS;
  if (e_out <= 0) {            // subnormal result: drop more bits, exponent field 0
    shift += 1 - e_out;
    e_out = 0;
  }
  if (shift > 25) return 0;    // below half of the smallest subnormal
  const uint32_t kept = sig >> shift;
  const uint32_t rem = sig & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  uint32_t q = kept;
  if (rem > half || (rem == half && (kept & 1u))) ++q;
  // For a normal result q holds 1.m (MAN+1 bits): adding (e_out-1) << MAN lets a mantissa
  // carry fall into the exponent; for a subnormal result q is the mantissa itself and a carry
  // becomes the smallest normal.
  return e_out > 0 ? q + ((uint32_t)(e_out - 1) << MAN) : q;
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  const uint32_t bits = __float_as_uint(x);
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80);
  const uint32_t a = bits & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return sign | 0x7F;          // NaN
  if (a == 0x7F800000u) return sign | 0x7E;         // inf saturates
  if ((a >> 23) == 0) return sign;                  // zero and f32 subnormals
  if ((int)(a >> 23) - 127 > 8) return sign | 0x7E;
  const uint32_t m = fp8_round_magnitude<3, 7>(a);
  return sign | (uint8_t)(m > 0x7E ? 0x7E : m);
}

__device__ __forceinline__ uint8_t f32_to_e5m2(float x) {
  const uint32_t bits = __float_as_uint(x);
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80);
  const uint32_t a = bits & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return sign | 0x7F;
  if (a == 0x7F800000u) return sign | 0x7C;
  if ((a >> 23) == 0) return sign;
  if ((int)(a >> 23) - 127 > 15) return sign | 0x7C;
  const uint32_t m = fp8_round_magnitude<2, 15>(a);
  return sign | (uint8_t)(m > 0x7C ? 0x7C : m);
}

// ---- typed load / store helpers -----------------------------------------------
template <int OUT, typename T>
__device__ __forceinline__ float to_f32(T v) {
  if constexpr (OUT == OUT_F32) return v;
  else if constexpr (OUT == OUT_BF16) return __bfloat162float(v);
  else if constexpr (OUT == OUT_F16) return __half2float(v);
  else if constexpr (OUT == OUT_E4M3) return e4m3_to_f32(v);
  else if constexpr (OUT == OUT_E5M2) return e5m2_to_f32(v);
  else return (float)v;
}

template <int OUT, typename T>
__device__ __forceinline__ float load_f32(const T* p, uint32_t i) {
  return to_f32<OUT>(__ldg(p + i));
}

template <int OUT>
__device__ __forceinline__ auto from_f32(float x) {
  if constexpr (OUT == OUT_F32) return x;
  else if constexpr (OUT == OUT_BF16) return __float2bfloat16_rn(x);
  else if constexpr (OUT == OUT_F16) return __float2half_rn(x);
  else if constexpr (OUT == OUT_E4M3) return f32_to_e4m3(x);
  else if constexpr (OUT == OUT_E5M2) return f32_to_e5m2(x);
  else return (int32_t)x;
}

// Two f32 values narrowed to FP8 (low byte = a) by the hardware conversion (round to nearest even,
// saturating), then brought to the reference's rules where they differ (src/dtype/fp8.rs:503-667): a NaN
// keeps its sign (0x7F | sign), and E5M2 overflows to infinity where the hardware saturates to the largest
// finite value (|x| >= 61440 rounds to 2^16). The same bytes as f32_to_e4m3 / f32_to_e5m2 above at a
// fifth of the instructions.
template <int OUT>
__device__ __forceinline__ uint32_t fp8x2_from_f32(float a, float b) {
  constexpr bool kE5 = OUT == OUT_E5M2;
  uint32_t h = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kE5 ? __NV_E5M2 : __NV_E4M3);
  const float v[2] = {a, b};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t bits = __float_as_uint(v[i]);
    const uint32_t mag = bits & 0x7FFFFFFFu, sign = (bits >> 24) & 0x80u;
    uint32_t byte = (h >> (8 * i)) & 0xFFu;
    if (kE5 && mag >= 0x47700000u) byte = sign | 0x7Cu;   // 61440 and beyond (and infinity itself)
    if (mag > 0x7F800000u) byte = sign | 0x7Fu;           // NaN
    h = (h & ~(0xFFu << (8 * i))) | (byte << (8 * i));
  }
  return h;
}

// Element `i` of a 16-byte vector of output-typed values held in registers, and the packing of
// finished values into such a vector: bit operations only, so nothing is addressed through memory.
template <int OUT>
__device__ __forceinline__ float vec_elem_f32(const int4& v, int i) {
  const uint32_t w[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
  if constexpr (OUT == OUT_F32) return __uint_as_float(w[i]);
  else if constexpr (OUT == OUT_BF16) return __uint_as_float((i & 1) ? (w[i >> 1] & 0xFFFF0000u) : (w[i >> 1] << 16));
  else if constexpr (OUT == OUT_F16) return __half2float(__ushort_as_half((unsigned short)(w[i >> 1] >> (16 * (i & 1)))));
  else if constexpr (OUT == OUT_E4M3) return e4m3_to_f32((uint8_t)(w[i >> 2] >> (8 * (i & 3))));
  else if constexpr (OUT == OUT_E5M2) return e5m2_to_f32((uint8_t)(w[i >> 2] >> (8 * (i & 3))));
  else return (float)(int32_t)w[i];
}

// Packs the 16 / sizeof(T) finished values x[0..] into one 16-byte vector (one rounding each).
template <int OUT>
__device__ __forceinline__ uint4 pack_out(const float* x) {
  uint32_t w[4];
  if constexpr (OUT == OUT_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __float_as_uint(x[i]);
  } else if constexpr (OUT == OUT_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);   // one conversion per pair
      w[i] = (uint32_t)__bfloat16_as_ushort(h.x) | ((uint32_t)__bfloat16_as_ushort(h.y) << 16);
    }
  } else if constexpr (OUT == OUT_F16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
      w[i] = (uint32_t)__half_as_ushort(h.x) | ((uint32_t)__half_as_ushort(h.y) << 16);
    }
  } else if constexpr (OUT == OUT_E4M3 || OUT == OUT_E5M2) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = fp8x2_from_f32<OUT>(x[4 * i], x[4 * i + 1]) | (fp8x2_from_f32<OUT>(x[4 * i + 2], x[4 * i + 3]) << 16);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (uint32_t)(int32_t)x[i];
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// clamp((int64)a + (int64)b) to the int32 range, as one instruction
__device__ __forceinline__ uint32_t add_sat_s32(uint32_t a, uint32_t b) {
  int32_t d;
  asm("add.sat.s32 %0, %1, %2;" : "=r"(d) : "r"((int32_t)a), "r"((int32_t)b));
  return (uint32_t)d;
}

__device__ __forceinline__ int32_t finish_i32(uint32_t acc_bits, const int32_t* bias, uint32_t col) {
  return (int32_t)add_sat_s32(acc_bits, bias ? (uint32_t)__ldg(bias + col) : 0u);
}

}  // namespace nb
