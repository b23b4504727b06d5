// TEST INFRASTRUCTURE — CPU oracle for the numr dense-GEMM path.
//
// A from-scratch C++ restatement of what numr's CPU backend computes for matmul,
// matmul_bias, the fused GEMM epilogue ops, I8 x I8 -> I32 and FP8 scaled matmul.
// It is the checker for the CUDA path and the timed CPU baseline; nothing in the
// shipped library links or calls it.
//
// Pinning: numr is Rust and cannot be built where this oracle is developed, so the
// oracle is pinned against the literals of numr's own tests (I8 and FP8 known
// answers, FP8 codec constants and rounding cases, shape tables) in
// tests/test_oracle_kat.py, and against float64 ground truth.
//
// Reference files each part follows (paths inside the numr repository):
//   f32 GEMM blocking (MR=6, NR=32, KC=256, MC=126, NC=512; bias preloaded into C,
//     then every K block accumulates)  src/runtime/cpu/kernels/simd/matmul/dispatch.rs:51-118,
//                                      src/runtime/cpu/kernels/simd/matmul/tiling.rs:117-142
//   128-column parallel chunks         src/ops/cpu/matmul_columns.rs:75,99-103
//   bf16/f16 via f32                   src/runtime/cpu/kernels/simd/matmul/half_convert.rs:74-154
//   epilogue ops                       src/runtime/cpu/kernels/gemm_epilogue/forward.rs:21-330
//   I8 -> I32                          src/ops/cpu/matmul_i8.rs:24-118,
//                                      src/runtime/cpu/kernels/simd/matmul/int8.rs:18-91
//   FP8 scaled matmul                  src/ops/cpu/fp8_matmul.rs:81-133
//   FP8 codecs                         src/dtype/fp8.rs:503-667 (E4M3), :670-860 (E5M2)
//   bf16/f16 conversion                half crate 2.7.1 (Cargo.lock:923-924): round to nearest even
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

enum { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2, DT_E4M3 = 3, DT_E5M2 = 4, DT_I8 = 5, DT_I32 = 6 };
enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SILU = 3, ACT_SIGMOID = 4, ACT_TANH = 5 };

// ------------------------------------------------------------------ scalar codecs
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

ORC_API uint16_t orc_f32_to_bf16(float x) {
  uint32_t u = f2u(x);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);   // quiet NaN
  const uint32_t round = 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)((u + round) >> 16);
}
ORC_API float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

ORC_API uint16_t orc_f32_to_f16(float x) {
  const uint32_t u = f2u(x);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((a >> 13) & 0x3FFu));
  if (a >= 0x47800000u) return (uint16_t)(sign | 0x7C00u);       // >= 65536 -> inf (65520 rounds below)
  const int exp = (int)(a >> 23) - 127;
  if (exp < -25) return (uint16_t)sign;
  uint32_t sig = (a & 0x7FFFFFu) | 0x800000u;
  int shift = 13;
  int e_out = exp + 15;
  if (e_out <= 0) { shift += 1 - e_out; e_out = 0; }
  const uint32_t kept = sig >> shift;
  const uint32_t rem = sig & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  uint32_t q = kept + ((rem > half || (rem == half && (kept & 1u))) ? 1u : 0u);
  const uint32_t mag = e_out > 0 ? q + ((uint32_t)(e_out - 1) << 10) : q;
  return (uint16_t)(sign | (mag > 0x7C00u ? 0x7C00u : mag));
}
ORC_API float orc_f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
  if (exp == 31) return u2f(sign | 0x7F800000u | (man << 13));
  if (exp == 0) {
    const float f = (float)man * 5.9604644775390625e-08f;   // man * 2^-24
    return u2f(f2u(f) | sign);
  }
  return u2f(sign | ((exp + 112u) << 23) | (man << 13));
}

// Rounds |x| (normal f32, bits `a`) to MAN mantissa bits with exponent bias BIAS, nearest even;
// returns the magnitude field, where a mantissa carry moves into the exponent.
template <int MAN, int BIAS>
static inline uint32_t fp8_magnitude(uint32_t a) {
  const int exp = (int)(a >> 23) - 127;
  const uint32_t sig = (a & 0x7FFFFFu) | 0x800000u;
  int shift = 23 - MAN;
  int e_out = exp + BIAS;
  if (e_out <= 0) { shift += 1 - e_out; e_out = 0; }
  if (shift > 25) return 0;
  const uint32_t kept = sig >> shift;
  const uint32_t rem = sig & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  const uint32_t q = kept + ((rem > half || (rem == half && (kept & 1u))) ? 1u : 0u);
  return e_out > 0 ? q + ((uint32_t)(e_out - 1) << MAN) : q;
}

ORC_API uint8_t orc_f32_to_e4m3(float x) {
  const uint32_t u = f2u(x);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return sign | 0x7F;        // NaN keeps its sign
  if (a == 0x7F800000u) return sign | 0x7E;       // no infinity in E4M3: saturate
  if ((a >> 23) == 0) return sign;                // zero and f32 subnormals
  if ((int)(a >> 23) - 127 > 8) return sign | 0x7E;
  const uint32_t m = fp8_magnitude<3, 7>(a);
  return sign | (uint8_t)(m > 0x7Eu ? 0x7Eu : m); // 0x7F would be NaN: clamp to max
}
ORC_API float orc_e4m3_to_f32(uint8_t v) {
  const uint32_t sign = (uint32_t)(v & 0x80u) << 24;
  const uint32_t exp = (v >> 3) & 0xFu, man = v & 7u;
  if (exp == 15 && man == 7) return u2f(sign | 0x7FC00000u);
  if (exp == 0) return u2f(f2u((float)man * 0.001953125f) | sign);
  return u2f(sign | ((exp + 120u) << 23) | (man << 20));
}
ORC_API uint8_t orc_f32_to_e5m2(float x) {
  const uint32_t u = f2u(x);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return sign | 0x7F;
  if (a == 0x7F800000u) return sign | 0x7C;
  if ((a >> 23) == 0) return sign;
  if ((int)(a >> 23) - 127 > 15) return sign | 0x7C;   // overflow -> infinity
  const uint32_t m = fp8_magnitude<2, 15>(a);
  return sign | (uint8_t)(m > 0x7Cu ? 0x7Cu : m);
}
ORC_API float orc_e5m2_to_f32(uint8_t v) {
  const uint32_t sign = (uint32_t)(v & 0x80u) << 24;
  const uint32_t exp = (v >> 2) & 0x1Fu, man = v & 3u;
  if (exp == 31) return u2f(sign | 0x7F800000u | (man ? 0x400000u : 0u));
  if (exp == 0) return u2f(f2u((float)man * 1.52587890625e-05f) | sign);   // man * 2^-16
  return u2f(sign | ((exp + 112u) << 23) | (man << 21));
}

static inline size_t dt_size(int dt) {
  switch (dt) { case DT_F32: case DT_I32: return 4; case DT_BF16: case DT_F16: return 2; default: return 1; }
}
static inline float load_as_f32(const void* p, size_t i, int dt) {
  switch (dt) {
    case DT_F32: return ((const float*)p)[i];
    case DT_BF16: return orc_bf16_to_f32(((const uint16_t*)p)[i]);
    case DT_F16: return orc_f16_to_f32(((const uint16_t*)p)[i]);
    case DT_E4M3: return orc_e4m3_to_f32(((const uint8_t*)p)[i]);
    case DT_E5M2: return orc_e5m2_to_f32(((const uint8_t*)p)[i]);
    case DT_I8: return (float)((const int8_t*)p)[i];
    default: return (float)((const int32_t*)p)[i];
  }
}
static inline void store_from_f32(void* p, size_t i, int dt, float v) {
  switch (dt) {
    case DT_F32: ((float*)p)[i] = v; break;
    case DT_BF16: ((uint16_t*)p)[i] = orc_f32_to_bf16(v); break;
    case DT_F16: ((uint16_t*)p)[i] = orc_f32_to_f16(v); break;
    case DT_E4M3: ((uint8_t*)p)[i] = orc_f32_to_e4m3(v); break;
    case DT_E5M2: ((uint8_t*)p)[i] = orc_f32_to_e5m2(v); break;
    default: break;
  }
}

ORC_API void orc_encode(const float* in, void* out, size_t n, int dt) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; ++i) store_from_f32(out, (size_t)i, dt, in[i]);
}
ORC_API void orc_decode(const void* in, float* out, size_t n, int dt) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; ++i) out[i] = load_as_f32(in, (size_t)i, dt);
}

// ------------------------------------------------------------------ activations
static inline float act_f32(float x, int act) {
  switch (act) {
    case ACT_RELU: return x < 0.0f ? 0.0f : x;
    case ACT_GELU: {
      const float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(inner));
    }
    case ACT_SILU: return x / (1.0f + expf(-x));
    case ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case ACT_TANH: return tanhf(x);
    default: return x;
  }
}
static inline double act_f64(double x, int act) {
  switch (act) {
    case ACT_RELU: return x < 0.0 ? 0.0 : x;
    case ACT_GELU: {
      const double inner = 0.7978845608028654 * (x + 0.044715 * x * x * x);
      return 0.5 * x * (1.0 + tanh(inner));
    }
    case ACT_SILU: return x / (1.0 + exp(-x));
    case ACT_SIGMOID: return 1.0 / (1.0 + exp(-x));
    case ACT_TANH: return tanh(x);
    default: return x;
  }
}

// ------------------------------------------------------------------ f32 blocked GEMM
namespace {
constexpr int MR = 6, NR = 32, MC = 126, KC = 256, NC = 512;
typedef float vf16 __attribute__((vector_size(64), aligned(4)));

// C[MR x NR] (+)= packed A panel (kc x MR, column of MR per k) * packed B panel (kc x NR).
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
void micro_kernel(const float* pa, const float* pb, float* c, int ldc, int kc, int mr, int nr, bool accumulate) {
  vf16 acc[MR][2];
  for (int i = 0; i < MR; ++i) { acc[i][0] = vf16{} ; acc[i][1] = vf16{}; }
  for (int p = 0; p < kc; ++p) {
    const vf16 b0 = *(const vf16*)(pb + (size_t)p * NR);
    const vf16 b1 = *(const vf16*)(pb + (size_t)p * NR + 16);
    for (int i = 0; i < MR; ++i) {
      const float a = pa[(size_t)p * MR + i];
      acc[i][0] += a * b0;
      acc[i][1] += a * b1;
    }
  }
  for (int i = 0; i < mr; ++i) {
    float tmp[NR];
    memcpy(tmp, &acc[i][0], 64);
    memcpy(tmp + 16, &acc[i][1], 64);
    float* crow = c + (size_t)i * ldc;
    if (accumulate) for (int j = 0; j < nr; ++j) crow[j] += tmp[j];
    else for (int j = 0; j < nr; ++j) crow[j] = tmp[j];
  }
}

// One column chunk [n0, n0+nc_total) of C = A*B (+ preloaded C when `preloaded`).
// b_t: B is stored as [N][ldb] (transposed operand), only the packing index changes.
void gemm_f32_columns(const float* a, const float* b, float* c, int m, int k, int lda, int ldb, int ldc,
                      int n0, int n_cols, bool preloaded, bool b_t) {
  std::vector<float> pack_a((size_t)MC * KC), pack_b((size_t)KC * NC);
  for (int jc = 0; jc < n_cols; jc += NC) {
    const int nc = std::min(NC, n_cols - jc);
    for (int pc = 0; pc < k; pc += KC) {
      const int kc = std::min(KC, k - pc);
      // Pack B: NR-wide panels, k-major inside a panel, zero padded.
      for (int jr = 0; jr < nc; jr += NR) {
        float* dst = pack_b.data() + (size_t)jr * kc;
        const int nr = std::min(NR, nc - jr);
        for (int p = 0; p < kc; ++p)
          for (int j = 0; j < NR; ++j) {
            float v = 0.0f;
            if (j < nr) {
              const int col = n0 + jc + jr + j;
              v = b_t ? b[(size_t)col * ldb + (pc + p)] : b[(size_t)(pc + p) * ldb + col];
            }
            dst[(size_t)p * NR + j] = v;
          }
      }
      const bool accumulate = preloaded || pc > 0;
      for (int ic = 0; ic < m; ic += MC) {
        const int mc = std::min(MC, m - ic);
        for (int ir = 0; ir < mc; ir += MR) {
          float* dst = pack_a.data() + (size_t)ir * kc;
          const int mr = std::min(MR, mc - ir);
          for (int p = 0; p < kc; ++p)
            for (int i = 0; i < MR; ++i)
              dst[(size_t)p * MR + i] = i < mr ? a[(size_t)(ic + ir + i) * lda + (pc + p)] : 0.0f;
        }
        for (int jr = 0; jr < nc; jr += NR)
          for (int ir = 0; ir < mc; ir += MR)
            micro_kernel(pack_a.data() + (size_t)ir * kc, pack_b.data() + (size_t)jr * kc,
                         c + (size_t)(ic + ir) * ldc + (n0 + jc + jr), ldc, kc, std::min(MR, mc - ir),
                         std::min(NR, nc - jr), accumulate);
      }
    }
  }
}

inline int resolve_threads(int threads) {
#ifdef _OPENMP
  return threads > 0 ? threads : omp_get_max_threads();
#else
  (void)threads;
  return 1;
#endif
}
}  // namespace

// C = A @ B (+ bias broadcast over rows). 128-column chunks are spread over `threads`
// (0 = all); the chunking is shape-pure so the result does not depend on the thread count.
ORC_API void orc_matmul_f32(const float* a, const float* b, const float* bias, float* c, int m, int n,
                            int k, int lda, int ldb, int ldc, int b_transposed, int threads) {
  if (m <= 0 || n <= 0) return;
  if (bias)
    for (int i = 0; i < m; ++i) memcpy(c + (size_t)i * ldc, bias, (size_t)n * sizeof(float));
  if (k == 0) {
    if (!bias) for (int i = 0; i < m; ++i) memset(c + (size_t)i * ldc, 0, (size_t)n * sizeof(float));
    return;
  }
  const int chunk = 128;
  const int chunks = (n + chunk - 1) / chunk;
  const int nt = resolve_threads(threads);
  (void)nt;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
  for (int ci = 0; ci < chunks; ++ci) {
    const int n0 = ci * chunk;
    gemm_f32_columns(a, b, c, m, k, lda, ldb, ldc, n0, std::min(chunk, n - n0), bias != nullptr,
                     b_transposed != 0);
  }
}

// ------------------------------------------------------------------ I8 -> I32
// Exact: i32 partial sums are folded into an i64 every 16384 products, bias joins the wide
// sum, one clamp to i32 at the end.
namespace {
__attribute__((target_clones("avx512f", "avx2", "default")))
long long dot_i8_wide(const int8_t* x, const int8_t* y, int k) {
  long long wide = 0;
  for (int p0 = 0; p0 < k; p0 += 16384) {
    const int p1 = std::min(k, p0 + 16384);
    int part = 0;
    for (int p = p0; p < p1; ++p) part += (int)x[p] * (int)y[p];
    wide += part;
  }
  return wide;
}
}  // namespace

ORC_API void orc_matmul_i8_i32(const int8_t* a, const int8_t* b, const int32_t* bias, int32_t* c, int m,
                               int n, int k, int b_transposed, int threads) {
  if (m <= 0 || n <= 0) return;
  std::vector<int8_t> bt;
  const int8_t* bcol = b;
  if (!b_transposed && k > 0) {   // column-pack B so every dot product reads contiguous bytes
    bt.resize((size_t)n * k);
    for (int p = 0; p < k; ++p)
      for (int j = 0; j < n; ++j) bt[(size_t)j * k + p] = b[(size_t)p * n + j];
    bcol = bt.data();
  }
  const int nt = resolve_threads(threads);
  (void)nt;
#pragma omp parallel for schedule(static) num_threads(nt)
  for (int i = 0; i < m; ++i) {
    const int8_t* arow = a + (size_t)i * k;
    for (int j = 0; j < n; ++j) {
      const int8_t* bc = bcol + (size_t)j * k;
      long long wide = dot_i8_wide(arow, bc, k);
      if (bias) wide += bias[j];
      wide = std::min<long long>(std::max<long long>(wide, INT32_MIN), INT32_MAX);
      c[(size_t)i * n + j] = (int32_t)wide;
    }
  }
}

// ------------------------------------------------------------------ FP8 scaled matmul
// Scalar triple loop: decode per multiply, f32 accumulation in k order, one multiply by
// scale_a*scale_b, then act(x + bias) + residual in f32 (the fused superset) and one narrowing.
ORC_API void orc_fp8_matmul(const uint8_t* a, const uint8_t* b, int a_dt, int b_dt, const void* bias,
                            const void* residual, void* out, int out_dt, int m, int n, int k,
                            int b_transposed, float scale_a, float scale_b, int act, int threads) {
  float lut_a[256], lut_b[256];
  for (int v = 0; v < 256; ++v) {
    lut_a[v] = a_dt == DT_E5M2 ? orc_e5m2_to_f32((uint8_t)v) : orc_e4m3_to_f32((uint8_t)v);
    lut_b[v] = b_dt == DT_E5M2 ? orc_e5m2_to_f32((uint8_t)v) : orc_e4m3_to_f32((uint8_t)v);
  }
  const float combined = scale_a * scale_b;
  const int nt = resolve_threads(threads);
  (void)nt;
#pragma omp parallel for schedule(static) num_threads(nt)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int p = 0; p < k; ++p) {
        const float av = lut_a[a[(size_t)i * k + p]];
        const float bv = lut_b[b_transposed ? b[(size_t)j * k + p] : b[(size_t)p * n + j]];
        acc += av * bv;
      }
      acc *= combined;
      if (bias) acc += load_as_f32(bias, (size_t)j, out_dt);
      acc = act_f32(acc, act);
      if (residual) acc += load_as_f32(residual, (size_t)i * n + j, out_dt);
      store_from_f32(out, (size_t)i * n + j, out_dt, acc);
    }
}

// ------------------------------------------------------------------ the ops, per dtype
// mode 0 ("f32acc"): widen, accumulate in f32, epilogue in f32, narrow once — what numr's
//   matmul / matmul_bias do for every float type and what its CUDA tensor-core kernels do.
// mode 1 ("literal"): numr's CPU epilogue-op loops for non-f32 types: out = bias (+ residual),
//   then out = T(out + T(a*b)) in i-k-j order with every step rounded to T, activation through
//   f64. Only meaningful for small K.
// One matrix (no batch); B is [K,N] (b_transposed = 0) or [N,K] (1). Returns 0 on success.
ORC_API int orc_gemm(int dt, int mode, const void* a, const void* b, const void* bias, const void* residual,
                     void* out, int m, int n, int k, int b_transposed, int act, int threads) {
  if (m <= 0 || n <= 0) return 0;
  if (dt == DT_I8) {
    if (act != ACT_NONE || residual) return 2;
    orc_matmul_i8_i32((const int8_t*)a, (const int8_t*)b, (const int32_t*)bias, (int32_t*)out, m, n, k,
                      b_transposed, threads);
    return 0;
  }
  const size_t mn = (size_t)m * n;
  if (dt == DT_F32) {
    float* c = (float*)out;
    if (!residual) {
      orc_matmul_f32((const float*)a, (const float*)b, (const float*)bias, c, m, n, k, k,
                     b_transposed ? k : n, n, b_transposed, threads);
      if (act != ACT_NONE) for (size_t i = 0; i < mn; ++i) c[i] = act_f32(c[i], act);
    } else {
      // matmul_bias_residual: out = bias + residual, then i-k-j accumulation in f32.
      const float* bi = (const float*)bias; const float* re = (const float*)residual;
      const float* A = (const float*)a; const float* B = (const float*)b;
      for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) c[(size_t)i * n + j] = (bi ? bi[j] : 0.0f) + re[(size_t)i * n + j];
#pragma omp parallel for schedule(static)
      for (int i = 0; i < m; ++i)
        for (int p = 0; p < k; ++p) {
          const float av = A[(size_t)i * k + p];
          float* crow = c + (size_t)i * n;
          if (!b_transposed) { const float* brow = B + (size_t)p * n; for (int j = 0; j < n; ++j) crow[j] += av * brow[j]; }
          else for (int j = 0; j < n; ++j) crow[j] += av * B[(size_t)j * k + p];
        }
      if (act != ACT_NONE) return 2;
    }
    return 0;
  }
  if (mode == 0) {
    std::vector<float> af((size_t)m * k), bf((size_t)k * n), cf(mn), biasf;
    orc_decode(a, af.data(), af.size(), dt);
    orc_decode(b, bf.data(), bf.size(), dt);
    if (bias) { biasf.resize(n); orc_decode(bias, biasf.data(), n, dt); }
    orc_matmul_f32(af.data(), bf.data(), bias ? biasf.data() : nullptr, cf.data(), m, n, k, k,
                   b_transposed ? k : n, n, b_transposed, threads);
    for (size_t i = 0; i < mn; ++i) {
      float x = act_f32(cf[i], act);
      if (residual) x += load_as_f32(residual, i, dt);
      store_from_f32(out, i, dt, x);
    }
    return 0;
  }
  // literal mode: every intermediate lives in T.
  auto rnd = [dt](float v) { uint64_t tmp = 0; store_from_f32(&tmp, 0, dt, v); return load_as_f32(&tmp, 0, dt); };
  std::vector<float> c(mn);
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      float v = bias ? load_as_f32(bias, j, dt) : 0.0f;
      if (residual) v = rnd(v + load_as_f32(residual, (size_t)i * n + j, dt));
      c[(size_t)i * n + j] = v;
    }
  for (int i = 0; i < m; ++i)
    for (int p = 0; p < k; ++p) {
      const float av = load_as_f32(a, (size_t)i * k + p, dt);
      for (int j = 0; j < n; ++j) {
        const float bv = load_as_f32(b, b_transposed ? (size_t)j * k + p : (size_t)p * n + j, dt);
        float& o = c[(size_t)i * n + j];
        o = rnd(o + rnd(av * bv));
      }
    }
  for (size_t i = 0; i < mn; ++i) {
    float v = c[i];
    if (act == ACT_RELU) v = v < 0.0f ? 0.0f : v;
    else if (act != ACT_NONE) {
      // T::from_f64: one rounding from the f64 result (double -> float -> T can double round only
      // on exact ties of the narrower format, which a transcendental result does not hit).
      v = (float)act_f64((double)v, act);
    }
    store_from_f32(out, i, dt, v);
  }
  return 0;
}

// ------------------------------------------------------------------ f64 ground truth
// out64 = act(scale * (A @ B) + bias) + residual on the decoded operands, all in f64.
// Only rows listed in `rows` (n_rows of them; NULL = all rows) are computed, into
// out64[r * n + j] for the r-th listed row.
ORC_API void orc_truth_f64(int a_dt, int b_dt, int epi_dt, const void* a, const void* b, const void* bias,
                           const void* residual, double* out64, int m, int n, int k, int b_transposed,
                           double scale, int act, const int* rows, int n_rows, int threads) {
  const int count = rows ? n_rows : m;
  const int nt = resolve_threads(threads);
  (void)nt;
  std::vector<double> bd((size_t)k * n);   // decoded B as [K][N]
#pragma omp parallel for schedule(static) num_threads(nt)
  for (int p = 0; p < k; ++p)
    for (int j = 0; j < n; ++j)
      bd[(size_t)p * n + j] = (double)load_as_f32(b, b_transposed ? (size_t)j * k + p : (size_t)p * n + j, b_dt);
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
  for (int r = 0; r < count; ++r) {
    const int i = rows ? rows[r] : r;
    double* orow = out64 + (size_t)r * n;
    for (int j = 0; j < n; ++j) orow[j] = 0.0;
    for (int p = 0; p < k; ++p) {
      const double av = (double)load_as_f32(a, (size_t)i * k + p, a_dt);
      const double* brow = bd.data() + (size_t)p * n;
      for (int j = 0; j < n; ++j) orow[j] += av * brow[j];
    }
    for (int j = 0; j < n; ++j) {
      double x = orow[j] * scale;
      if (bias) x += (double)load_as_f32(bias, (size_t)j, epi_dt);
      x = act_f64(x, act);
      if (residual) x += (double)load_as_f32(residual, (size_t)i * n + j, epi_dt);
      orow[j] = x;
    }
  }
}

// ------------------------------------------------------------------ wide-integer matmul
// I16 / I32 / I64 / U8 / U16 / U32 / U64 (and I8 -> I8, unused by numr): a SIGNED 128-bit accumulator
// for every element type, seeded by the bias, products added in k order with i128 saturating
// multiply and add, one saturating narrow at the store
// (src/runtime/cpu/kernels/matmul/kernel.rs:145-175 `matmul_scalar_acc::<T, i128>`,
// src/runtime/cpu/kernels/wide_acc.rs:109-135, src/runtime/cuda/kernels/matmul_int.cu:1-104).
typedef __int128 i128_t;
typedef unsigned __int128 u128_t;
static const i128_t kI128Max = (i128_t)(~(u128_t)0 >> 1);
static const i128_t kI128Min = -kI128Max - 1;

static inline i128_t sat_add_i128(i128_t a, i128_t b) {
  i128_t r;
  if (__builtin_add_overflow(a, b, &r)) return a < 0 ? kI128Min : kI128Max;
  return r;
}
static inline i128_t sat_mul_i128(i128_t a, i128_t b) {
  i128_t r;
  if (__builtin_mul_overflow(a, b, &r)) return ((a < 0) != (b < 0)) ? kI128Min : kI128Max;
  return r;
}

template <typename T>
static void matmul_wide(const T* a, const T* b, const T* bias, T* c, int m, int n, int k, int b_transposed) {
  const bool sg = static_cast<T>(-1) < static_cast<T>(0);
  const int bits = sizeof(T) * 8;
  const i128_t hi = sg ? (((i128_t)1 << (bits - 1)) - 1) : (((i128_t)1 << bits) - 1);
  const i128_t lo = sg ? (-hi - 1) : (i128_t)0;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      i128_t acc = bias ? (i128_t)bias[j] : (i128_t)0;
      for (int p = 0; p < k; ++p) {
        const i128_t x = (i128_t)a[(size_t)i * k + p];
        const i128_t y = (i128_t)(b_transposed ? b[(size_t)j * k + p] : b[(size_t)p * n + j]);
        acc = sat_add_i128(acc, sat_mul_i128(x, y));
      }
      c[(size_t)i * n + j] = (T)(acc > hi ? hi : (acc < lo ? lo : acc));
    }
}

ORC_API int orc_matmul_wide_int(int elem, int is_signed, const void* a, const void* b, const void* bias, void* c,
                                int m, int n, int k, int b_transposed) {
  switch (elem * 2 + (is_signed ? 1 : 0)) {
    case 3: matmul_wide<int8_t>((const int8_t*)a, (const int8_t*)b, (const int8_t*)bias, (int8_t*)c, m, n, k, b_transposed); return 0;
    case 2: matmul_wide<uint8_t>((const uint8_t*)a, (const uint8_t*)b, (const uint8_t*)bias, (uint8_t*)c, m, n, k, b_transposed); return 0;
    case 5: matmul_wide<int16_t>((const int16_t*)a, (const int16_t*)b, (const int16_t*)bias, (int16_t*)c, m, n, k, b_transposed); return 0;
    case 4: matmul_wide<uint16_t>((const uint16_t*)a, (const uint16_t*)b, (const uint16_t*)bias, (uint16_t*)c, m, n, k, b_transposed); return 0;
    case 9: matmul_wide<int32_t>((const int32_t*)a, (const int32_t*)b, (const int32_t*)bias, (int32_t*)c, m, n, k, b_transposed); return 0;
    case 8: matmul_wide<uint32_t>((const uint32_t*)a, (const uint32_t*)b, (const uint32_t*)bias, (uint32_t*)c, m, n, k, b_transposed); return 0;
    case 17: matmul_wide<int64_t>((const int64_t*)a, (const int64_t*)b, (const int64_t*)bias, (int64_t*)c, m, n, k, b_transposed); return 0;
    case 16: matmul_wide<uint64_t>((const uint64_t*)a, (const uint64_t*)b, (const uint64_t*)bias, (uint64_t*)c, m, n, k, b_transposed); return 0;
    default: return 2;
  }
}

// ---------------------------------------------------------------- convolutions (direct form)
// numr's CPU convolution kernels, restated: conv2d (conv1d is the 1-row case) follows
// src/runtime/cpu/kernels/conv.rs:199-262 (loops oc, oy, ox outside; ic, ky, kx inside; bias added
// last) and conv_transpose1d follows src/runtime/cpu/kernels/conv_transpose.rs:75-117 (for an output
// position and a tap, the input sample (ot + pad_left - k*dilation) / stride when that is a
// non-negative multiple of the stride inside the input; weight [c_in, c_out, k]). groups = 1, the case
// the GEMM formulation covers. Accumulation in f32 with one narrowing, or (truth = 1) in float64 with
// a float64 result.
template <typename Acc>
static void conv_direct(int dt, int transposed, const void* in, const void* w, const void* bias, void* out,
                        double* out64, int batch, int c_in, int c_out, int in_h, int in_w, int kh, int kw,
                        int out_h, int out_w, int stride_h, int stride_w, int pad_top, int pad_left, int dil_h,
                        int dil_w, int threads) {
  const int nt = resolve_threads(threads);
  const long long total = (long long)batch * c_out;
#pragma omp parallel for schedule(static) num_threads(nt)
  for (long long bo = 0; bo < total; ++bo) {
    const int b = (int)(bo / c_out), oc = (int)(bo % c_out);
    for (int oy = 0; oy < out_h; ++oy) {
      for (int ox = 0; ox < out_w; ++ox) {
        Acc sum = 0;
        if (!transposed) {
          for (int ic = 0; ic < c_in; ++ic)
            for (int ky = 0; ky < kh; ++ky)
              for (int kx = 0; kx < kw; ++kx) {
                const int iy = oy * stride_h + ky * dil_h - pad_top, ix = ox * stride_w + kx * dil_w - pad_left;
                if (iy < 0 || iy >= in_h || ix < 0 || ix >= in_w) continue;
                const Acc x = load_as_f32(in, (((size_t)b * c_in + ic) * in_h + iy) * in_w + ix, dt);
                const Acc wv = load_as_f32(w, (((size_t)oc * c_in + ic) * kh + ky) * kw + kx, dt);
                sum += x * wv;
              }
        } else {
          for (int k = 0; k < kw; ++k) {
            const int num = ox + pad_left - k * dil_w;
            if (num < 0 || num % stride_w != 0) continue;
            const int l = num / stride_w;
            if (l >= in_w) continue;
            for (int ic = 0; ic < c_in; ++ic) {
              const Acc x = load_as_f32(in, ((size_t)b * c_in + ic) * in_w + l, dt);
              const Acc wv = load_as_f32(w, ((size_t)ic * c_out + oc) * kw + k, dt);
              sum += x * wv;
            }
          }
        }
        if (bias) sum += (Acc)load_as_f32(bias, (size_t)oc, dt);
        const size_t o = (((size_t)b * c_out + oc) * out_h + oy) * out_w + ox;
        if (out64) out64[o] = (double)sum;
        else store_from_f32(out, o, dt, (float)sum);
      }
    }
  }
}

ORC_API void orc_conv(int dt, int transposed, int truth, const void* in, const void* w, const void* bias, void* out,
                      int batch, int c_in, int c_out, int in_h, int in_w, int kh, int kw, int out_h, int out_w,
                      int stride_h, int stride_w, int pad_top, int pad_left, int dil_h, int dil_w, int threads) {
  if (truth)
    conv_direct<double>(dt, transposed, in, w, bias, nullptr, static_cast<double*>(out), batch, c_in, c_out, in_h,
                        in_w, kh, kw, out_h, out_w, stride_h, stride_w, pad_top, pad_left, dil_h, dil_w, threads);
  else
    conv_direct<float>(dt, transposed, in, w, bias, out, nullptr, batch, c_in, c_out, in_h, in_w, kh, kw, out_h,
                       out_w, stride_h, stride_w, pad_top, pad_left, dil_h, dil_w, threads);
}

ORC_API int orc_max_threads(void) { return resolve_threads(0); }
