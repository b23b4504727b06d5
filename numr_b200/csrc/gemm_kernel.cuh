// Persistent, warp-specialised tcgen05 GEMM with a fused epilogue for sm_100a.
//
// One CTA per SM walks a rasterised list of 128 x tile_n output tiles. Roles:
//   warp 0      TMA producer: streams 128-byte-wide K slices of A and B into a ring of
//               shared-memory stages (128-byte swizzle), one mbarrier per stage.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (UMMA 128 x tile_n x 32 bytes of K)
//               from shared-memory descriptors into one of two TMEM accumulators, and
//               commits stage releases / accumulator completion to mbarriers.
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (each warp owns the 32 TMEM
//               lanes its warp id allows), apply scale, bias, activation, residual, convert
//               once and store; the other accumulator is filled meanwhile.
// The same main loop serves every operand type, because a stage always holds 128 bytes
// of K per row: 64 bf16/f16, 32 f32 (TF32) or 128 fp8/int8 elements = 4 MMA steps.
//
// It replaces the reference's matmul_wmma* / matmul_f32_tiled / matmul_int / fp8_matmul
// kernels (src/runtime/cuda/kernels/matmul_wmma.cuh:283-412, matmul_f32_tiled.cuh:220-330,
// matmul_int.cu:105-222, fp8_matmul.cu:43-155) and their epilogue functors
// (matmul_wmma.cuh:243-276, gemm_epilogue.cu:1377-1395, gemm_activation.cuh:14-35).
#pragma once
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>

#include "epilogue_math.cuh"
#include "gemm_internal.h"
#include "gemm_params.h"
#include "sm100_ptx.cuh"

namespace nb {

struct TileCoord {
  uint32_t bi, m_blk, n_blk;
};

struct WorkUnit {
  uint32_t tile;       // output tile
  uint32_t kb0, kb1;   // stages [kb0, kb1) of K
  uint32_t split;      // index of this part of K, or 0xFFFFFFFF for a whole tile
  uint32_t slot;       // tail-tile index (valid when split != 0xFFFFFFFF)
  uint32_t n_off;      // first column of the unit inside its tile (0 unless the tile is cut along N)
  uint32_t width;      // columns the unit computes (UMMA N): tile_n, or cut_n for a column slice
  uint32_t narrow;     // 1: a column slice of a tile of the last wave
};

__device__ __forceinline__ WorkUnit work_unit(const KParams& p, uint32_t u, uint32_t krank = 0) {
  WorkUnit wu;
  wu.n_off = 0; wu.width = p.tile_n; wu.narrow = 0;
  if (p.kc > 1) {
    // K-split cluster: every CTA of the cluster works on tile u, each on its own range of K blocks;
    // the partial sums meet in the leader's shared memory (see the epilogue).
    wu.tile = u; wu.split = 0xFFFFFFFFu; wu.slot = 0;
    wu.kb0 = krank * p.kc_kbs;
    wu.kb1 = min(p.num_kb, wu.kb0 + p.kc_kbs);
  } else if (u < p.n_full) {
    wu.tile = u; wu.kb0 = 0; wu.kb1 = p.num_kb; wu.split = 0xFFFFFFFFu; wu.slot = 0;
  } else if (p.cut > 1) {
    // Last, partly filled wave: its tiles are cut along N into `cut` slices that run side by side
    // on workers that would otherwise idle. Every slice walks all of K, so the sums (and their
    // order) are those of the whole tile: no reduction, bitwise the same result.
    const uint32_t v = u - p.n_full;
    const uint32_t t = v / p.cut;
    wu.tile = p.n_full + t; wu.kb0 = 0; wu.kb1 = p.num_kb; wu.split = 0xFFFFFFFFu; wu.slot = 0;
    wu.n_off = (v - t * p.cut) * p.cut_n; wu.width = p.cut_n; wu.narrow = 1;
  } else {
    const uint32_t v = u - p.n_full;
    wu.slot = v / p.splits;
    wu.split = v - wu.slot * p.splits;
    wu.tile = p.n_full + wu.slot;
    wu.kb0 = wu.split * p.kb_per_split;
    wu.kb1 = min(p.num_kb, wu.kb0 + p.kb_per_split);
  }
  return wu;
}

__device__ __forceinline__ TileCoord tile_coord(const KParams& p, uint32_t t) {
  const uint32_t per_batch = p.tiles_m * p.tiles_n;
  TileCoord c;
  if (p.plan) {
    // Grouped: the plan cuts the row tiles into bands (consecutive tiles of one group); a band is
    // walked column by column before the next one starts. All tiles before a band belong to earlier
    // bands, so the band of tile slot t / tiles_n is the band unit t falls into.
    const int4 e = __ldg(p.plan + t / p.tiles_n);
    const uint32_t first = (uint32_t)e.w, size = (uint32_t)e.x >> 24;
    const uint32_t r = t - first * p.tiles_n;
    c.bi = 0;
    c.m_blk = first + r % size;
    c.n_blk = r / size;
    return c;
  }
  // (a division by a run-time value costs a lone thread about 0.1 us, and the first tile's coordinates
  // stand between every launch and its first load: the common cases divide as little as they can)
  c.bi = 0;
  uint32_t r = t;
  if (t >= per_batch) {
    c.bi = t / per_batch;
    r = t - c.bi * per_batch;
  }
  if (p.tiles_m == 1) {   // one row of tiles: no rasterisation groups to walk
    c.m_blk = 0;
    c.n_blk = r;
    return c;
  }
  const uint32_t group_span = p.group_m * p.tiles_n;
  uint32_t g = 0, in_g = r;
  if (r >= group_span) {
    g = r / group_span;
    in_g = r - g * group_span;
  }
  const uint32_t first_m = g * p.group_m;
  const uint32_t gsize = min(p.group_m, p.tiles_m - first_m);
  c.n_blk = in_g / gsize;
  c.m_blk = first_m + (in_g - c.n_blk * gsize);
  return c;
}

// Control block at the end of dynamic shared memory.
struct SmemCtrl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t teardown;
  uint64_t red_full;    // K-split cluster, in the leader: every peer has delivered its partial sums
  uint64_t red_empty;   // K-split cluster, in a peer: the leader has read this CTA's last partial sums
  uint32_t tmem_base;
  int abort;
  uint32_t last_flag;   // epilogue: this CTA delivered the last partial sum of a split tile
};
static_assert(sizeof(SmemCtrl) <= kSmemCtrlBytes, "control block too large");

template <int OUT>
struct OutType;
template <> struct OutType<OUT_F32> { using T = float; };
template <> struct OutType<OUT_BF16> { using T = __nv_bfloat16; };
template <> struct OutType<OUT_F16> { using T = __half; };
template <> struct OutType<OUT_E4M3> { using T = uint8_t; };
template <> struct OutType<OUT_E5M2> { using T = uint8_t; };
template <> struct OutType<OUT_I32> { using T = int32_t; };

// The arithmetic of the epilogue on W values of one output row: x[j] holds accumulator * scale + bias
// (+ the per-row bias) on entry and the finished value on return; res[j] is the residual (forward) or
// the incoming gradient (backward) when `has_res`. Written as passes over the W values, each free of
// branches, so that the W dependency chains interleave: a branch per element (forward or backward?
// residual or not?) makes the compiler finish one element before it starts the next, about 150 cycles
// per element for GELU, which made one 32-column chunk cost 3 - 4 us per warp. W = 8 keeps the live
// values well inside the register file.
constexpr int kFinishWidth = 8;
template <int ACT, int W>
__device__ __forceinline__ void activation_pass(float (&x)[W], bool derivative) {
  if (derivative) {
#pragma unroll
    for (int j = 0; j < W; ++j) x[j] = activation_derivative<ACT>(x[j]);
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j) x[j] = activation<ACT>(x[j]);
  }
}

template <int W>
__device__ __forceinline__ void finish_values(const KParams& p, float (&x)[W], const float (&res)[W], bool has_res) {
  // one uniform branch per W values selects the formula; the code around it exists once
  switch (p.act) {
    case NUMR_B200_ACT_RELU: activation_pass<NUMR_B200_ACT_RELU, W>(x, p.bwd != 0); break;
    case NUMR_B200_ACT_GELU: activation_pass<NUMR_B200_ACT_GELU, W>(x, p.bwd != 0); break;
    case NUMR_B200_ACT_SILU: activation_pass<NUMR_B200_ACT_SILU, W>(x, p.bwd != 0); break;
    case NUMR_B200_ACT_SIGMOID: activation_pass<NUMR_B200_ACT_SIGMOID, W>(x, p.bwd != 0); break;
    case NUMR_B200_ACT_TANH: activation_pass<NUMR_B200_ACT_TANH, W>(x, p.bwd != 0); break;
    default: activation_pass<NUMR_B200_ACT_NONE, W>(x, p.bwd != 0); break;
  }
  if (p.bwd) {
    if (has_res) {
#pragma unroll
      for (int j = 0; j < W; ++j) x[j] = res[j] * x[j];
    } else {
#pragma unroll
      for (int j = 0; j < W; ++j) x[j] = 0.0f * x[j];
    }
  } else if (has_res) {
#pragma unroll
    for (int j = 0; j < W; ++j) x[j] += res[j];
  }
}

// Finishes `ncols` (<= 32) accumulator values of one output row and stores them with plain stores:
// the path of outputs whose rows are not 16-byte aligned and of column groups that straddle a tile's
// edge. The activation is a template parameter, and the routine is a function of its own, not inlined
// at its call sites, so the main path's code stays small.
template <int OUT>
__device__ __noinline__ void finish_row_chunk(const KParams& p, const uint32_t (&acc)[32], size_t row_off,
                                              uint32_t col0, uint32_t ncols, float rb) {
  using T = typename OutType<OUT>::T;
  T* __restrict__ orow = static_cast<T*>(p.out) + row_off + col0;
  if constexpr (OUT == OUT_I32) {
    const int32_t* bias = static_cast<const int32_t*>(p.bias);
    if (ncols == 32 && p.vec_ok) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        int4 v;
        v.x = finish_i32(acc[j + 0], bias, col0 + j + 0);
        v.y = finish_i32(acc[j + 1], bias, col0 + j + 1);
        v.z = finish_i32(acc[j + 2], bias, col0 + j + 2);
        v.w = finish_i32(acc[j + 3], bias, col0 + j + 3);
        *reinterpret_cast<int4*>(orow + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < (int)ncols) orow[j] = finish_i32(acc[j], bias, col0 + j);
    }
  } else {
    // (a per-row bias arrives as `rb`; the per-column one is read here)
    const T* bias = p.bias_row ? nullptr : static_cast<const T*>(p.bias);
    const T* rrow = p.residual ? static_cast<const T*>(p.residual) + row_off + col0 : nullptr;
    constexpr int VEC = 16 / sizeof(T);   // elements per 16-byte store
    const bool vec = ncols == 32 && p.vec_ok;
    constexpr int W = VEC > kFinishWidth ? VEC : kFinishWidth;   // whole 16-byte vectors
    constexpr int NV = 32 / VEC;
    // the residual's 16-byte loads of the whole chunk are issued before the first use
    int4 resv[NV];
    if (rrow && vec) {
#pragma unroll
      for (int v = 0; v < NV; ++v) resv[v] = __ldg(reinterpret_cast<const int4*>(rrow) + v);
    }
#pragma unroll
    for (int g = 0; g < 32; g += W) {
      if (g < (int)ncols) {
        float res[W];
        T bv[W];
        if (rrow) {
          if (vec) {
#pragma unroll
            for (int e = 0; e < W; ++e) res[e] = vec_elem_f32<OUT>(resv[(g + e) / VEC], (g + e) % VEC);
          } else {
#pragma unroll
            for (int e = 0; e < W; ++e) res[e] = g + e < (int)ncols ? to_f32<OUT>(rrow[g + e]) : 0.0f;
          }
        }
        if (bias) {
#pragma unroll
          for (int e = 0; e < W; ++e) bv[e] = g + e < (int)ncols ? __ldg(bias + col0 + g + e) : T(0);
        }
        float x[W];
#pragma unroll
        for (int e = 0; e < W; ++e) x[e] = __uint_as_float(acc[g + e]) * p.scale + rb;
        if (bias) {
#pragma unroll
          for (int e = 0; e < W; ++e) x[e] += to_f32<OUT>(bv[e]);
        }
        finish_values<W>(p, x, res, rrow != nullptr);
        if (vec) {
#pragma unroll
          for (int e = 0; e < W; e += VEC) *reinterpret_cast<uint4*>(orow + g + e) = pack_out<OUT>(x + e);
        } else {
#pragma unroll
          for (int e = 0; e < W; ++e)
            if (g + e < (int)ncols) orow[g + e] = from_f32<OUT>(x[e]);
        }
      }
    }
  }
}

template <bool PAIR>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1,
                                          int c2) {
  if constexpr (PAIR) tma_load_3d_pair(dst, tm, bar, c0, c1, c2);
  else tma_load_3d(dst, tm, bar, c0, c1, c2);
}

template <bool PAIR>
__device__ __forceinline__ void load_tile4(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c1, int c2,
                                           int c3) {
  if constexpr (PAIR) tma_load_4d_pair(dst, tm, bar, 0, c1, c2, c3);
  else tma_load_4d(dst, tm, bar, 0, c1, c2, c3);
}

template <int KIND, bool PAIR>
__device__ __forceinline__ void issue_mma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                          uint32_t accumulate) {
  if constexpr (PAIR) umma_pair<KIND>(d_tmem, a, b, idesc, accumulate);
  else umma<KIND>(d_tmem, a, b, idesc, accumulate);
}

// Arrival on barrier `bar` (a CTA-local address) once the MMAs issued so far have retired; in a
// pair the barrier at the same address in the peer CTA gets its own arrival.
template <bool PAIR>
__device__ __forceinline__ void commit_to(uint32_t bar) {
  if constexpr (PAIR) {
    umma_commit_pair_multicast(bar, (uint16_t)3);   // one instruction for both CTAs (two commits cost the issuer ~40 cycles more per stage)
  } else {
    umma_commit(bar);
  }
}

// Bias of the current tile as 32-bit values in shared memory: float for the float outputs
// (converted once per tile), raw int32 for the I8 path.
template <int OUT>
__device__ __forceinline__ void load_bias_tile(const KParams& p, uint32_t* bias_s, uint32_t n0,
                                               uint32_t width, uint32_t epi_tid) {
  using T = typename OutType<OUT>::T;
#pragma unroll
  for (uint32_t i = epi_tid; i < 256; i += 128) {
    const uint32_t col = n0 + i;
    uint32_t v = 0;
    if (p.bias && !p.bias_row && i < width && col < p.N) {
      if constexpr (OUT == OUT_I32) v = (uint32_t)__ldg(static_cast<const int32_t*>(p.bias) + col);
      else v = __float_as_uint(load_f32<OUT>(static_cast<const T*>(p.bias), col));
    }
    bias_s[i] = v;
  }
}

// Finishes 32 accumulator columns of one row (tile columns [tc0, tc0+32)) and writes them as
// 16-byte chunks into the warp's staging buffer: row `lane` at lane*128, chunk c of the row at
// position c ^ (lane & 7) (the 128-byte swizzle the output tensor map expects).
//
// The epilogue warps are bound by instruction issue (one warp per scheduler, nothing to switch to),
// so this is written for few instructions and no branches inside a group of 8 columns: the bias comes
// from shared memory four values at a time, scale and bias and the activation work on pairs of values
// (f32x2), narrowing converts two values at once, and the residual's 16-byte loads of `PRE` columns are
// issued together before the arithmetic that needs them. (With a branch per element, forward or
// backward, residual or not, the compiler finished one element before starting the next: 4600 cycles
// for 32 columns of GELU instead of 1000.)
template <int OUT, int ACT, bool BWD, bool RES, int PRE>
__device__ __forceinline__ void finish_chunk_to_stage(const KParams& p, const uint32_t (&acc)[32], uint32_t bias_addr,
                                                      uint32_t chunk0, uint32_t buf, uint32_t lane, const void* res_row,
                                                      uint32_t res_valid, float rb) {
  using T = typename OutType<OUT>::T;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int W = VEC > 8 ? VEC : 8;   // columns per group: whole 16-byte vectors
  constexpr int NV = PRE / VEC;
  const T* rrow = static_cast<const T*>(res_row);
  const float2 s2 = pair_of(p.scale), rb2 = pair_of(rb);
#pragma unroll
  for (int h = 0; h < 32; h += PRE) {
    int4 resv[NV];
    if constexpr (RES) {
#pragma unroll
      for (int v = 0; v < NV; ++v)   // (at the matrix's right edge: only the vectors that exist; rows are whole vectors)
        resv[v] = (uint32_t)(h + v * VEC) < res_valid ? __ldg(reinterpret_cast<const int4*>(rrow + h) + v) : make_int4(0, 0, 0, 0);
    }
#pragma unroll
    for (int g = h; g < h + PRE; g += W) {
      float x[W];
#pragma unroll
      for (int e = 0; e < W; e += 4) {
        const uint4 b = ld_shared_v4(bias_addr + (uint32_t)(g + e) * 4u);
        const float2 lo = __fadd2_rn(__ffma2_rn(make_float2(__uint_as_float(acc[g + e]), __uint_as_float(acc[g + e + 1])), s2,
                                                make_float2(__uint_as_float(b.x), __uint_as_float(b.y))), rb2);
        const float2 hi = __fadd2_rn(__ffma2_rn(make_float2(__uint_as_float(acc[g + e + 2]), __uint_as_float(acc[g + e + 3])), s2,
                                                make_float2(__uint_as_float(b.z), __uint_as_float(b.w))), rb2);
        x[e] = lo.x; x[e + 1] = lo.y; x[e + 2] = hi.x; x[e + 3] = hi.y;
      }
      float res[W];
#pragma unroll
      for (int e = 0; e < W; ++e) res[e] = RES ? vec_elem_f32<OUT>(resv[(g - h + e) / VEC], (g + e) % VEC) : 0.0f;
      if constexpr (BWD) {
#pragma unroll
        for (int e = 0; e < W; ++e) x[e] = res[e] * activation_derivative<ACT>(x[e]);
      } else {
#pragma unroll
        for (int e = 0; e < W; e += 2) {
          float2 y = activation2<ACT>(make_float2(x[e], x[e + 1]));
          if constexpr (RES) y = __fadd2_rn(y, make_float2(res[e], res[e + 1]));
          x[e] = y.x; x[e + 1] = y.y;
        }
      }
#pragma unroll
      for (int e = 0; e < W; e += VEC) {
        const uint32_t chunk = chunk0 + (uint32_t)(g + e) / VEC;
        st_shared_v4(buf + lane * 128u + ((chunk ^ (lane & 7u)) << 4), pack_out<OUT>(x + e));
      }
    }
  }
}

template <int OUT, bool BWD, bool RES, int PRE>
__device__ __forceinline__ void finish_to_stage_dir(const KParams& p, const uint32_t (&acc)[32], uint32_t bias_addr,
                                                    uint32_t chunk0, uint32_t buf, uint32_t lane, const void* res_row,
                                                    uint32_t res_valid, float rb) {
  switch (p.act) {   // once per 32 columns
    case NUMR_B200_ACT_RELU: finish_chunk_to_stage<OUT, NUMR_B200_ACT_RELU, BWD, RES, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb); break;
    case NUMR_B200_ACT_GELU: finish_chunk_to_stage<OUT, NUMR_B200_ACT_GELU, BWD, RES, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb); break;
    case NUMR_B200_ACT_SILU: finish_chunk_to_stage<OUT, NUMR_B200_ACT_SILU, BWD, RES, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb); break;
    case NUMR_B200_ACT_SIGMOID: finish_chunk_to_stage<OUT, NUMR_B200_ACT_SIGMOID, BWD, RES, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb); break;
    case NUMR_B200_ACT_TANH: finish_chunk_to_stage<OUT, NUMR_B200_ACT_TANH, BWD, RES, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb); break;
    default: finish_chunk_to_stage<OUT, NUMR_B200_ACT_NONE, BWD, RES, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb); break;
  }
}

// `LEAN`: for call sites that hold much other state (the exact-F32 sums): fewer residual loads in flight.
template <int OUT, bool LEAN = false>
__device__ __forceinline__ void finish_to_stage(const KParams& p, const uint32_t (&acc)[32],
                                                const uint32_t* bias_s, uint32_t tc0, uint32_t chunk0,
                                                uint32_t buf, uint32_t lane, const void* res_row,
                                                bool res_vec, uint32_t res_valid, float rb) {
  using T = typename OutType<OUT>::T;
  constexpr int VEC = 16 / sizeof(T);
  if constexpr (OUT == OUT_I32) {
    // accumulator + bias with ONE saturation to the int32 range (matmul_int.cu:87-103): the saturating
    // 32-bit add is exactly clamp(a + b) of the wide sum
    const uint32_t bias_addr = smem_u32(bias_s) + tc0 * 4u;
#pragma unroll
    for (int j = 0; j < 32; j += VEC) {
      const uint4 b = ld_shared_v4(bias_addr + (uint32_t)j * 4u);
      const uint32_t chunk = chunk0 + (uint32_t)j / VEC;
      st_shared_v4(buf + lane * 128u + ((chunk ^ (lane & 7u)) << 4),
                   make_uint4(add_sat_s32(acc[j], b.x), add_sat_s32(acc[j + 1], b.y), add_sat_s32(acc[j + 2], b.z),
                              add_sat_s32(acc[j + 3], b.w)));
    }
  } else {
    constexpr int W = VEC > 8 ? VEC : 8;
    constexpr int PRE = LEAN ? W : (sizeof(T) == 4 ? 16 : 32);
    const uint32_t bias_addr = smem_u32(bias_s) + tc0 * 4u;
    (void)res_vec;
    if (p.bwd) {
      if (res_row) finish_to_stage_dir<OUT, true, true, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb);
      else finish_to_stage_dir<OUT, true, false, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb);
    } else {
      if (res_row) finish_to_stage_dir<OUT, false, true, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb);
      else finish_to_stage_dir<OUT, false, false, PRE>(p, acc, bias_addr, chunk0, buf, lane, res_row, res_valid, rb);
    }
  }
}

// I8 with K beyond the exact range of one s32 accumulator (K * 128 * 128 < 2^31): the MMA issuer
// accumulates K in TMEM in chunks of at most 65536 values and this routine adds the chunk sums of one
// work unit in 64 bits; bias and the one saturation come last, as the reference's i64 accumulator does
// (src/runtime/cuda/kernels/matmul_int.cu:87-103). A rare shape: plain stores, and a function of its
// own so that its 128 64-bit sums per thread do not weigh on the register allocation of the kernel.
template <bool PAIR>
__device__ __noinline__ uint32_t i8_long_k_unit(const KParams& p, SmemCtrl* ctrl, WaitCtx w, uint32_t tmem_base,
                                                uint32_t quarter, uint32_t lane, bool leader, uint32_t kb_first,
                                                uint32_t kb_last, uint32_t width, uint32_t n0, uint32_t n_end,
                                                size_t row_off, bool row_ok, uint32_t acc, uint32_t acc_phase) {
  // returns acc | acc_phase << 1 | live << 2 (state is passed by value so the caller keeps it in registers)
  bool live = true;
  long long sum[4][32];
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int j = 0; j < 32; ++j) sum[q][j] = 0;
  for (uint32_t kb0 = kb_first; live && kb0 < kb_last; kb0 += p.chunk_kb) {
    if (!mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, w, KSTAT_TIMEOUT_EPILOGUE)) { live = false; break; }
    tc_fence_after();
    const uint32_t taddr = tmem_base + acc * kAccStride + ((quarter * 32u) << 16);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if ((uint32_t)q * 32 < width && n0 + q * 32 < n_end) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + q * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[q][j] += (long long)(int32_t)r[j];
      }
    }
    // this warp is done reading accumulator `acc`
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      if (leader) mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
      else mbar_arrive_cluster(mapa(smem_u32(&ctrl->tmem_empty[acc]), 0));
    }
    acc ^= 1;
    if (acc == 0) acc_phase ^= 1;
  }
  if (live && row_ok) {
    const int32_t* bias = static_cast<const int32_t*>(p.bias);
    int32_t* orow = static_cast<int32_t*>(p.out) + row_off;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const uint32_t col = n0 + q * 32 + j;
        if ((uint32_t)q * 32 + j < width && col < n_end) {
          long long v = sum[q][j] + (bias ? (long long)__ldg(bias + col) : 0ll);
          v = v > 2147483647ll ? 2147483647ll : v;
          v = v < -2147483648ll ? -2147483648ll : v;
          orow[col] = (int32_t)v;
        }
      }
    }
  }
  return acc | (acc_phase << 1) | (live ? 4u : 0u);
}

// Timeline marks for experiments, compiled in only with -DNUMR_B200_TRACE (the marks inside the
// producer's and the MMA issuer's loops cost the normal build about 6 % on long-K problems): when
// KParams::trace is set (NUMR_B200_TRACE_PTR), the first 8 CTAs
// write the global timer and the SM's cycle counter at a few points of their life into
// trace[(cta * 16 + mark) * 2 + {0, 1}]. Off otherwise.
enum : uint32_t { TR_ENTRY = 0, TR_SETUP = 1, TR_DEPS = 2, TR_FIRST_LOAD = 3, TR_FIRST_FULL = 4, TR_LAST_MMA = 5,
                  TR_FIRST_ACC = 6, TR_LAST_STORE = 7, TR_STORES_READ = 8, TR_DONE = 9, TR_E_BIAS = 10,
                  TR_E_LD = 11, TR_E_FIN = 12, TR_E_ST = 13,
                  TR_UNIT0 = 10 /* 10..15: the start of the MMA issuer's first six units */ };
__device__ __forceinline__ void trace_mark(const KParams& p, uint32_t mark) {
#ifdef NUMR_B200_TRACE
  if (p.trace && blockIdx.x < 8) {
    p.trace[(blockIdx.x * 16 + mark) * 2] = global_timer_ns();
    p.trace[(blockIdx.x * 16 + mark) * 2 + 1] = (unsigned long long)clock64();
  }
#else
  (void)p; (void)mark;
#endif
}

// The MMA issuer's whole life (warp 1 of the leader CTA), a function of its own that is not inlined:
// the issue loop is sensitive to how the compiler treats it (descriptors in uniform registers, no
// moves between register files on the way to the MMA), and as a separate function its code does not
// change when the epilogue's does.
template <int KIND, bool PAIR>
__device__ __noinline__ void mma_issuer_role(const KParams& p, SmemCtrl* ctrl, uint32_t smem_base, uint32_t tmem_base,
                                            uint32_t worker, uint32_t num_workers, uint32_t krank, uint32_t lane,
                                            WaitCtx w) {
  const uint32_t parts = p.split3 ? 2u : 1u;
  if (p.plan) grid_dependency_wait();   // the only global memory this role reads
  // The whole warp walks the loop in step and one elected lane issues: descriptors and
  // addresses are then warp-uniform values the compiler keeps in uniform registers, which the
  // MMA instruction reads directly. (Issuing from inside a one-lane branch costs a
  // register-to-uniform move per operand, about 110 ns per MMA.) Waits are done by lane 0 and
  // their outcome is broadcast, so the warp stays converged.
  const uint32_t num_kb = p.num_kb, stages = p.stages, split3 = p.split3;
  (void)num_kb;
  const uint32_t a_hi32 = (1024u >> 4) | (1u << 14) | (2u << 29);
  const uint32_t b_hi32 = ((p.b_sbo >> 4) & 0x3FFF) | (1u << 14) | ((p.b_swizzle & 7) << 29);
  const uint32_t a_lo_fixed = (16u >> 4) << 16;
  const uint32_t b_lo_fixed = ((p.b_lbo >> 4) & 0x3FFF) << 16;
  const uint32_t stage_units = p.stage_bytes >> 4;
  const uint32_t a_units0 = (smem_base & 0x3FFFF) >> 4;
  const uint32_t ks = p.ks;
  const uint32_t b_off_units = (parts * ks * p.a_kk_bytes) >> 4;
  const uint32_t b_step_units = p.b_kstep_bytes >> 4;
  const uint32_t a_part_units = (ks * p.a_kk_bytes) >> 4;
  const uint32_t a_kk_units = p.a_kk_bytes >> 4;
  const uint32_t b_mn_major = p.b_mn_major;
  const uint32_t full0 = smem_u32(&ctrl->full[0]);
  const uint32_t empty0 = smem_u32(&ctrl->empty[0]);
  auto desc = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | lo; };
  auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
    uint32_t ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, w, code) ? 1u : 0u;
    return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
  };

  uint32_t stage = 0, phase = 0;
  uint32_t a_units = a_units0;       // stage base of A in 16-byte units
  uint32_t acc = 0, acc_phase = 0;
  bool ok = true;
  bool ready = false;   // outcome of the early test of the stage about to be used
  bool traced_full = false;
  uint32_t traced_units = 0;
  const uint32_t chunk_kb = p.chunk_kb ? p.chunk_kb : num_kb;
  for (uint32_t u = worker; ok && u < p.units_total; u += num_workers) {
   const WorkUnit wu = work_unit(p, u, krank);
   const TileCoord tc = tile_coord(p, wu.tile);
   if (p.plan) {   // empty row tile
     const int4 e = __ldg(p.plan + tc.m_blk);
     if (e.z <= e.y) continue;
   }
   if (tc.n_blk * p.tile_n + wu.n_off >= p.N) continue;       // a slice past the last column
   // Per unit: the instruction descriptor (UMMA N) and the spacing of B's K blocks and parts.
   const uint32_t idesc = wu.narrow ? p.idesc2 : p.idesc;
   const uint32_t u_rows = wu.narrow ? p.b_rows_cta2 : p.b_rows_cta;
   const uint32_t b_kk_units = b_mn_major ? (p.b_kk_bytes >> 4) : ((u_rows * kRowBytes) >> 4);
   const uint32_t b_part_units = (ks * u_rows * kRowBytes) >> 4;
   // One accumulator per chunk of K: the unit's whole K range normally; in exact-F32 mode a few
   // stages, which the epilogue then adds up in registers (see the epilogue).
   for (uint32_t kb0 = wu.kb0; ok && kb0 < wu.kb1; kb0 += chunk_kb) {
    if (!wait_all(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1, KSTAT_TIMEOUT_MMA_TMEM)) {
      ok = false;
      break;
    }
    tc_fence_after();
    if (kb0 == wu.kb0 && lane == 0 && traced_units < 6) trace_mark(p, TR_UNIT0 + traced_units++);
    const uint32_t d_tmem = tmem_base + acc * kAccStride;
    const uint32_t kb_end = min(wu.kb1, kb0 + chunk_kb);
    for (uint32_t kb = kb0; kb < kb_end; kb += ks) {
      // Every lane waits for the stage (the test issued before the previous stage's MMAs usually
      // answers it already); one vote keeps the outcome uniform should a wait run out.
      bool got = ready;
      if (!got) got = mbar_wait(full0 + stage * 8u, phase, w, KSTAT_TIMEOUT_MMA_FULL);
      if (!__all_sync(0xFFFFFFFFu, got)) {
        ok = false;
        break;
      }
      if (!traced_full) { traced_full = true; if (lane == 0) trace_mark(p, TR_FIRST_FULL); }
      {
        uint32_t ns = stage + 1, np = phase;
        if (ns == stages) { ns = 0; np ^= 1; }
        ready = mbar_test_wait(full0 + ns * 8u, np);   // looked at while the MMAs below are issued
      }
      const uint32_t kk_end = min(ks, kb_end - kb);
      // Warp-uniform operand descriptors of the stage's K blocks, computed by the whole warp (see
      // above); the elected lane then only issues.
      uint32_t al[4], bl[4];
#pragma unroll
      for (uint32_t kk = 0; kk < 4; ++kk) {
        al[kk] = (a_units + kk * a_kk_units) | a_lo_fixed;
        bl[kk] = (a_units + b_off_units + kk * b_kk_units) | b_lo_fixed;
      }
      const uint32_t first = kb - kb0;
      if (elect_one()) {
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {
          if (kk < kk_end) {
            if (!split3) {
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j)
                issue_mma<KIND, PAIR>(d_tmem, desc(a_hi32, al[kk] + j * 2u),
                                      desc(b_hi32, bl[kk] + j * b_step_units), idesc, (first | kk | j) ? 1u : 0u);
            } else {
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j) {
                const uint64_t a_hi = desc(a_hi32, al[kk] + j * 2u);
                const uint64_t a_lo = desc(a_hi32, al[kk] + a_part_units + j * 2u);
                const uint64_t b_hi = desc(b_hi32, bl[kk] + j * b_step_units);
                const uint64_t b_lo = desc(b_hi32, bl[kk] + b_part_units + j * b_step_units);
                issue_mma<KIND, PAIR>(d_tmem, a_lo, b_hi, idesc, (first | kk | j) ? 1u : 0u);
                issue_mma<KIND, PAIR>(d_tmem, a_hi, b_lo, idesc, 1u);
                issue_mma<KIND, PAIR>(d_tmem, a_hi, b_hi, idesc, 1u);
              }
            }
          }
        }
        commit_to<PAIR>(empty0 + stage * 8u);   // frees the stage (in both CTAs) once these MMAs retire
      }
      __syncwarp();
      a_units += stage_units;
      if (++stage == stages) { stage = 0; phase ^= 1; a_units = a_units0; }
    }
    if (!ok) break;
    // accumulator complete (both CTAs' epilogues); a test can withhold this one arrival to see
    // the epilogue's bounded wait run out
    if (elect_one() && !p.test_hold) commit_to<PAIR>(smem_u32(&ctrl->tmem_full[acc]));
    __syncwarp();
    acc ^= 1;
    if (acc == 0) acc_phase ^= 1;
   }
  }
  if (lane == 0) trace_mark(p, TR_LAST_MMA);
  // All MMAs issued by the elected lane must retire before TMEM is released.
  if (elect_one()) {
    if constexpr (PAIR) umma_commit_pair(smem_u32(&ctrl->teardown)); else umma_commit(smem_u32(&ctrl->teardown));
    const uint64_t t0 = global_timer_ns();
    while (!mbar_try_wait(smem_u32(&ctrl->teardown), 0)) {
      if (global_timer_ns() - t0 > p.limit_ns) {
        atomicCAS(p.status, 0, KSTAT_TIMEOUT_TEARDOWN);
        break;
      }
    }
  }
  __syncwarp();
}

template <int KIND, int OUT, bool PAIR>
__global__ void __launch_bounds__(192, 1) gemm_tcgen05_kernel(const __grid_constant__ KParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // ring of stages | partial sums of a K-split cluster (leader) | epilogue staging (4 warps x 2 x 4 KB) |
  // bias tile | control block
  const uint32_t ring_bytes = p.stages * p.stage_bytes;
  const uint32_t red_base = smem_base + ring_bytes;
  const uint32_t epi_base = red_base + p.red_bytes;
  uint32_t* bias_s = reinterpret_cast<uint32_t*>(smem_gen + ring_bytes + p.red_bytes + kEpiStageBytes);
  SmemCtrl* ctrl = reinterpret_cast<SmemCtrl*>(smem_gen + ring_bytes + p.red_bytes + kEpiStageBytes + kBiasTileBytes);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (threadIdx.x == 0) trace_mark(p, TR_ENTRY);
  // In a pair, CTA rank 0 (the leader) issues the MMAs for both; each CTA loads its own operand
  // halves and finishes its own 128 rows. Work is dealt to pairs (or to single CTAs).
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  // K-split cluster (single-CTA tiles only): `kc` CTAs share a tile, CTA `krank` takes K range krank.
  const uint32_t kc = PAIR ? 1u : p.kc;
  const uint32_t krank = (!PAIR && kc > 1) ? cluster_ctarank() : 0u;
  const uint32_t worker = PAIR ? blockIdx.x >> 1 : blockIdx.x / kc;
  const uint32_t num_workers = PAIR ? gridDim.x >> 1 : gridDim.x / kc;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[b]), PAIR ? 8 : 4);
    }
    mbar_init(smem_u32(&ctrl->teardown), 1);
    mbar_init(smem_u32(&ctrl->red_full), (kc > 1 ? kc - 1 : 1) * 128);
    mbar_init(smem_u32(&ctrl->red_empty), 128);
    ctrl->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&p.tmA);
    prefetch_tensormap(&p.tmB);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(&ctrl->tmem_base), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR || kc > 1) {   // the peer's barriers must exist before anything signals them
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  // Set-up is done without touching global memory. From here on the kernel reads what earlier work in
  // the stream wrote (operands, workspace, plan) and overwrites buffers that work may still read: every
  // thread that touches global memory waits for that work first, each role as late as it can (the
  // producer after it has worked out its first tile, the epilogue warps before they read the bias, the
  // MMA issuer only if it reads a plan). The next kernel in the stream may start its own set-up on SMs
  // this one has left.
  if (threadIdx.x == 0) trace_mark(p, TR_SETUP);
  grid_launch_dependents();

  WaitCtx w{p.status, &ctrl->abort, p.limit_ns};
  const uint32_t parts = p.split3 ? 2u : 1u;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t stages = p.stages, stage_bytes = p.stage_bytes;
      const uint32_t kb_elems = p.kb_elems, b_tile_bytes = p.b_tile_bytes, tile_n = p.tile_n;
      const uint32_t b_mn_major = p.b_mn_major, b_panels = p.b_panels, b_panel_n = p.b_panel_n;
      const uint32_t a_batch = p.a_batch, b_batch = p.b_batch;
      const uint32_t ks = p.ks, map4 = p.map4;
      const uint32_t panel_bytes = ks * kb_elems * kRowBytes;
      const uint32_t a_part_bytes = ks * p.a_kk_bytes;
      (void)b_tile_bytes; (void)b_panels;
      const uint32_t full0 = smem_u32(&ctrl->full[0]);
      const uint32_t empty0 = smem_u32(&ctrl->empty[0]);
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;   // stages armed so far (for the teardown drain)
      bool ok = true;
      bool ready = false;    // outcome of the early test of the stage about to be refilled
      bool waited = p.plan != nullptr;   // (a plan is itself the output of the kernel before this one)
      if (waited) grid_dependency_wait();
      for (uint32_t u = worker; ok && u < p.units_total; u += num_workers) {
        const WorkUnit wu = work_unit(p, u, krank);
        const TileCoord c = tile_coord(p, wu.tile);
        const int a_bi = c.bi ? (int)(c.bi % a_batch) : 0;
        int b_bi = c.bi ? (int)(c.bi % b_batch) : 0;
        int m0 = (int)(c.m_blk * p.tile_m + cta_rank * kTileM);
        if (p.plan) {   // grouped: this row tile's rows and weight come from the plan
          const int4 e = __ldg(p.plan + c.m_blk);
          if (e.z <= e.y) continue;
          // the tile lies on the absolute row grid (rows of a neighbouring group inside it are loaded
          // and computed, never stored): every TMA row coordinate stays a multiple of the tile height
          m0 = (int)((uint32_t)e.y / p.tile_m * p.tile_m + cta_rank * kTileM);
          b_bi = e.x & 0xFFFFFF;
        }
        if (c.n_blk * tile_n + wu.n_off >= p.N) continue;   // a slice past the last column: nothing to do
        // Rows of B this CTA loads for the unit, and what follows from them.
        const uint32_t u_rows = wu.narrow ? p.b_rows_cta2 : p.b_rows_cta;
        const uint32_t u_tx = wu.narrow ? p.tx_bytes2 : p.tx_bytes;
        const uint32_t b_part_bytes = ks * u_rows * kRowBytes;
        const uint32_t u_panels = b_mn_major ? u_rows / b_panel_n : 1u;
        const CUtensorMap* tm_b = (wu.narrow && !b_mn_major) ? &p.tmB2 : &p.tmB;
        const int n0 = (int)(c.n_blk * tile_n + wu.n_off + cta_rank * u_rows);
        int k0 = (int)(wu.kb0 * kb_elems);
        if (!waited) {   // the first tile's coordinates are known: now the operands must be
          grid_dependency_wait();
          waited = true;
          trace_mark(p, TR_DEPS);
        }
        for (uint32_t kb = wu.kb0; kb < wu.kb1; kb += ks, k0 += (int)(ks * kb_elems)) {
          if (!ready && !mbar_wait(empty0 + stage * 8u, phase ^ 1, w, KSTAT_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          {
            uint32_t ns = stage + 1, np = phase;
            if (ns == stages) { ns = 0; np ^= 1; }
            ready = mbar_test_wait(empty0 + ns * 8u, np ^ 1);   // answered while the copies below are issued
          }
          // A pair's loads are all credited to the leader's barrier, which the leader arms for both.
          const uint32_t bar = PAIR ? mapa(full0 + stage * 8u, 0) : full0 + stage * 8u;
          if (leader) mbar_arrive_expect_tx(full0 + stage * 8u, u_tx);
          if (++issued == 1) trace_mark(p, TR_FIRST_LOAD);
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + parts * a_part_bytes;
          for (uint32_t part = 0; part < parts; ++part) {
            const int az = a_bi + (int)(part * a_batch);
            if (map4) load_tile4<PAIR>(sa + part * a_part_bytes, &p.tmA, bar, m0, (int)kb, az);
            else load_tile<PAIR>(sa + part * a_part_bytes, &p.tmA, bar, k0, m0, az);
            const uint32_t sbp = sb + part * b_part_bytes;
            const int bz = b_bi + (int)(part * b_batch);
            if (!b_mn_major) {
              if (map4) load_tile4<PAIR>(sbp, tm_b, bar, n0, (int)kb, bz);
              else load_tile<PAIR>(sbp, tm_b, bar, k0, n0, bz);
            } else {
              for (uint32_t pn = 0; pn < u_panels; ++pn)
                load_tile<PAIR>(sbp + pn * panel_bytes, tm_b, bar, n0 + (int)(pn * b_panel_n), k0, bz);
            }
          }
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && leader) {
        // Drain: every armed stage still receives its bytes; wait for them (bounded) so
        // no copy is in flight into this CTA's shared memory when it exits.
        const uint32_t pending = min(issued, p.stages);
        uint32_t s = stage, ph = phase;
        for (uint32_t i = 0; i < pending; ++i) {
          if (s == 0) { s = p.stages; ph ^= 1; }
          --s;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(smem_u32(&ctrl->full[s]), ph)) {
            if (global_timer_ns() - t0 > p.limit_ns) {
              atomicCAS(p.status, 0, KSTAT_TIMEOUT_TEARDOWN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (the leader's, in a pair)
    if (leader) mma_issuer_role<KIND, PAIR>(p, ctrl, smem_base, tmem_base, worker, num_workers, krank, lane, w);
  } else {
    // ------------------------------------------------------------ epilogue warps
    using T = typename OutType<OUT>::T;
    constexpr uint32_t kGroupCols = 128 / sizeof(T);   // output columns per 128-byte staging row
    constexpr bool kInt = OUT == OUT_I32;
    const uint32_t quarter = warp & 3;                 // TMEM lanes [32*quarter, 32*quarter+32)
    const uint32_t epi_tid = (warp - 2) * 32 + lane;
    const uint32_t stage_buf = epi_base + (warp - 2) * 8192u;   // this warp's two 4 KB buffers
    const uint32_t row_in_cta = quarter * 32 + lane;
    uint32_t buf_sel = 0;
    uint32_t acc = 0, acc_phase = 0;
    uint32_t red_phase = 0;   // K-split cluster: parity of the partial-sum hand-over barriers
    bool traced_acc = false;
    const bool tr_me = quarter == 0 && lane == 0;
    bool live = true;   // after a failed wait the warp still walks the units to keep the named barrier balanced
    grid_dependency_wait();
    for (uint32_t u = worker; u < p.units_total; u += num_workers) {
      const WorkUnit wu = work_unit(p, u, krank);
      const bool is_split = wu.split != 0xFFFFFFFFu;
      const TileCoord c = tile_coord(p, wu.tile);
      const uint32_t n0 = c.n_blk * p.tile_n + wu.n_off;
      const uint32_t width = wu.width;
      if (n0 >= p.N) continue;   // a slice past the last column (skipped by every role)
      // Rows this unit may write: [m_lo, m_lim) within the tile that starts at tile_row0. A grouped row
      // tile lies on the absolute row grid and keeps only the rows of its own group.
      uint32_t tile_row0 = c.m_blk * p.tile_m + cta_rank * kTileM;
      uint32_t m_lo = 0, m_lim = p.M;
      if (p.plan) {
        const int4 e = __ldg(p.plan + c.m_blk);
        if (e.z <= e.y) continue;
        tile_row0 = (uint32_t)e.y / p.tile_m * p.tile_m + cta_rank * kTileM;
        m_lo = (uint32_t)e.y;
        m_lim = (uint32_t)e.z;
      }
      bar_sync(1, 128);                                  // everyone is done with the previous bias tile
      if (live) load_bias_tile<OUT>(p, bias_s, n0, width, epi_tid);
      bar_sync(1, 128);
      const uint32_t row0 = tile_row0 + quarter * 32;
      const uint32_t row = row0 + lane;
      const bool row_ok = row >= m_lo && row < m_lim;
      // a 32-row box store must not touch another group's rows (dense: the copy clips at M itself)
      const bool tma_rows_ok = !p.plan || (row0 >= m_lo && row0 + 32 <= m_lim);
      const size_t row_off = ((size_t)c.bi * p.M + row) * (size_t)p.N;   // (grouped: c.bi is 0)
      // A bias per output ROW (convolution as GEMM: a row is an output channel) is one value per thread.
      float rb = 0.0f;
      if constexpr (OUT != OUT_I32) {
        if (p.bias_row && p.bias && row_ok) rb = load_f32<OUT>(static_cast<const T*>(p.bias), row);
      }
      const uint32_t n_end = min(p.N, n0 + width);
      // Partial sums of a split tile, as 16-byte units: [slot][CTA][split][32-column chunk][unit 0..7]
      // [128 rows]. A thread always meets its own (row, chunk, unit) again when the parts are added,
      // so the order inside a part is free: this one makes every warp access 512 contiguous bytes.
      const uint32_t ctas = PAIR ? 2u : 1u;
      const size_t part_stride = (size_t)kTileM * p.tile_n / 4;   // 16-byte units per part
      uint4* part_base = static_cast<uint4*>(p.ws_part) +
                         ((size_t)(wu.slot * ctas + cta_rank) * p.splits) * part_stride + row_in_cta;
      auto release_acc = [&]() {   // this warp is done reading accumulator `acc`
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
          else mbar_arrive_cluster(mapa(smem_u32(&ctrl->tmem_empty[acc]), 0));
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      };
      // Finishes and stores the tile; get_chunk(tc0, r) supplies the 32 accumulators of tile
      // columns [tc0, tc0 + 32) of this thread's row.
      auto emit_tile = [&](auto get_chunk) {
        // Staged whenever possible: through TMA stores when the output's rows are 16-byte aligned, else
        // (no residual to read with vector loads) finished into the staging buffer all the same and
        // copied out by each lane, one 32-bit word or one element at a time.
        if ((p.c_tma || !p.residual) && row0 < m_lim && row0 + 32 > m_lo) {
          for (uint32_t g0 = 0; g0 < width && n0 + g0 < n_end; g0 += kGroupCols) {
            // One 128-byte group of output columns: finish it into the staging buffer, then store the
            // 32 x 128-byte box with TMA (the copy clips rows >= M and columns >= N). Two cases take
            // another last hop, each lane copying its own row out of the staging buffer instead: a
            // box that holds rows of two groups (grouped matmul), and a group cut short by the tile's
            // edge (tile widths that are not whole groups). Same arithmetic path either way.
            const uint32_t gcols = min(kGroupCols, width - g0);
            const uint32_t buf = stage_buf + buf_sel * 4096u;
            if (lane == 0) bulk_wait_group_read<1>();    // the store that last read this buffer is done
            __syncwarp();
#pragma unroll
            for (uint32_t sub = 0; sub < kGroupCols; sub += 32) {
              const uint32_t tc0 = g0 + sub;
              if (sub < gcols && n0 + tc0 < n_end) {
                uint32_t r[32];
                get_chunk(tc0, r);
                const void* res_row = nullptr;
                uint32_t res_valid = 0;
                if constexpr (!kInt) {
                  if (p.residual && row_ok) {
                    res_row = static_cast<const T*>(p.residual) + row_off + n0 + tc0;
                    res_valid = n_end - (n0 + tc0);
                  }
                }
                finish_to_stage<OUT>(p, r, bias_s, tc0, sub * sizeof(T) / 16, buf, lane, res_row,
                                     res_valid >= 32, res_valid, rb);
              }
            }
            if (p.c_tma && tma_rows_ok && gcols == kGroupCols) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&p.tmC, buf, (int)(n0 + g0), (int)row0, (int)c.bi);
                // fused all-gather: the same box goes into every other rank's buffer over NVLink
                for (uint32_t d = 0; d < p.n_peers; ++d)
                  tma_store_3d(&p.tmCp[d], buf, (int)(n0 + g0), (int)row0, (int)c.bi);
                bulk_commit_group();
              }
            } else if (row_ok && p.c_tma) {
              constexpr uint32_t kVec = 16 / sizeof(T);
              T* orow = static_cast<T*>(p.out) + row_off + n0 + g0;
#pragma unroll
              for (uint32_t ch = 0; ch < 8; ++ch)
                if (ch * kVec < gcols && n0 + g0 + ch * kVec < n_end)
                  *reinterpret_cast<uint4*>(orow + ch * kVec) = ld_shared_v4(buf + lane * 128u + ((ch ^ (lane & 7u)) << 4));
            } else if (row_ok) {
              // rows that are not 16-byte aligned: the lane copies its own staged row out, by 32-bit words
              // when the row starts on one, else element by element
              using U = std::conditional_t<sizeof(T) == 4, uint32_t, std::conditional_t<sizeof(T) == 2, uint16_t, uint8_t>>;
              constexpr uint32_t kPerWord = 4 / sizeof(T);
              U* orow = reinterpret_cast<U*>(static_cast<T*>(p.out) + row_off + n0 + g0);
              const uint32_t ncopy = min(gcols, n_end - (n0 + g0));
              const bool word_ok = (reinterpret_cast<uintptr_t>(orow) & 3u) == 0;
#pragma unroll
              for (uint32_t wd = 0; wd < 32; ++wd) {   // the 32 words of the lane's 128-byte staged row
                const uint32_t e0 = wd * kPerWord;
                if (e0 < ncopy) {
                  const uint32_t v = ld_shared_u32(buf + lane * 128u + (((wd >> 2) ^ (lane & 7u)) << 4) + (wd & 3u) * 4u);
                  if (word_ok && e0 + kPerWord <= ncopy) {
                    *reinterpret_cast<uint32_t*>(orow + e0) = v;
                  } else {
#pragma unroll
                    for (uint32_t i = 0; i < kPerWord; ++i)
                      if (e0 + i < ncopy) orow[e0 + i] = (U)(v >> (8u * (uint32_t)sizeof(T) * i));
                  }
                }
              }
            }
            buf_sel ^= 1;
            // Pacing: while the MMAs of this CTA's next tile still run there is no hurry, and a tile's
            // stores issued in one burst get in the way of the operand loads.
            if (p.pace_ns && u + num_workers < p.units_total &&
                !mbar_test_wait(smem_u32(&ctrl->tmem_full[acc ^ 1]), acc ? acc_phase ^ 1 : acc_phase))
              __nanosleep(p.pace_ns);
          }
        } else {
          for (uint32_t tc0 = 0; n0 + tc0 < n_end; tc0 += 32) {
            uint32_t r[32];
            get_chunk(tc0, r);
            if (row_ok) finish_row_chunk<OUT>(p, r, row_off, n0 + tc0, min(32u, n_end - (n0 + tc0)), rb);
          }
        }
      };
      auto store_partial = [&](uint32_t tc0, const uint32_t (&r)[32]) {
        uint4* dst = part_base + (size_t)wu.split * part_stride + (size_t)(tc0 / 32) * 8 * kTileM;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          __stcg(dst + j * kTileM, make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
      };

      bool have_sum = false;
      if constexpr (KIND == KIND_TF32) {
        if (p.chunk_kb) {
          // Exact-F32: the tensor core truncates each time it adds into its accumulator, an error
          // that grows with the number of steps. K is therefore accumulated in TMEM a few stages at
          // a time and the partial sums are added here in registers, rounded to nearest.
          have_sum = true;
          float sum[4][32];
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[q][j] = 0.0f;
          for (uint32_t kb0 = wu.kb0; live && kb0 < wu.kb1; kb0 += p.chunk_kb) {
            if (!mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, w, KSTAT_TIMEOUT_EPILOGUE)) { live = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + acc * kAccStride + ((quarter * 32u) << 16);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if ((uint32_t)q * 32 < width && n0 + q * 32 < n_end) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + q * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) sum[q][j] += __uint_as_float(r[j]);
              }
            }
            release_acc();
          }
          if (live) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t tc0 = q * 32;
              if (tc0 < width && n0 + tc0 < n_end) {
                uint32_t r[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(sum[q][j]);
                if (is_split) {
                  if (row_ok) store_partial(tc0, r);
                } else if (p.c_tma && tma_rows_ok && row0 < m_lim && row0 + 32 > m_lo) {
                  const uint32_t buf = stage_buf + buf_sel * 4096u;
                  if (lane == 0) bulk_wait_group_read<1>();
                  __syncwarp();
                  const void* res_row = nullptr;
                  uint32_t res_valid = 0;
                  if (p.residual && row_ok) {
                    res_row = static_cast<const T*>(p.residual) + row_off + n0 + tc0;
                    res_valid = n_end - (n0 + tc0);
                  }
                  finish_to_stage<OUT, true>(p, r, bias_s, tc0, 0, buf, lane, res_row, res_valid >= 32, res_valid, rb);
                  fence_proxy_async_smem();
                  __syncwarp();
                  if (lane == 0) {
                    tma_store_3d(&p.tmC, buf, (int)(n0 + tc0), (int)row0, (int)c.bi);
                    for (uint32_t d = 0; d < p.n_peers; ++d)
                      tma_store_3d(&p.tmCp[d], buf, (int)(n0 + tc0), (int)row0, (int)c.bi);
                    bulk_commit_group();
                  }
                  buf_sel ^= 1;
                } else if (row_ok) {
                  finish_row_chunk<OUT>(p, r, row_off, n0 + tc0, min(32u, n_end - (n0 + tc0)), rb);
                }
              }
            }
          }
        }
      }
      if constexpr (KIND == KIND_I8) {
        if (p.chunk_kb) {
          have_sum = true;
          if (live) {
            const uint32_t st = i8_long_k_unit<PAIR>(p, ctrl, w, tmem_base, quarter, lane, leader, wu.kb0, wu.kb1,
                                                     width, n0, n_end, row_off, row_ok, acc, acc_phase);
            acc = st & 1u;
            acc_phase = (st >> 1) & 1u;
            live = (st & 4u) != 0;
          }
        }
      }
      if (!have_sum) {
        if (live && !mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, w, KSTAT_TIMEOUT_EPILOGUE)) live = false;
        if (live) {
          tc_fence_after();
          if (!traced_acc) { traced_acc = true; if (tr_me) trace_mark(p, TR_FIRST_ACC); }
          const uint32_t taddr = tmem_base + acc * kAccStride + ((quarter * 32u) << 16);
          auto from_tmem = [&](uint32_t tc0, uint32_t (&r)[32]) {
            tmem_ld_32x32(taddr + tc0, r);
            tmem_ld_wait();
          };
          if (!PAIR && kc > 1) {
            // K-split cluster. Partial sums travel through the leader's shared memory as 16-byte units of
            // four columns, laid out [peer][TMEM quarter][32-column chunk][column / 4][row 0..31] (problems
            // of at most 32 rows: only the warp that owns TMEM lanes 0..31 has rows to send, red_q = 1;
            // up to 128 rows: all four; consecutive lanes touch consecutive units on both sides). A peer waits until the leader has read its previous
            // partial sums, writes the new ones into the leader's buffer and arrives (release, cluster
            // scope) on the leader's barrier; the leader adds the peers' sums to its own in rank order,
            // finishes the tile and hands the buffer back.
            const uint32_t chunk_bytes = 32u * 32u * 4u;
            const uint32_t chunks = (width + 31u) / 32u;
            if (krank != 0) {
              if (!mbar_wait_cluster(smem_u32(&ctrl->red_empty), red_phase ^ 1, w, KSTAT_TIMEOUT_REDUCE)) live = false;
              if (live) {
                const uint32_t dst0 = mapa(red_base, 0) + ((krank - 1) * p.red_q + quarter) * chunks * chunk_bytes + lane * 16u;
                for (uint32_t tc0 = 0; n0 + tc0 < n_end; tc0 += 32) {
                  uint32_t r[32];
                  from_tmem(tc0, r);
                  if (quarter < p.red_q) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                      st_shared_cluster_v4(dst0 + (tc0 / 32) * chunk_bytes + (uint32_t)q * 512u,
                                           make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]));
                  }
                }
                mbar_arrive_cluster(mapa(smem_u32(&ctrl->red_full), 0));
              }
            } else {
              if (!mbar_wait_cluster(smem_u32(&ctrl->red_full), red_phase, w, KSTAT_TIMEOUT_REDUCE)) live = false;
              if (live) {
                auto from_all = [&](uint32_t tc0, uint32_t (&r)[32]) {
                  from_tmem(tc0, r);
                  if (quarter < p.red_q) {
                    for (uint32_t s = 0; s + 1 < kc; ++s) {
                      const uint32_t src0 = red_base + ((s * p.red_q + quarter) * chunks + tc0 / 32) * chunk_bytes + lane * 16u;
#pragma unroll
                      for (int q = 0; q < 8; ++q) {
                        const uint4 v = ld_shared_v4(src0 + (uint32_t)q * 512u);
                        const uint32_t e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                          if constexpr (kInt) r[4 * q + i] = (uint32_t)((int32_t)r[4 * q + i] + (int32_t)e[i]);
                          else r[4 * q + i] = __float_as_uint(__uint_as_float(r[4 * q + i]) + __uint_as_float(e[i]));
                        }
                      }
                    }
                  }
                };
                emit_tile(from_all);
                for (uint32_t s = 1; s < kc; ++s) mbar_arrive_cluster(mapa(smem_u32(&ctrl->red_empty), s));
              }
            }
            red_phase ^= 1;
          } else if (!is_split) {
            emit_tile(from_tmem);
          } else {
            for (uint32_t tc0 = 0; n0 + tc0 < n_end; tc0 += 32) {
              uint32_t r[32];
              from_tmem(tc0, r);
              if (row_ok) store_partial(tc0, r);   // rows past M are never read back
            }
          }
          release_acc();
        }
      }
      if (is_split) {
        // Publish this part; whoever delivers the last part of the tile (for this CTA's rows) adds
        // all parts in split order, so the result does not depend on which unit finished last.
        __threadfence();
        bar_sync(1, 128);
        if (epi_tid == 0) {
          unsigned int* counter = p.ws_count + wu.slot * ctas + cta_rank;
          const unsigned int old = live ? atomicAdd(counter, 1u) : 0u;
          const bool last = live && old == p.splits - 1;
          if (last) *counter = 0;        // ready for the next launch
          ctrl->last_flag = last ? 1u : 0u;
        }
        bar_sync(1, 128);
        if (live && ctrl->last_flag) {
          __threadfence();
          auto from_parts = [&](uint32_t tc0, uint32_t (&r)[32]) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
            for (uint32_t sp = 0; sp < p.splits && row_ok; ++sp) {
              const uint4* src = part_base + (size_t)sp * part_stride + (size_t)(tc0 / 32) * 8 * kTileM;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint4 v = __ldcg(src + j * kTileM);
                const uint32_t e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  if constexpr (kInt) r[4 * j + q] = (uint32_t)((int32_t)r[4 * j + q] + (int32_t)e[q]);
                  else r[4 * j + q] = __float_as_uint(__uint_as_float(r[4 * j + q]) + __uint_as_float(e[q]));
                }
              }
            }
          };
          emit_tile(from_parts);
        }
      }
    }
    // The staging buffers must outlive the stores' reads of them (the writes themselves are complete
    // before the grid is, which is all anything after this kernel can observe).
    if (tr_me) trace_mark(p, TR_LAST_STORE);
    if (lane == 0) bulk_wait_group_read<0>();
    __syncwarp();
    if (tr_me) trace_mark(p, TR_STORES_READ);
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR || kc > 1) {   // no CTA may leave while another can still signal its barriers or write its shared memory
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0) trace_mark(p, TR_DONE);
  }
}

}  // namespace nb

namespace nb {

template <int KIND, int OUT>
cudaError_t gemm_inst_launch(const KParams& kp, uint32_t grid, size_t smem, cudaStream_t stream, bool pair, bool pdl) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (pair || kp.kc > 1) {   // clusters along x: a CTA pair, or the CTAs that share a tile's K range
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = pair ? 2 : kp.kc;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl) {    // the set-up may overlap the tail of the kernel before this one in the stream
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  if (pair) return cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<KIND, OUT, true>, kp);
  return cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<KIND, OUT, false>, kp);
}

template <int KIND, int OUT>
cudaError_t gemm_inst_set_smem_attr() {
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND, OUT, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND, OUT, true>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
}

template <int KIND, int OUT>
cudaError_t gemm_inst_max_clusters(int* n, const cudaLaunchConfig_t* cfg, bool pair) {
  if (pair) return cudaOccupancyMaxActiveClusters(n, gemm_tcgen05_kernel<KIND, OUT, true>, cfg);
  return cudaOccupancyMaxActiveClusters(n, gemm_tcgen05_kernel<KIND, OUT, false>, cfg);
}

}  // namespace nb
