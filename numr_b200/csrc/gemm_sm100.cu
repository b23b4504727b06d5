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
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdio>
#include <mutex>

#include "epilogue_math.cuh"
#include "gemm_internal.h"
#include "sm100_ptx.cuh"

namespace nb {

struct alignas(64) KParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  CUtensorMap tmC;          // output, boxes of 32 rows x 128 bytes (valid when c_tma != 0)
  uint32_t M, N;
  uint32_t a_batch, b_batch;
  uint32_t tiles_m, tiles_n, tiles_total, num_kb;
  uint32_t tile_n;          // UMMA N, multiple of 16, <= 256
  uint32_t stages;
  uint32_t stage_bytes;     // bytes of one stage in one CTA (A + B, both parts in split mode)
  uint32_t tx_bytes;        // bytes the stage's full barrier expects (both CTAs of a pair)
  uint32_t tile_m;          // rows of C per tile: 128, or 256 for a CTA pair
  uint32_t b_rows_cta;      // columns of the tile whose B rows this CTA loads (tile_n, or tile_n / 2 in a pair)
  uint32_t b_tile_bytes;    // bytes of one B tile
  uint32_t kb_elems;        // K elements per stage (128 / elt_bytes)
  uint32_t b_mn_major;      // 1: B tile rows are K (B given as [K,N])
  uint32_t b_panels;        // MN-major: number of 128-byte-wide column panels per tile
  uint32_t b_panel_n;       // MN-major: N elements per panel
  uint32_t b_kstep_bytes;   // descriptor advance of B per MMA step
  uint32_t b_lbo;           // leading byte offset of the B descriptor
  uint32_t b_sbo;           // stride byte offset of the B descriptor
  uint32_t b_swizzle;       // descriptor layout type of B (2: 16-byte chunks, 1: 32-byte chunks)
  uint32_t split3;          // exact-F32: three products per step from hi/lo parts
  uint32_t chunk_kb;        // stages accumulated in TMEM before the epilogue takes the partial sum (0: all of K)
  uint32_t a_box_rows;      // rows of A one load brings in (128, or fewer when M < 128)
  uint32_t bwd;             // backward form of the epilogue: out = residual * activation'(scale*acc + bias)
  const int4* plan;         // grouped GEMM: per row tile {group, first row, rows (0 = nothing here), 0}; else null
  uint32_t ks;              // K blocks (of 128 bytes) one pipeline stage holds, loaded by one copy per operand
  uint32_t map4;            // A (and a K-major B) are addressed through 4-D maps (inner, row, K block, batch)
  uint32_t a_kk_bytes;      // distance between the K blocks of A inside a stage (= bytes one K block of A takes)
  uint32_t b_kk_bytes;      // same for B
  uint32_t idesc;
  uint32_t group_m;         // rasterisation: tile rows per group
  // Work units: tiles [0, n_full) are computed whole; each remaining tile is cut along K into
  // `splits` units whose f32 / s32 partial sums meet in the workspace (the unit that arrives last
  // adds them in split order and runs the epilogue).
  uint32_t n_full, splits, kb_per_split, units_total;
  void* ws_part;            // [tail tile][CTA of the unit][split] parts of 128 x tile_n 32-bit partial sums
  unsigned int* ws_count;   // [tail tile][CTA of the unit] arrival counters, zero before the launch
  const void* bias;
  const void* residual;
  void* out;
  float scale;
  int act;
  int vec_ok;               // output rows are 16-byte aligned
  int c_tma;                // stage the output in shared memory and store it with TMA
  int* status;
  unsigned long long limit_ns;
};

struct TileCoord {
  uint32_t bi, m_blk, n_blk;
};

struct WorkUnit {
  uint32_t tile;       // output tile
  uint32_t kb0, kb1;   // stages [kb0, kb1) of K
  uint32_t split;      // index of this part of K, or 0xFFFFFFFF for a whole tile
  uint32_t slot;       // tail-tile index (valid when split != 0xFFFFFFFF)
};

__device__ __forceinline__ WorkUnit work_unit(const KParams& p, uint32_t u) {
  WorkUnit wu;
  if (u < p.n_full) {
    wu.tile = u; wu.kb0 = 0; wu.kb1 = p.num_kb; wu.split = 0xFFFFFFFFu; wu.slot = 0;
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
  c.bi = t / per_batch;
  const uint32_t r = t - c.bi * per_batch;
  const uint32_t group_span = p.group_m * p.tiles_n;
  const uint32_t g = r / group_span;
  const uint32_t first_m = g * p.group_m;
  const uint32_t gsize = min(p.group_m, p.tiles_m - first_m);
  const uint32_t in_g = r - g * group_span;
  c.m_blk = first_m + in_g % gsize;
  c.n_blk = in_g / gsize;
  return c;
}

// Control block at the end of dynamic shared memory.
struct SmemCtrl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t teardown;
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

// Finishes `ncols` (<= 32) accumulator values of one output row and stores them.
template <int OUT>
__device__ __forceinline__ void finish_row_chunk(const KParams& p, const uint32_t (&acc)[32],
                                                 size_t row_off, uint32_t col0, uint32_t ncols) {
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
    const T* bias = static_cast<const T*>(p.bias);
    const T* rrow = p.residual ? static_cast<const T*>(p.residual) + row_off + col0 : nullptr;
    constexpr int VEC = 16 / sizeof(T);   // elements per 16-byte store
    if (ncols == 32 && p.vec_ok) {
#pragma unroll
      for (int j = 0; j < 32; j += VEC) {
        alignas(16) T res[VEC];
        alignas(16) T outv[VEC];
        if (rrow) *reinterpret_cast<int4*>(res) = __ldg(reinterpret_cast<const int4*>(rrow + j));
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float x = __uint_as_float(acc[j + e]) * p.scale;
          if (bias) x += load_f32<OUT>(bias, col0 + j + e);
          if (p.bwd) {
            x = (rrow ? to_f32<OUT>(res[e]) : 0.0f) * apply_activation_derivative(x, p.act);
          } else {
            x = apply_activation(x, p.act);
            if (rrow) x += to_f32<OUT>(res[e]);
          }
          outv[e] = from_f32<OUT>(x);
        }
        *reinterpret_cast<int4*>(orow + j) = *reinterpret_cast<const int4*>(outv);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < (int)ncols) {
          float x = __uint_as_float(acc[j]) * p.scale;
          if (bias) x += load_f32<OUT>(bias, col0 + j);
          if (p.bwd) {
            x = (rrow ? to_f32<OUT>(rrow[j]) : 0.0f) * apply_activation_derivative(x, p.act);
          } else {
            x = apply_activation(x, p.act);
            if (rrow) x += to_f32<OUT>(rrow[j]);
          }
          orow[j] = from_f32<OUT>(x);
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
    umma_commit_pair(bar);
    umma_commit_pair(mapa(bar, 1));
  } else {
    umma_commit(bar);
  }
}

// Bias of the current tile as 32-bit values in shared memory: float for the float outputs
// (converted once per tile), raw int32 for the I8 path.
template <int OUT>
__device__ __forceinline__ void load_bias_tile(const KParams& p, uint32_t* bias_s, uint32_t n0,
                                               uint32_t epi_tid) {
  using T = typename OutType<OUT>::T;
#pragma unroll
  for (uint32_t i = epi_tid; i < 256; i += 128) {
    const uint32_t col = n0 + i;
    uint32_t v = 0;
    if (p.bias && i < p.tile_n && col < p.N) {
      if constexpr (OUT == OUT_I32) v = (uint32_t)__ldg(static_cast<const int32_t*>(p.bias) + col);
      else v = __float_as_uint(load_f32<OUT>(static_cast<const T*>(p.bias), col));
    }
    bias_s[i] = v;
  }
}

// Finishes 32 accumulator columns of one row (tile columns [tc0, tc0+32)) and writes them as
// 16-byte chunks into the warp's staging buffer: row `lane` at lane*128, chunk c of the row at
// position c ^ (lane & 7) (the 128-byte swizzle the output tensor map expects).
template <int OUT, int ACT>
__device__ __forceinline__ void finish_to_stage_act(const KParams& p, const uint32_t (&acc)[32],
                                                const uint32_t* bias_s, uint32_t tc0, uint32_t chunk0,
                                                uint32_t buf, uint32_t lane, const void* res_row,
                                                bool res_vec, uint32_t res_valid) {
  using T = typename OutType<OUT>::T;
  constexpr int VEC = 16 / sizeof(T);
  const T* rrow = static_cast<const T*>(res_row);
#pragma unroll
  for (int j = 0; j < 32; j += VEC) {
    alignas(16) T outv[VEC];
    alignas(16) T res[VEC];
    if constexpr (OUT != OUT_I32) {
      if (rrow) {
        if (res_vec) {
          *reinterpret_cast<int4*>(res) = __ldg(reinterpret_cast<const int4*>(rrow + j));
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) res[e] = (uint32_t)(j + e) < res_valid ? rrow[j + e] : T(0);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      if constexpr (OUT == OUT_I32) {
        long long v = (long long)(int32_t)acc[j + e] + (long long)(int32_t)bias_s[tc0 + j + e];
        v = v > 2147483647ll ? 2147483647ll : v;
        v = v < -2147483648ll ? -2147483648ll : v;
        outv[e] = (int32_t)v;
      } else {
        float x = __uint_as_float(acc[j + e]) * p.scale + __uint_as_float(bias_s[tc0 + j + e]);
        if (p.bwd) {
          x = (rrow ? to_f32<OUT>(res[e]) : 0.0f) * activation_derivative<ACT>(x);
        } else {
          x = activation<ACT>(x);
          if (rrow) x += to_f32<OUT>(res[e]);
        }
        outv[e] = from_f32<OUT>(x);
      }
    }
    const uint32_t chunk = chunk0 + (uint32_t)j / VEC;
    st_shared_v4(buf + lane * 128u + ((chunk ^ (lane & 7u)) << 4), *reinterpret_cast<const uint4*>(outv));
  }
}

template <int OUT>
__device__ __forceinline__ void finish_to_stage(const KParams& p, const uint32_t (&acc)[32],
                                                const uint32_t* bias_s, uint32_t tc0, uint32_t chunk0,
                                                uint32_t buf, uint32_t lane, const void* res_row,
                                                bool res_vec, uint32_t res_valid) {
  if constexpr (OUT == OUT_I32) {
    finish_to_stage_act<OUT, 0>(p, acc, bias_s, tc0, chunk0, buf, lane, res_row, res_vec, res_valid);
  } else {
    switch (p.act) {
      case NUMR_B200_ACT_RELU: finish_to_stage_act<OUT, NUMR_B200_ACT_RELU>(p, acc, bias_s, tc0, chunk0, buf, lane, res_row, res_vec, res_valid); break;
      case NUMR_B200_ACT_GELU: finish_to_stage_act<OUT, NUMR_B200_ACT_GELU>(p, acc, bias_s, tc0, chunk0, buf, lane, res_row, res_vec, res_valid); break;
      case NUMR_B200_ACT_SILU: finish_to_stage_act<OUT, NUMR_B200_ACT_SILU>(p, acc, bias_s, tc0, chunk0, buf, lane, res_row, res_vec, res_valid); break;
      case NUMR_B200_ACT_SIGMOID: finish_to_stage_act<OUT, NUMR_B200_ACT_SIGMOID>(p, acc, bias_s, tc0, chunk0, buf, lane, res_row, res_vec, res_valid); break;
      case NUMR_B200_ACT_TANH: finish_to_stage_act<OUT, NUMR_B200_ACT_TANH>(p, acc, bias_s, tc0, chunk0, buf, lane, res_row, res_vec, res_valid); break;
      default: finish_to_stage_act<OUT, NUMR_B200_ACT_NONE>(p, acc, bias_s, tc0, chunk0, buf, lane, res_row, res_vec, res_valid); break;
    }
  }
}

template <int KIND, int OUT, bool PAIR>
__global__ void __launch_bounds__(192, 1) gemm_tcgen05_kernel(const __grid_constant__ KParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // ring of stages | epilogue staging (4 warps x 2 x 4 KB) | bias tile | control block
  const uint32_t ring_bytes = p.stages * p.stage_bytes;
  const uint32_t epi_base = smem_base + ring_bytes;
  uint32_t* bias_s = reinterpret_cast<uint32_t*>(smem_gen + ring_bytes + kEpiStageBytes);
  SmemCtrl* ctrl = reinterpret_cast<SmemCtrl*>(smem_gen + ring_bytes + kEpiStageBytes + kBiasTileBytes);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  // In a pair, CTA rank 0 (the leader) issues the MMAs for both; each CTA loads its own operand
  // halves and finishes its own 128 rows. Work is dealt to pairs (or to single CTAs).
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const uint32_t worker = PAIR ? blockIdx.x >> 1 : blockIdx.x;
  const uint32_t num_workers = PAIR ? gridDim.x >> 1 : gridDim.x;

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
  if constexpr (PAIR) {   // the peer's barriers must exist before anything signals them
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

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
      const uint32_t a_part_bytes = ks * p.a_kk_bytes, b_part_bytes = ks * b_tile_bytes;
      const uint32_t full0 = smem_u32(&ctrl->full[0]);
      const uint32_t empty0 = smem_u32(&ctrl->empty[0]);
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;   // stages armed so far (for the teardown drain)
      bool ok = true;
      bool ready = false;    // outcome of the early test of the stage about to be refilled
      for (uint32_t u = worker; ok && u < p.units_total; u += num_workers) {
        const WorkUnit wu = work_unit(p, u);
        const TileCoord c = tile_coord(p, wu.tile);
        const int a_bi = (int)(c.bi % a_batch);
        int b_bi = (int)(c.bi % b_batch);
        int m0 = (int)(c.m_blk * p.tile_m + cta_rank * kTileM);
        if (p.plan) {   // grouped: this row tile's rows and weight come from the plan
          const int4 e = __ldg(p.plan + c.m_blk);
          if (e.z == 0) continue;
          m0 = e.y + (int)(cta_rank * kTileM);
          b_bi = e.x;
        }
        const int n0 = (int)(c.n_blk * tile_n + cta_rank * p.b_rows_cta);
        int k0 = (int)(wu.kb0 * kb_elems);
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
          if (leader) mbar_arrive_expect_tx(full0 + stage * 8u, p.tx_bytes);
          ++issued;
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + parts * a_part_bytes;
          for (uint32_t part = 0; part < parts; ++part) {
            const int az = a_bi + (int)(part * a_batch);
            if (map4) load_tile4<PAIR>(sa + part * a_part_bytes, &p.tmA, bar, m0, (int)kb, az);
            else load_tile<PAIR>(sa + part * a_part_bytes, &p.tmA, bar, k0, m0, az);
            const uint32_t sbp = sb + part * b_part_bytes;
            const int bz = b_bi + (int)(part * b_batch);
            if (!b_mn_major) {
              if (map4) load_tile4<PAIR>(sbp, &p.tmB, bar, n0, (int)kb, bz);
              else load_tile<PAIR>(sbp, &p.tmB, bar, k0, n0, bz);
            } else {
              for (uint32_t pn = 0; pn < b_panels; ++pn)
                load_tile<PAIR>(sbp + pn * panel_bytes, &p.tmB, bar, n0 + (int)(pn * b_panel_n), k0, bz);
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
    if (leader) {
      // The whole warp walks the loop in step and one elected lane issues: descriptors and
      // addresses are then warp-uniform values the compiler keeps in uniform registers, which the
      // MMA instruction reads directly. (Issuing from inside a one-lane branch costs a
      // register-to-uniform move per operand, about 110 ns per MMA.) Waits are done by lane 0 and
      // their outcome is broadcast, so the warp stays converged.
      const uint32_t idesc = p.idesc;
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
      const uint32_t b_part_units = (ks * p.b_tile_bytes) >> 4;
      const uint32_t a_kk_units = p.a_kk_bytes >> 4, b_kk_units = p.b_kk_bytes >> 4;
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
      const uint32_t chunk_kb = p.chunk_kb ? p.chunk_kb : num_kb;
      for (uint32_t u = worker; ok && u < p.units_total; u += num_workers) {
       const WorkUnit wu = work_unit(p, u);
       if (p.plan && __ldg(p.plan + tile_coord(p, wu.tile).m_blk).z == 0) continue;   // empty row tile
       // One accumulator per chunk of K: the unit's whole K range normally; in exact-F32 mode a few
       // stages, which the epilogue then adds up in registers (see the epilogue).
       for (uint32_t kb0 = wu.kb0; ok && kb0 < wu.kb1; kb0 += chunk_kb) {
        if (!wait_all(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1, KSTAT_TIMEOUT_MMA_TMEM)) {
          ok = false;
          break;
        }
        tc_fence_after();
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
        if (elect_one()) commit_to<PAIR>(smem_u32(&ctrl->tmem_full[acc]));   // accumulator complete (both CTAs' epilogues)
        __syncwarp();
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
       }
      }
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
    bool live = true;   // after a failed wait the warp still walks the units to keep the named barrier balanced
    for (uint32_t u = worker; u < p.units_total; u += num_workers) {
      const WorkUnit wu = work_unit(p, u);
      const bool is_split = wu.split != 0xFFFFFFFFu;
      const TileCoord c = tile_coord(p, wu.tile);
      const uint32_t n0 = c.n_blk * p.tile_n;
      // Rows this unit may write: [tile_row0, m_lim). A grouped row tile ends where its group ends.
      uint32_t tile_row0 = c.m_blk * p.tile_m + cta_rank * kTileM;
      uint32_t m_lim = p.M;
      bool tma_rows_ok = true;
      if (p.plan) {
        const int4 e = __ldg(p.plan + c.m_blk);
        if (e.z == 0) continue;
        tile_row0 = (uint32_t)e.y + cta_rank * kTileM;
        m_lim = (uint32_t)(e.y + e.z);
        tma_rows_ok = tile_row0 + kTileM <= m_lim;   // else a box store would run into the next group's rows
      }
      bar_sync(1, 128);                                  // everyone is done with the previous bias tile
      if (live) load_bias_tile<OUT>(p, bias_s, n0, epi_tid);
      bar_sync(1, 128);
      const uint32_t row0 = tile_row0 + quarter * 32;
      const uint32_t row = row0 + lane;
      const size_t row_off = ((size_t)c.bi * p.M + row) * (size_t)p.N;   // (grouped: c.bi is 0)
      const uint32_t n_end = min(p.N, n0 + p.tile_n);
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
        if (p.c_tma && tma_rows_ok && row0 < m_lim) {
          for (uint32_t g0 = 0; g0 < p.tile_n && n0 + g0 < n_end; g0 += kGroupCols) {
            if (g0 + kGroupCols <= p.tile_n) {
              // Whole 128-byte group inside this tile's columns: stage and store with TMA (the copy
              // clips rows >= M and columns >= N).
              const uint32_t buf = stage_buf + buf_sel * 4096u;
              if (lane == 0) bulk_wait_group_read<1>();    // the store that last read this buffer is done
              __syncwarp();
#pragma unroll
              for (uint32_t sub = 0; sub < kGroupCols; sub += 32) {
                const uint32_t tc0 = g0 + sub;
                if (n0 + tc0 < n_end) {
                  uint32_t r[32];
                  get_chunk(tc0, r);
                  const void* res_row = nullptr;
                  uint32_t res_valid = 0;
                  if constexpr (!kInt) {
                    if (p.residual && row < m_lim) {
                      res_row = static_cast<const T*>(p.residual) + row_off + n0 + tc0;
                      res_valid = n_end - (n0 + tc0);
                    }
                  }
                  finish_to_stage<OUT>(p, r, bias_s, tc0, sub * sizeof(T) / 16, buf, lane, res_row,
                                       res_valid >= 32, res_valid);
                }
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&p.tmC, buf, (int)(n0 + g0), (int)row0, (int)c.bi);
                bulk_commit_group();
              }
              buf_sel ^= 1;
            } else {
              // Group that would cross into the next tile's columns: direct stores.
              for (uint32_t tc0 = g0; tc0 < p.tile_n && n0 + tc0 < n_end; tc0 += 32) {
                uint32_t r[32];
                get_chunk(tc0, r);
                if (row < m_lim) finish_row_chunk<OUT>(p, r, row_off, n0 + tc0, min(32u, n_end - (n0 + tc0)));
              }
            }
          }
        } else {
          for (uint32_t tc0 = 0; n0 + tc0 < n_end; tc0 += 32) {
            uint32_t r[32];
            get_chunk(tc0, r);
            if (row < m_lim) finish_row_chunk<OUT>(p, r, row_off, n0 + tc0, min(32u, n_end - (n0 + tc0)));
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
              if ((uint32_t)q * 32 < p.tile_n && n0 + q * 32 < n_end) {
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
              if (tc0 < p.tile_n && n0 + tc0 < n_end) {
                uint32_t r[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(sum[q][j]);
                if (is_split) {
                  if (row < m_lim) store_partial(tc0, r);
                } else if (p.c_tma && tma_rows_ok && row0 < m_lim) {
                  const uint32_t buf = stage_buf + buf_sel * 4096u;
                  if (lane == 0) bulk_wait_group_read<1>();
                  __syncwarp();
                  const void* res_row = nullptr;
                  uint32_t res_valid = 0;
                  if (p.residual && row < m_lim) {
                    res_row = static_cast<const T*>(p.residual) + row_off + n0 + tc0;
                    res_valid = n_end - (n0 + tc0);
                  }
                  finish_to_stage<OUT>(p, r, bias_s, tc0, 0, buf, lane, res_row, res_valid >= 32, res_valid);
                  fence_proxy_async_smem();
                  __syncwarp();
                  if (lane == 0) {
                    tma_store_3d(&p.tmC, buf, (int)(n0 + tc0), (int)row0, (int)c.bi);
                    bulk_commit_group();
                  }
                  buf_sel ^= 1;
                } else if (row < m_lim) {
                  finish_row_chunk<OUT>(p, r, row_off, n0 + tc0, min(32u, n_end - (n0 + tc0)));
                }
              }
            }
          }
        }
      }
      if (!have_sum) {
        if (live && !mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, w, KSTAT_TIMEOUT_EPILOGUE)) live = false;
        if (live) {
          tc_fence_after();
          const uint32_t taddr = tmem_base + acc * kAccStride + ((quarter * 32u) << 16);
          auto from_tmem = [&](uint32_t tc0, uint32_t (&r)[32]) {
            tmem_ld_32x32(taddr + tc0, r);
            tmem_ld_wait();
          };
          if (!is_split) {
            emit_tile(from_tmem);
          } else {
            for (uint32_t tc0 = 0; n0 + tc0 < n_end; tc0 += 32) {
              uint32_t r[32];
              from_tmem(tc0, r);
              if (row < m_lim) store_partial(tc0, r);   // rows past M are never read back
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
            for (uint32_t sp = 0; sp < p.splits && row < m_lim; ++sp) {
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
    // The staging buffers must outlive the stores that read them.
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {   // neither CTA may leave while the other can still signal its barriers
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault,
                                         &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 4-D map (inner = one 128-byte K block, rows, K blocks, batch) over a K-major operand whose rows
// are whole K blocks; the box takes `ks` K blocks of `box_rows` rows.
bool encode_map4(CUtensorMap* tm, CUtensorMapDataType dt, uint32_t elt, const void* base, uint64_t k,
                 uint64_t rows, uint64_t batches, uint64_t pitch_bytes, uint32_t box_rows, uint32_t ks) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const uint64_t kb_elems = kRowBytes / elt;
  cuuint64_t dims[4] = {kb_elems, rows, k / kb_elems, batches};
  cuuint64_t strides[3] = {pitch_bytes, kRowBytes, pitch_bytes * rows};
  cuuint32_t box[4] = {(cuuint32_t)kb_elems, box_rows, ks, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 3-D map (inner, rows, batch) with a 128-byte-wide box of `box_rows` rows.
bool encode_map(CUtensorMap* tm, CUtensorMapDataType dt, uint32_t elt, const void* base,
                uint64_t inner, uint64_t rows, uint64_t batches, uint64_t pitch_bytes,
                uint32_t box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {inner, rows, batches};
  cuuint64_t strides[2] = {pitch_bytes, pitch_bytes * rows};
  cuuint32_t box[3] = {kRowBytes / elt, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

struct DeviceInfo {
  bool ready = false;
  bool ok = false;
  int sm_count = 0;
  int cc_major = 0;
};
DeviceInfo g_dev[64];
std::mutex g_dev_mutex;

template <int KIND, int OUT>
cudaError_t set_smem_attr() {
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND, OUT, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND, OUT, true>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
}

// Queries the device once and opts every kernel instantiation into the large
// dynamic shared-memory carve-out.
const DeviceInfo* device_info(int device_index) {
  if (device_index < 0 || device_index >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceInfo& d = g_dev[device_index];
  if (d.ready) return &d;
  d.ready = true;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_index) != cudaSuccess) {
    cudaGetLastError();
    return &d;
  }
  d.sm_count = prop.multiProcessorCount;
  d.cc_major = prop.major;
  if (prop.major != 10) return &d;
  cudaError_t e = cudaSuccess;
  auto acc = [&](cudaError_t x) { if (e == cudaSuccess) e = x; };
  acc(set_smem_attr<KIND_F16, OUT_BF16>());
  acc(set_smem_attr<KIND_F16, OUT_F16>());
  acc(set_smem_attr<KIND_TF32, OUT_F32>());
  acc(set_smem_attr<KIND_F8F6F4, OUT_F32>());
  acc(set_smem_attr<KIND_F8F6F4, OUT_BF16>());
  acc(set_smem_attr<KIND_F8F6F4, OUT_F16>());
  acc(set_smem_attr<KIND_F8F6F4, OUT_E4M3>());
  acc(set_smem_attr<KIND_F8F6F4, OUT_E5M2>());
  acc(set_smem_attr<KIND_I8, OUT_I32>());
  if (e != cudaSuccess) {
    cudaGetLastError();
    return &d;
  }
  d.ok = true;
  return &d;
}

// Launches `grid` CTAs; in pair mode as clusters of two CTAs along x.
template <int KIND, int OUT>
cudaError_t do_launch(const KParams& kp, uint32_t grid, size_t smem, cudaStream_t stream, bool pair) {
  if (!pair) {
    gemm_tcgen05_kernel<KIND, OUT, false><<<grid, 192, smem, stream>>>(kp);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<KIND, OUT, true>, kp);
}

// How many CTA pairs of the largest configuration the device runs at once (cached per device).
int max_active_pairs(int device_index, int sm_count) {
  static int cached[64] = {0};
  if (cached[device_index]) return cached[device_index];
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * (sm_count / 2), 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = kSmemBudget;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_kernel<KIND_F16, OUT_BF16, true>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  if (n > sm_count / 2) n = sm_count / 2;
  cached[device_index] = n > 0 ? n : -1;
  return cached[device_index];
}

}  // namespace

uint64_t wait_limit_ns() {
  static uint64_t v = [] {
    const char* s = getenv("NUMR_B200_WAIT_LIMIT_MS");
    long ms = s ? atol(s) : 2000;
    if (ms < 1) ms = 1;
    if (ms > 60000) ms = 60000;
    return (uint64_t)ms * 1000000ull;
  }();
  return v;
}

namespace {

// Shape-dependent choices of one launch: work-unit form, tile width, pipeline depth, K split.
// Depends only on the problem (not on pointers), so the workspace query can run it too.
struct Config {
  bool pair_mode = false;
  int pairs = 0;
  size_t split_ws_bytes = 0;     // workspace the K split needs (counters, then partial sums)
  size_t split_count_bytes = 0;  // of which arrival counters
};

int configure(const GemmLaunch& g, const DeviceInfo* dev, KParams& kp, Config& cfg) {
  memset(&kp, 0, sizeof(kp));
  const uint32_t elt = g.elt_bytes;
  kp.kb_elems = kRowBytes / elt;
  kp.split3 = (g.a_lo != nullptr) ? 1u : 0u;
  kp.b_mn_major = (g.b_layout == NUMR_B200_B_KN) ? 1u : 0u;
  kp.b_panel_n = kRowBytes / elt;

  // Tile width.
  // Widths are whole 128-byte groups of the output type (what one staged TMA store covers) and,
  // for an MN-major B, whole 128-byte panels of the operand type.
  static const uint32_t out_elt[6] = {4, 2, 2, 1, 1, 4};
  const uint32_t out_group = kRowBytes / out_elt[g.out_kind];
  const uint32_t hard_step = kp.b_mn_major ? kp.b_panel_n : 16u;      // what the MMA and the loads need
  const uint32_t step = std::max<uint32_t>(hard_step, out_group);     // what the heuristic offers
  // Two shapes of work unit: one CTA per 128 x tile_n tile, or a CTA pair per 256 x tile_n tile
  // (each CTA then loads only half of B, 2/3 of the bytes per flop at tile_n = 256). Pick the pair
  // form when its modelled time (waves x rows of 128 bytes loaded per stage) is lower.
  const uint32_t max_n_single = kp.split3 ? 128u : 256u;
  const uint32_t max_n_pair = kp.split3 ? 128u : 256u;   // exact-F32 keeps its sums in 128 registers per thread
  const uint32_t hard_step_pair = kp.b_mn_major ? 2 * kp.b_panel_n : 16u;
  const uint32_t step_pair = std::max<uint32_t>(hard_step_pair, out_group);
  const int pairs = max_active_pairs(g.device_index, dev->sm_count);
  uint32_t tile_n = g.force_tile_n;
  int mode = -1;   // -1 choose, 0 single, 1 pair
  if (const char* env = getenv("NUMR_B200_FORCE_TILE")) { if (tile_n == 0) tile_n = (uint32_t)atoi(env); }
  if (const char* env = getenv("NUMR_B200_FORCE_PAIR")) mode = atoi(env) ? 1 : 0;
  if (pairs <= 0 || g.m <= kTileM) mode = 0;   // a pair's second CTA would own rows that do not exist
  // Time model in microseconds, fitted to measurements on B200 with one K block per stage: a K
  // block (128 bytes of K) costs a CTA at least about 0.36 us in the loops' own instructions and
  // more with the rows it loads (0.41 us at 256 rows, 0.55 us at the 384 rows of a single CTA's
  // 128 x 256 tile, which is bound by shared-memory traffic); a tile costs about 1.5 us of switch
  // and epilogue tail. Several K blocks per stage lower the constant, not the ranking of the shapes.
  // A problem that fills less than half a wave may also be cut along K (see below), at about 25 us
  // for the counter memset and the reduction.
  const uint32_t num_kb_all = (g.k + kp.kb_elems - 1) / kp.kb_elems;
  const char* no_split_env = getenv("NUMR_B200_NO_SPLIT");
  const bool may_split = !(no_split_env && atoi(no_split_env)) && !g.group_offsets;
  auto split_parts = [&](uint64_t tiles, uint64_t workers, uint32_t* kbs_out) {
    uint32_t parts = 1, kbs = num_kb_all;
    if (may_split && tiles * 2 <= workers) {
      parts = (uint32_t)std::min<uint64_t>(8, workers / tiles);
      kbs = (num_kb_all + parts - 1) / parts;
      kbs = std::max<uint32_t>(8u, (kbs + 3) / 4 * 4);
      parts = (num_kb_all + kbs - 1) / kbs;
      // The reduction is a chain of L2 round trips (measured 20 - 30 us), so the cut has to save
      // clearly more than that: long K only.
      if (parts < 2 || 0.36 * (kp.split3 ? 3.0 : 1.0) * (num_kb_all - kbs) < 40.0) { parts = 1; kbs = num_kb_all; }
    }
    if (const char* env = getenv("NUMR_B200_FORCE_SPLIT")) {     // experiments: cut K into this many parts
      const uint32_t want = g.group_offsets ? 0u : (uint32_t)atoi(env);
      if (want >= 2 && num_kb_all >= 2 * want) {
        kbs = (num_kb_all + want - 1) / want;
        kbs = (kbs + 3) / 4 * 4;
        parts = (num_kb_all + kbs - 1) / kbs;
      }
    }
    if (kbs_out) *kbs_out = kbs;
    return parts;
  };
  auto model = [&](bool pm, uint32_t tn) {
    const uint64_t tm = pm ? 256 : 128;
    const uint64_t tiles = ((g.m + tm - 1) / tm + (g.group_offsets ? g.groups : 0u)) * ((g.n + tn - 1) / tn) * g.batch;
    const uint64_t workers = pm ? (uint64_t)pairs : (uint64_t)dev->sm_count;
    const uint64_t waves = (tiles + workers - 1) / workers;
    const double rows = 128.0 + (pm ? tn / 2 : tn) + 24.0;
    const double t_kb = std::max(0.36, 0.41 * rows / 280.0) * (kp.split3 ? 3.0 : 1.0);
    uint32_t kbs = num_kb_all;
    const uint32_t parts = split_parts(tiles, workers, &kbs);
    return (double)waves * (kbs * t_kb + 1.5) + (parts > 1 ? 25.0 : 0.0);
  };
  bool pair_mode = false;
  if (tile_n == 0) {
    double best = 1e300;
    for (int pm = 0; pm < 2; ++pm) {
      if (mode >= 0 && pm != mode) continue;
      const uint32_t st = pm ? step_pair : step;
      const uint32_t mx = pm ? max_n_pair : max_n_single;
      for (uint32_t tn = mx / st * st; tn >= st; tn -= st) {
        const double c = model(pm != 0, tn);
        if (c < best * 0.999) { best = c; tile_n = tn; pair_mode = pm != 0; }
        if (tn == st) break;
      }
    }
  } else {
    pair_mode = mode == 1;
  }
  const uint32_t hs = pair_mode ? hard_step_pair : hard_step;
  const uint32_t mx = pair_mode ? max_n_pair : max_n_single;
  if (tile_n < hs || tile_n > mx || tile_n % hs != 0)
    return fail(NUMR_B200_EINVAL, "tile width %u is not a multiple of %u in [%u, %u]", tile_n, hs, hs, mx);
  kp.tile_n = tile_n;
  kp.tile_m = pair_mode ? 256u : 128u;
  kp.b_rows_cta = pair_mode ? tile_n / 2 : tile_n;
  kp.b_panels = kp.b_mn_major ? kp.b_rows_cta / kp.b_panel_n : 1u;
  kp.b_tile_bytes = kp.b_rows_cta * kRowBytes;
  // K blocks per stage. One copy per operand brings in `ks` consecutive K blocks (a 4-D box over
  // inner, row, K block, batch): issuing a copy costs the producer thread about 60 ns and arming the
  // barrier about 100 ns whatever the box holds, which at one K block per stage (0.25 us for the
  // pair of copies) was slower than the tensor core needs for the block. The 4-D view needs rows
  // that are whole K blocks (no partial block whose tail would alias the next row).
  // Fewer than 128 rows in all: the A box, and the room a K block of A takes in a stage, cover only
  // the rows that exist (in whole 8-row swizzle groups). The MMA still reads 128 rows from there:
  // what lies beyond the box (the next K block, B, the staging area behind the ring) is unrelated
  // data that feeds output rows >= M only, and those are never stored (an output row depends on
  // its own row of A alone).
  kp.a_box_rows = (!pair_mode && g.m < kTileM) ? (g.m + 7u) / 8u * 8u : kTileM;
  kp.a_kk_bytes = kp.a_box_rows * kRowBytes;
  const uint32_t parts_n = kp.split3 ? 2u : 1u;
  const uint32_t kb_bytes = (kp.a_kk_bytes + kp.b_tile_bytes) * parts_n;
  const uint32_t ring_budget = kSmemBudget - kSmemCtrlBytes - kEpiStageBytes - kBiasTileBytes - 1024u;
  kp.map4 = (g.k % kp.kb_elems == 0) ? 1u : 0u;
  if (const char* env = getenv("NUMR_B200_MAP4")) { if (!atoi(env)) kp.map4 = 0; }
  kp.ks = 1;
  if (kp.map4) {
    const uint32_t max_ks = kp.b_mn_major ? std::min(4u, 256u / kp.kb_elems) : 4u;   // box rows <= 256
    for (uint32_t c = max_ks; c >= 2; c >>= 1)
      if (ring_budget / (kb_bytes * c) >= 3 && num_kb_all >= c) { kp.ks = c; break; }
    if (const char* env = getenv("NUMR_B200_KS")) {
      const uint32_t c = (uint32_t)atoi(env);
      if ((c == 1 || c == 2 || c == 4) && c <= max_ks && ring_budget / (kb_bytes * c) >= 2) kp.ks = c;
    }
  }
  kp.stage_bytes = kb_bytes * kp.ks;
  kp.tx_bytes = (kp.a_box_rows * kRowBytes + kp.b_tile_bytes) * kp.ks * parts_n * (pair_mode ? 2u : 1u);
  kp.chunk_kb = kp.split3 ? 4u : 0u;   // exact-F32: partial sums of 4 stages (128 values of K)
  kp.stages = std::min<uint32_t>(8u, ring_budget / kp.stage_bytes);
  if (kp.stages < 2) return fail(NUMR_B200_EINVAL, "internal: fewer than 2 pipeline stages fit");
  kp.b_sbo = 1024;
  kp.b_swizzle = 2;
  if (!kp.b_mn_major) {
    kp.b_kstep_bytes = 32;
    kp.b_lbo = 16;
    kp.b_kk_bytes = kp.b_tile_bytes;
  } else {
    kp.b_kstep_bytes = (kp.kb_elems / 4) * kRowBytes;
    kp.b_lbo = kp.ks * kp.kb_elems * kRowBytes;   // a panel holds the stage's K rows, all K blocks
    kp.b_kk_bytes = kp.kb_elems * kRowBytes;
    if (g.kind == KIND_TF32) {
      // MN-major 32-bit operands exist only in the 32-byte-chunk swizzle: 4-row groups.
      kp.b_sbo = 512;
      kp.b_swizzle = 1;
    }
  }

  kp.M = g.m;
  kp.N = g.n;
  kp.a_batch = g.a_batch;
  kp.b_batch = g.b_batch;
  kp.tiles_m = (g.m + kp.tile_m - 1) / kp.tile_m + (g.group_offsets ? g.groups : 0u);   // grouped: an upper bound
  kp.tiles_n = (g.n + tile_n - 1) / tile_n;
  const uint64_t total = (uint64_t)kp.tiles_m * kp.tiles_n * g.batch;
  if (total > 0x7FFFFFFFull) return fail(NUMR_B200_EINVAL, "too many output tiles (%llu)", (unsigned long long)total);
  kp.tiles_total = (uint32_t)total;
  kp.num_kb = (g.k + kp.kb_elems - 1) / kp.kb_elems;
  kp.group_m = 8;

  // K split of a partly filled wave: with `rem` tiles for `workers` workers each tile is cut into
  // up to workers / rem parts (at least 8 stages each, a multiple of the exact-F32 chunk), so the
  // wave costs 1 / parts of a tile time plus a reduction.
  const uint32_t workers = pair_mode ? (uint32_t)pairs : (uint32_t)dev->sm_count;
  kp.n_full = kp.tiles_total;
  kp.splits = 1;
  kp.kb_per_split = kp.num_kb;
  kp.units_total = kp.tiles_total;
  {
    uint32_t kbs = kp.num_kb;
    const uint32_t parts = split_parts(kp.tiles_total, workers, &kbs);
    if (parts >= 2) {
      const uint32_t ctas = pair_mode ? 2u : 1u;
      const uint32_t rem = kp.tiles_total;
      cfg.split_count_bytes = ((size_t)rem * ctas * sizeof(unsigned int) + 255) / 256 * 256;
      cfg.split_ws_bytes = cfg.split_count_bytes + (size_t)rem * ctas * parts * kTileM * tile_n * 4;
      kp.n_full = 0;
      kp.splits = parts;
      kp.kb_per_split = kbs;
      kp.units_total = rem * parts;
    }
  }
  cfg.pair_mode = pair_mode;
  cfg.pairs = pairs;
  return NUMR_B200_OK;
}

}  // namespace

size_t gemm_split_workspace_bytes(const GemmLaunch& g) {
  const DeviceInfo* dev = device_info(g.device_index);
  if (!dev || !dev->ok || g.k == 0 || g.m == 0 || g.n == 0 || g.batch == 0) return 0;
  KParams kp;
  Config cfg;
  if (configure(g, dev, kp, cfg) != NUMR_B200_OK) return 0;
  return cfg.split_ws_bytes;
}

int launch_gemm_sm100(const GemmLaunch& g) {
  const DeviceInfo* dev = device_info(g.device_index);
  if (!dev || !dev->ok)
    return fail(NUMR_B200_ECUDA,
                "device %d is not a usable sm_100 GPU (compute capability major %d); there is no fallback path",
                g.device_index, dev ? dev->cc_major : -1);
  if (g.k == 0 || g.m == 0 || g.n == 0 || g.batch == 0)
    return fail(NUMR_B200_EINVAL, "launch_gemm_sm100: empty problem reached the kernel launcher");

  KParams kp;
  Config cfg;
  int cst = configure(g, dev, kp, cfg);
  if (cst != NUMR_B200_OK) return cst;
  const bool pair_mode = cfg.pair_mode;
  const int pairs = cfg.pairs;
  const uint32_t elt = g.elt_bytes;
  const uint32_t tile_n = kp.tile_n;
  if (kp.splits > 1) {
    if (!g.split_ws || g.split_ws_bytes < cfg.split_ws_bytes) {
      // No room for the partial sums: run the tail tiles whole.
      kp.n_full = kp.tiles_total;
      kp.splits = 1;
      kp.kb_per_split = kp.num_kb;
      kp.units_total = kp.tiles_total;
    } else {
      kp.ws_count = static_cast<unsigned int*>(g.split_ws);
      kp.ws_part = static_cast<char*>(g.split_ws) + cfg.split_count_bytes;
      cudaError_t me = cudaMemsetAsync(kp.ws_count, 0, cfg.split_count_bytes, g.stream);
      if (me != cudaSuccess)
        return fail(NUMR_B200_ECUDA, "clearing the split counters failed: %s", cudaGetErrorString(me));
    }
  }

  // Instruction descriptor: D format, A/B formats, B major, N >> 3, M >> 4.
  const uint32_t c_fmt = (g.kind == KIND_I8) ? 2u : 1u;
  kp.idesc = (c_fmt << 4) | (g.a_fmt << 7) | (g.b_fmt << 10) | (0u << 15) | (kp.b_mn_major << 16) |
             ((tile_n >> 3) << 17) | ((kp.tile_m >> 4) << 24);

  CUtensorMapDataType dt;
  switch (g.kind) {
    case KIND_F16: dt = (g.a_fmt == 1) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case KIND_TF32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
  }
  const uint32_t parts = kp.split3 ? 2u : 1u;
  if (kp.split3) {
    // The low parts must directly follow the high parts so one map covers both.
    const char* a_exp = static_cast<const char*>(g.a) + (size_t)g.a_batch * g.m * g.lda * elt;
    const size_t b_rows = kp.b_mn_major ? g.k : g.n;
    const char* b_exp = static_cast<const char*>(g.b) + (size_t)g.b_batch * b_rows * g.ldb * elt;
    if (g.a_lo != a_exp || g.b_lo != b_exp)
      return fail(NUMR_B200_EINVAL, "internal: hi/lo operand parts are not adjacent");
  }
  const bool a_ok = kp.map4 ? encode_map4(&kp.tmA, dt, elt, g.a, g.k, g.m, (uint64_t)g.a_batch * parts,
                                         (uint64_t)g.lda * elt, kp.a_box_rows, kp.ks)
                            : encode_map(&kp.tmA, dt, elt, g.a, g.k, g.m, (uint64_t)g.a_batch * parts,
                                         (uint64_t)g.lda * elt, kp.a_box_rows);
  if (!a_ok)
    return fail(NUMR_B200_ECUDA, "cuTensorMapEncodeTiled failed for A (ptr %p, K %u, M %u, pitch %llu B)",
                g.a, g.k, g.m, (unsigned long long)g.lda * elt);
  bool okb;
  if (!kp.b_mn_major)
    okb = kp.map4 ? encode_map4(&kp.tmB, dt, elt, g.b, g.k, g.n, (uint64_t)g.b_batch * parts,
                                (uint64_t)g.ldb * elt, kp.b_rows_cta, kp.ks)
                  : encode_map(&kp.tmB, dt, elt, g.b, g.k, g.n, (uint64_t)g.b_batch * parts,
                               (uint64_t)g.ldb * elt, kp.b_rows_cta);
  else
    okb = encode_map(&kp.tmB, dt, elt, g.b, g.n, g.k, (uint64_t)g.b_batch * parts,
                     (uint64_t)g.ldb * elt, kp.ks * kp.kb_elems,
                     kp.b_swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
  if (!okb)
    return fail(NUMR_B200_ECUDA, "cuTensorMapEncodeTiled failed for B (ptr %p, pitch %llu B)", g.b,
                (unsigned long long)g.ldb * elt);

  if (g.group_offsets) {
    int pst = launch_group_plan(g.group_offsets, g.groups, g.m, g.group_plan, kp.tiles_m, kp.tile_m, g.stream);
    if (pst != NUMR_B200_OK) return pst;
    kp.plan = static_cast<const int4*>(g.group_plan);
  }
  kp.bias = g.bias;
  kp.residual = g.residual;
  kp.out = g.out;
  kp.scale = g.scale;
  kp.act = g.activation;
  kp.bwd = g.epilogue_bwd ? 1u : 0u;
  static const uint32_t out_bytes[6] = {4, 2, 2, 1, 1, 4};
  const uint32_t ob = out_bytes[g.out_kind];
  kp.vec_ok = ((reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && ((size_t)g.n * ob) % 16 == 0 &&
               (!g.residual || (reinterpret_cast<uintptr_t>(g.residual) & 15) == 0))
                  ? 1
                  : 0;
  // Output through TMA when its rows are 16-byte aligned: boxes of 32 rows x 128 bytes.
  kp.c_tma = 0;
  if (kp.vec_ok) {
    CUtensorMapDataType cdt;
    switch (g.out_kind) {
      case OUT_F32: cdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
      case OUT_BF16: cdt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
      case OUT_F16: cdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
      case OUT_I32: cdt = CU_TENSOR_MAP_DATA_TYPE_INT32; break;
      default: cdt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    }
    if (!encode_map(&kp.tmC, cdt, ob, g.out, g.n, g.m, g.batch, (uint64_t)g.n * ob, 32))
      return fail(NUMR_B200_ECUDA, "cuTensorMapEncodeTiled failed for the output (ptr %p, N %u)", g.out, g.n);
    kp.c_tma = 1;
  }
  kp.status = device_status_ptr();
  if (!kp.status) return fail(NUMR_B200_ECUDA, "cannot resolve the device status word");
  kp.limit_ns = wait_limit_ns();

  const uint32_t grid = pair_mode ? 2u * std::min<uint32_t>(kp.units_total, (uint32_t)pairs)
                                  : std::min<uint32_t>(kp.units_total, (uint32_t)dev->sm_count);
  const size_t smem = (size_t)kp.stages * kp.stage_bytes + kEpiStageBytes + kBiasTileBytes + kSmemCtrlBytes + 1024;
  cudaError_t e = cudaErrorInvalidValue;
  const int key = g.kind * 16 + g.out_kind;
  switch (key) {
    case KIND_F16 * 16 + OUT_BF16: e = do_launch<KIND_F16, OUT_BF16>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_F16 * 16 + OUT_F16: e = do_launch<KIND_F16, OUT_F16>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_TF32 * 16 + OUT_F32: e = do_launch<KIND_TF32, OUT_F32>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_F8F6F4 * 16 + OUT_F32: e = do_launch<KIND_F8F6F4, OUT_F32>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_F8F6F4 * 16 + OUT_BF16: e = do_launch<KIND_F8F6F4, OUT_BF16>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_F8F6F4 * 16 + OUT_F16: e = do_launch<KIND_F8F6F4, OUT_F16>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_F8F6F4 * 16 + OUT_E4M3: e = do_launch<KIND_F8F6F4, OUT_E4M3>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_F8F6F4 * 16 + OUT_E5M2: e = do_launch<KIND_F8F6F4, OUT_E5M2>(kp, grid, smem, g.stream, pair_mode); break;
    case KIND_I8 * 16 + OUT_I32: e = do_launch<KIND_I8, OUT_I32>(kp, grid, smem, g.stream, pair_mode); break;
    default:
      return fail(NUMR_B200_EUNSUPPORTED, "no kernel for MMA kind %d with output kind %d", g.kind,
                  g.out_kind);
  }
  if (e != cudaSuccess)
    return fail(NUMR_B200_ECUDA, "GEMM kernel launch failed: %s", cudaGetErrorString(e));
  return NUMR_B200_OK;
}

}  // namespace nb
