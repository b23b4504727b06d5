// Kernel parameter block of the tcgen05 GEMM and the per-instantiation entry points that the
// host-side launcher calls. Every (MMA kind, output kind) pair is compiled in a translation unit
// of its own (gemm_inst.cu with NB_INST_KIND / NB_INST_OUT), so the instantiations build in parallel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_internal.h"

namespace nb {

struct alignas(64) KParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  CUtensorMap tmC;          // output, boxes of 32 rows x 128 bytes (valid when c_tma != 0)
  CUtensorMap tmB2;         // K-major B with the box of a column slice (valid when cut > 1 and B is K-major)
  // Fused all-gather: the output column block as it lies inside each OTHER rank's [M, N_total] buffer
  // (peer memory, written with plain tiled stores; no load ever touches them). tmC is then the
  // block inside this rank's own buffer.
  CUtensorMap tmCp[7];
  uint32_t n_peers;
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
  // Or (never both) the tiles past n_full are cut along N into `cut` slices of cut_n columns, each a
  // unit that walks all of K: b_rows_cta2 / tx_bytes2 / idesc2 are b_rows_cta / tx_bytes / idesc of a slice.
  uint32_t cut, cut_n, b_rows_cta2, tx_bytes2, idesc2;
  // Or (single-CTA tiles, at most 32 rows) every tile is shared by a cluster of `kc` CTAs, CTA r of the
  // cluster taking K blocks [r * kc_kbs, (r + 1) * kc_kbs); their partial sums meet in `red_bytes` of the
  // leader's shared memory (distributed shared memory, no workspace). kc = 1: off.
  uint32_t kc, kc_kbs, red_bytes;
  void* ws_part;            // [tail tile][CTA of the unit][split] parts of 128 x tile_n 32-bit partial sums
  unsigned int* ws_count;   // [tail tile][CTA of the unit] arrival counters, zero before the launch
  const void* bias;
  const void* residual;
  void* out;
  float scale;
  int act;
  int vec_ok;               // output rows are 16-byte aligned
  int c_tma;                // stage the output in shared memory and store it with TMA
  uint32_t bias_row;        // the bias has one value per output ROW (M of them) instead of per column
  uint32_t red_q;           // K-split cluster: epilogue warps (TMEM lane quarters) that have rows to hand over: 1 (M <= 32) or 4
  uint32_t pace_ns;         // epilogue: pause after each stored column group while the next tile is still being computed
  uint32_t test_hold;       // test hook: the MMA issuer never signals "accumulator complete"
  int* status;
  unsigned long long* trace;   // experiments: timeline marks of the first 8 CTAs (null = off)
  unsigned long long limit_ns;
};

// Launches `grid` CTAs of gemm_tcgen05_kernel<KIND, OUT, pair>; in pair mode as clusters of two CTAs
// along x; with `pdl` as a programmatic dependent launch (see grid_dependency_wait in sm100_ptx.cuh).
template <int KIND, int OUT>
cudaError_t gemm_inst_launch(const KParams& kp, uint32_t grid, size_t smem, cudaStream_t stream, bool pair,
                             bool pdl);
// (A single-CTA launch with kp.kc > 1 goes out as clusters of kp.kc CTAs.)
// Opts both forms of the instantiation into the large dynamic shared-memory carve-out (current device).
template <int KIND, int OUT>
cudaError_t gemm_inst_set_smem_attr();
// cudaOccupancyMaxActiveClusters of the pair form for the launch configuration `cfg`.
template <int KIND, int OUT>
cudaError_t gemm_inst_max_clusters(int* n, const cudaLaunchConfig_t* cfg, bool pair);

}  // namespace nb
