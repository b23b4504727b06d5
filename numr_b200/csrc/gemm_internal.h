// Internal interface between the C ABI (capi.cu), the op layer (ops.cpp) and the
// kernel launchers (gemm_sm100.cu, prepass.cu). Nothing here is exported.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/numr_b200.h"

namespace nb {

// Output element kinds the epilogue can store.
enum OutKind : int { OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2, OUT_E4M3 = 3, OUT_E5M2 = 4, OUT_I32 = 5 };

constexpr uint32_t kTileM = 128;        // rows of C per CTA tile (UMMA M)
constexpr uint32_t kRowBytes = 128;     // bytes of the contiguous operand dimension per smem row
constexpr uint32_t kATileBytes = kTileM * kRowBytes;
constexpr uint32_t kSmemBudget = 227 * 1024;
constexpr uint32_t kSmemCtrlBytes = 1024;   // barriers, TMEM base, abort flag
constexpr uint32_t kEpiStageBytes = 4 * 2 * 4096;   // 4 epilogue warps x 2 staging buffers of 32 rows x 128 bytes
constexpr uint32_t kBiasTileBytes = 1024;           // bias of one tile as 256 32-bit values
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kI8ExactK = 131071;     // largest K whose I8 x I8 sums are exact in one s32 accumulator (K * 128 * 128 < 2^31)
constexpr uint32_t kAccStride = 256;        // TMEM columns between the two accumulators

// Everything one launch of the tcgen05 GEMM kernel needs, already validated.
// Operand pointers satisfy the TMA rules (16-byte aligned base and row pitch).
struct GemmLaunch {
  int kind;                 // MmaKind
  int out_kind;             // OutKind
  uint32_t elt_bytes;       // operand element size: 1, 2 or 4
  uint32_t a_fmt, b_fmt;    // instruction-descriptor operand formats
  const void* a;            // [a_batch][M][lda] (K contiguous)
  const void* b;            // layout KN: [b_batch][K][ldb] (N contiguous); NK: [b_batch][N][ldb] (K contiguous)
  uint32_t lda, ldb;        // row pitches in elements
  const void* a_lo;         // exact-F32 mode: low parts (same layout); else nullptr
  const void* b_lo;
  int b_layout;             // numr_b200_b_layout
  uint32_t batch, a_batch, b_batch, m, n, k;
  const void* bias;         // [N] of bias type (out type; int32 for I8) or nullptr
  const void* residual;     // [batch][M][N] of out type or nullptr
  void* out;                // [batch][M][N] (row pitch ldc when that is not 0)
  uint32_t ldc;             // row pitch of every output destination in elements; 0 = N (dense)
  void* peer_out[7];        // fused all-gather: the same column block inside other ranks' buffers (peer memory)
  uint32_t n_peer_out;      // how many of them (0 = none); needs 16-byte aligned rows (all stores go through TMA)
  float scale;              // multiplies the f32 accumulator
  int activation;
  int bias_per_row;         // bias holds M values, one per output row (convolution as GEMM), not N per column
  int epilogue_bwd;         // out = residual * activation'(scale*acc + bias) instead of activation(..) + residual
  cudaStream_t stream;
  int device_index;
  uint32_t force_tile_n;    // 0 = heuristic
  int f32_exact;            // F32 operands in exact (three-product) mode
  const int32_t* group_offsets;   // grouped GEMM: device array of groups + 1 row offsets; else nullptr
  uint32_t groups;
  void* group_plan;         // scratch for (ceil(M / 128) + groups) int4 plan entries (see launch_group_plan)
  void* split_ws;           // scratch for the K split of the last wave (may be null: no split)
  size_t split_ws_bytes;
};

// Launches the persistent tcgen05 GEMM. Returns a numr_b200_status.
int launch_gemm_sm100(const GemmLaunch& g);

// Scratch the kernel wants for splitting the tiles of its last wave along K (0 when it will not
// split). Only the shape fields, kind, element sizes and device of `g` are read.
size_t gemm_split_workspace_bytes(const GemmLaunch& g);

// Grouped GEMM plan: from offsets[0..groups] (int32, device) writes plan[0..plan_tiles): one entry
// {group | band size << 24, first row, rows, first tile of the band} per tile of `tile_rows` rows of every group's row range [offsets[g], offsets[g+1]) clipped to [0, total_rows),
// in group order; unused entries get rows = 0. Groups with end <= start or end > total_rows are
// skipped, as numr's CPU path does (src/ops/cpu/grouped_matmul.rs:96-103).
int launch_group_plan(const int32_t* offsets, uint32_t groups, uint32_t total_rows, void* plan,
                      uint32_t plan_tiles, uint32_t tile_rows, uint32_t band_tiles, cudaStream_t stream);

// Column sums of a row-major [rows, n] matrix of the given OutKind (F32, BF16, F16): f32 accumulation,
// one rounding, fixed order.
int launch_column_sums(int out_kind, const void* in, void* out, size_t rows, uint32_t n, cudaStream_t stream);

// Small-M path (B given as [N,K]; M = 1, exact F32 up to M = 8): HBM-bound streaming kernel on the CUDA cores.
// gemv_bt_applicable reads shapes, layout, pitches and pointer alignment; launch_gemv_bt returns a
// numr_b200_status, or -1 when the type combination is not offered (use the tensor-core path).
bool gemv_bt_applicable(const GemmLaunch& g);
int launch_gemv_bt(const GemmLaunch& g);

// Integer GEMM on the CUDA cores for the widths without a tensor-core form (numr_b200_dtype codes
// I16, I32, I64, U8, U16, U32, U64): 128-bit accumulation, bias seeds the sum, one saturating store.
int launch_matmul_int(int dtype, const void* a, const void* b, const void* bias, void* out, uint32_t batch,
                      uint32_t m, uint32_t n, uint32_t k, uint32_t a_batch, uint32_t b_batch, int b_nk,
                      cudaStream_t stream);

// out = cast(act(bias) + residual): the K == 0 form of every op (accumulator = 0).
int launch_epilogue_only(const GemmLaunch& g);

// F32 operand preparation for the tensor cores, rows x cols (pitch ld_in) ->
// rows x ld_out (ld_out >= cols, multiple of 4; the pad is zero filled):
//   hi = round-to-nearest TF32 of x; lo (optional) = TF32 of (x - hi).
int launch_split_tf32(const float* in, float* hi, float* lo, size_t rows, uint32_t cols,
                      size_t ld_in, uint32_t ld_out, cudaStream_t stream);

// The same for both (dense) operands of one GEMM in a single launch.
int launch_split_tf32_pair(const float* a_in, float* a_hi, float* a_lo, size_t a_rows, uint32_t a_cols, uint32_t a_ld,
                           const float* b_in, float* b_hi, float* b_lo, size_t b_rows, uint32_t b_cols, uint32_t b_ld,
                           cudaStream_t stream);

// Copies rows x row_bytes (pitch in_pitch bytes) into a zero-padded buffer with pitch
// out_pitch bytes (multiple of 16).
int launch_pad_rows(const void* in, void* out, size_t rows, uint32_t row_bytes, size_t in_pitch,
                    uint32_t out_pitch, cudaStream_t stream);

// Gathers an arbitrary strided view (up to 8 dims, strides in elements) into a
// contiguous buffer; elt_bytes in {1,2,4}.
int launch_gather_strided(const void* in, void* out, int ndim, const int64_t* shape,
                          const int64_t* strides, uint32_t elt_bytes, cudaStream_t stream);

// First-use work of the GEMM launcher for `device_index` (the current device): device query, the
// kernels' shared-memory attributes, the cluster occupancy query, the tensor-map encoder lookup.
// Returns a numr_b200_status; safe to call again.
int init_gemm_device(int device_index);

// Error text for the calling thread.
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);

// Device-side status word (0 = ok) of the current device.
int* device_status_ptr();
int read_and_clear_device_status(int* out);

// Switches for tests and experiments, read from the NUMR_B200_* environment variables ONCE (first
// use) and again only when numr_b200_reload_tuning() is called; none is needed in normal use.
struct Tuning {
  uint64_t wait_limit_ns = 2000000000ull;   // NUMR_B200_WAIT_LIMIT_MS: bound of every device-side wait
  int force_tile = 0;      // NUMR_B200_FORCE_TILE: tile width (0 = choose)
  int force_pair = -1;     // NUMR_B200_FORCE_PAIR: 0 single CTAs, 1 CTA pairs (-1 = choose)
  int ks = 0;              // NUMR_B200_KS: K blocks per stage, 1 / 2 / 4 (0 = choose)
  int map4 = 1;            // NUMR_B200_MAP4=0: 3-D tensor maps, one K block per stage
  int no_split = 0;        // NUMR_B200_NO_SPLIT=1: never cut K
  int force_split = 0;     // NUMR_B200_FORCE_SPLIT=n: cut K into n parts
  int tail_cut = -1;       // NUMR_B200_TAIL_CUT: 0 = never cut the last wave's tiles along N, n = into n slices (-1 = choose)
  unsigned long long trace_ptr = 0;   // NUMR_B200_TRACE_PTR: device address of 128 u64 for timeline marks (experiments)
  int epi_pace_ns = -1;    // NUMR_B200_EPI_PACE: pause after each stored column group while the next tile's MMAs still run (-1 = default)
  int f32_chunk = 0;       // NUMR_B200_F32_CHUNK: K blocks per TMEM accumulation chunk in exact-F32 mode (0 = default)
  int kcluster = 0;        // NUMR_B200_KCLUSTER: CTAs of a K-split cluster for problems of at most 32 rows: 1 = off, 2, 4 (0 = choose)
  int print_config = 0;    // NUMR_B200_PRINT_CONFIG=1: one line per GEMM launch on stderr with the configuration chosen
  int pdl = 1;             // NUMR_B200_PDL=0: plain launches (no programmatic dependent launch)
  int group_m = 0;         // NUMR_B200_GROUP_M: tile rows per rasterisation group (0 = choose)
  int no_gemv = 0;         // NUMR_B200_NO_GEMV=1: small-M problems take the tensor-core path
  int gemv_max_m = -1;     // NUMR_B200_GEMV_MAX_M: largest M the streaming kernel takes (-1 = default)
  int hold_arrival = 0;    // NUMR_B200_TEST_HOLD_ARRIVAL=1: test hook, see numr_b200_reload_tuning
};
Tuning tuning();
void reload_tuning();

}  // namespace nb
