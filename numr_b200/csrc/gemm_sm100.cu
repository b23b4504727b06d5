// Host side of the tcgen05 GEMM: shape-dependent configuration (work-unit form, tile width,
// pipeline depth, K split), tensor-map encoding and the launch. The kernel itself is in
// gemm_kernel.cuh and is instantiated per (MMA kind, output kind) by gemm_inst.cu.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "gemm_internal.h"
#include "gemm_params.h"

namespace nb {

// MMA kinds (the values of MmaKind in sm100_ptx.cuh, which is device-only).
enum : int { KIND_F16 = 0, KIND_TF32 = 1, KIND_F8F6F4 = 2, KIND_I8 = 3 };

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


// Queries the device once and opts every kernel instantiation into the large
// dynamic shared-memory carve-out.
const DeviceInfo* device_info(int device_index) {
  if (device_index < 0 || device_index >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceInfo& d = g_dev[device_index];
  if (d.ready) return &d;
  // (`ready` is set only once the answer is final: a transient failure is retried by the next call.)
  int sm = 0, major = 0;
  if (cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, device_index) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_index) != cudaSuccess) {
    cudaGetLastError();
    return &d;
  }
  d.sm_count = sm;
  d.cc_major = major;
  if (major != 10) {
    d.ready = true;   // not an sm_100 device: final
    return &d;
  }
  cudaError_t e = cudaSuccess;
  auto acc = [&](cudaError_t x) { if (e == cudaSuccess) e = x; };
  acc(gemm_inst_set_smem_attr<KIND_F16, OUT_BF16>());
  acc(gemm_inst_set_smem_attr<KIND_F16, OUT_F16>());
  acc(gemm_inst_set_smem_attr<KIND_TF32, OUT_F32>());
  acc(gemm_inst_set_smem_attr<KIND_F8F6F4, OUT_F32>());
  acc(gemm_inst_set_smem_attr<KIND_F8F6F4, OUT_BF16>());
  acc(gemm_inst_set_smem_attr<KIND_F8F6F4, OUT_F16>());
  acc(gemm_inst_set_smem_attr<KIND_F8F6F4, OUT_E4M3>());
  acc(gemm_inst_set_smem_attr<KIND_F8F6F4, OUT_E5M2>());
  acc(gemm_inst_set_smem_attr<KIND_I8, OUT_I32>());
  if (e != cudaSuccess) {
    cudaGetLastError();
    return &d;
  }
  d.ok = true;
  d.ready = true;
  return &d;
}

// How many clusters of the largest configuration the device runs at once (cached per device):
// slot 0 = CTA pairs (the pair kernel), slot 1 / 2 = clusters of 2 / 4 single-CTA kernels.
int max_active_clusters(int device_index, int sm_count, int slot) {
  static int cached[64][3] = {{0}};
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (cached[device_index][slot]) return cached[device_index][slot];
  const int cs = slot == 2 ? 4 : 2;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(cs * (sm_count / cs), 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = kSmemBudget;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = cs;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (gemm_inst_max_clusters<KIND_F16, OUT_BF16>(&n, &cfg, slot == 0) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  if (n > sm_count / cs) n = sm_count / cs;
  cached[device_index][slot] = n > 0 ? n : -1;
  return cached[device_index][slot];
}

int max_active_pairs(int device_index, int sm_count) { return max_active_clusters(device_index, sm_count, 0); }

}  // namespace

namespace {
std::mutex g_tuning_mutex;
Tuning g_tuning;
bool g_tuning_loaded = false;

int env_int(const char* name, int fallback) {
  const char* s = getenv(name);
  return (s && *s) ? atoi(s) : fallback;
}

void load_tuning_locked() {
  Tuning t;
  long ms = env_int("NUMR_B200_WAIT_LIMIT_MS", 2000);
  if (ms < 1) ms = 1;
  if (ms > 60000) ms = 60000;
  t.wait_limit_ns = (uint64_t)ms * 1000000ull;
  t.force_tile = env_int("NUMR_B200_FORCE_TILE", 0);
  t.force_pair = env_int("NUMR_B200_FORCE_PAIR", -1);
  if (t.force_pair > 1) t.force_pair = 1;
  t.ks = env_int("NUMR_B200_KS", 0);
  t.map4 = env_int("NUMR_B200_MAP4", 1) ? 1 : 0;
  t.no_split = env_int("NUMR_B200_NO_SPLIT", 0) ? 1 : 0;
  t.force_split = env_int("NUMR_B200_FORCE_SPLIT", 0);
  t.tail_cut = env_int("NUMR_B200_TAIL_CUT", -1);
  t.group_m = env_int("NUMR_B200_GROUP_M", 0);
  t.pdl = env_int("NUMR_B200_PDL", 1) ? 1 : 0;
  t.kcluster = env_int("NUMR_B200_KCLUSTER", 0);
  t.f32_chunk = env_int("NUMR_B200_F32_CHUNK", 0);
  t.epi_pace_ns = env_int("NUMR_B200_EPI_PACE", -1);
  t.print_config = env_int("NUMR_B200_PRINT_CONFIG", 0);
  if (const char* tp = getenv("NUMR_B200_TRACE_PTR")) t.trace_ptr = strtoull(tp, nullptr, 0);
  t.no_gemv = env_int("NUMR_B200_NO_GEMV", 0) ? 1 : 0;
  t.gemv_max_m = env_int("NUMR_B200_GEMV_MAX_M", -1);
  t.hold_arrival = env_int("NUMR_B200_TEST_HOLD_ARRIVAL", 0) ? 1 : 0;
  g_tuning = t;
  g_tuning_loaded = true;
}
}  // namespace

Tuning tuning() {
  std::lock_guard<std::mutex> lock(g_tuning_mutex);
  if (!g_tuning_loaded) load_tuning_locked();
  return g_tuning;
}

void reload_tuning() {
  std::lock_guard<std::mutex> lock(g_tuning_mutex);
  load_tuning_locked();
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

uint32_t out_group_of(int out_kind) {
  static const uint32_t out_elt[6] = {4, 2, 2, 1, 1, 4};
  return kRowBytes / out_elt[out_kind];
}

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
  // what the MMA and the loads need (exact-F32 adds its chunk sums 32 columns at a time)
  const uint32_t hard_step = kp.b_mn_major ? kp.b_panel_n : (kp.split3 ? 32u : 16u);
  // The heuristic also offers half groups (where that is still a multiple of the 32 columns an
  // epilogue step handles): the group that straddles the tile's edge is then stored with plain
  // vector stores instead of a staged copy. Problems of at most 128 rows keep whole groups, the
  // widths their time model was fitted on.
  const bool whole_groups = g.m <= kTileM || g.ldc || g.n_peer_out;   // (a strided / gathered output has no plain-store path)
  const uint32_t soft_step = whole_groups ? out_group : std::max<uint32_t>(32u, out_group / 2);
  const uint32_t step = std::max<uint32_t>(hard_step, soft_step);
  // Two shapes of work unit: one CTA per 128 x tile_n tile, or a CTA pair per 256 x tile_n tile
  // (each CTA then loads only half of B, 2/3 of the bytes per flop at tile_n = 256). Pick the pair
  // form when its modelled time (waves x rows of 128 bytes loaded per stage) is lower.
  // exact-F32 keeps its sums in 128 registers per thread; so does I8 beyond the exact range of the
  // s32 accumulator (64-bit sums)
  const bool i8_long = g.kind == KIND_I8 && g.k > kI8ExactK;
  const uint32_t max_n_single = (kp.split3 || i8_long) ? 128u : 256u;
  const uint32_t max_n_pair = (kp.split3 || i8_long) ? 128u : 256u;
  const uint32_t hard_step_pair = kp.b_mn_major ? 2 * kp.b_panel_n : (kp.split3 ? 32u : 16u);
  const uint32_t step_pair = std::max<uint32_t>(hard_step_pair, soft_step);
  const int pairs = max_active_pairs(g.device_index, dev->sm_count);
  uint32_t tile_n = g.force_tile_n;
  int mode = -1;   // -1 choose, 0 single, 1 pair
  const Tuning tune = tuning();
  if (tile_n == 0 && tune.force_tile > 0) tile_n = (uint32_t)tune.force_tile;
  if (tune.force_pair >= 0) mode = tune.force_pair;
  if (pairs <= 0 || g.m <= kTileM) mode = 0;   // a pair's second CTA would own rows that do not exist
  // A problem that fills less than half a wave may be cut along K (see below), at about 25 us for
  // the counter memset and the reduction.
  const uint32_t num_kb_all = (g.k + kp.kb_elems - 1) / kp.kb_elems;
  const bool may_split = !tune.no_split && !g.group_offsets && !i8_long;   // (32-bit partial sums)
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
    if (tune.force_split > 0) {     // experiments: cut K into this many parts
      const uint32_t want = g.group_offsets ? 0u : (uint32_t)tune.force_split;
      if (want >= 2 && num_kb_all >= 2 * want) {
        kbs = (num_kb_all + want - 1) / want;
        kbs = (kbs + 3) / 4 * 4;
        parts = (num_kb_all + kbs - 1) / kbs;
      }
    }
    if (kbs_out) *kbs_out = kbs;
    return parts;
  };
  // Slices a tile of the last, partly filled wave can be cut into along N (1 = leave it whole). A
  // slice keeps whole 128-byte groups of the output (one staged store), the MMA's N step and, for an
  // MN-major B, whole 128-byte panels per CTA; the slices of all `rem` tiles must fit in one wave.
  auto tail_cut = [&](bool pm, uint32_t tn, uint64_t rem, uint64_t workers) -> uint32_t {
    if (rem == 0 || g.group_offsets || tune.tail_cut == 0 || tune.tail_cut == 1) return 1u;
    const uint32_t unit = std::max<uint32_t>(out_group, pm ? hard_step_pair : hard_step);
    uint32_t best = 1;
    for (uint32_t c = 2; c <= 8; c *= 2) {
      if (tn % c != 0 || (tn / c) % unit != 0) break;
      if (tune.tail_cut > 1 ? c > (uint32_t)tune.tail_cut : rem * c > workers) break;
      best = c;
    }
    return best;
  };
  // Time model in microseconds, fitted to measurements on B200 (BF16, K = 4096, many waves): a K
  // block costs 0.10 us of loop overhead plus a share that grows with the tile width (the MMA time and
  // the shared-memory traffic both do): 0.29 us at 256 columns for a CTA pair's 256-row tile, 0.42 us
  // for a single CTA's 128-row tile; a tile costs about 1.5 us of switch and epilogue tail. Problems of
  // at most 128 rows (a trimmed A box, see below) keep the older rows-loaded form they were tuned with.
  auto kb_time = [&](bool pm, uint32_t tn) {
    double t;
    if (g.m <= kTileM) {
      const double rows = 128.0 + tn + 24.0;
      t = std::max(0.36, 0.41 * rows / 280.0);
    } else {
      t = 0.10 + (pm ? 0.29 : 0.42) * tn / 256.0;
    }
    return t * (kp.split3 ? 3.0 : 1.0);
  };
  // Problems of at most 128 rows (decode shapes, small batches) stream the weight once and do little arithmetic: what
  // counts is how many CTAs pull from HBM at once and how many bytes each keeps in flight, not the tensor
  // pipe. For a tile width, `decode_choice` picks how many CTAs share a tile's K range as a cluster (1, 2
  // or 4: the partial sums meet in the leader's shared memory, whose buffer comes out of the ring) and
  // estimates the launch: the slowest of HBM (6.2 TB/s), one CTA's stream (its ring in flight over 2.2 us,
  // at most 60 GB/s: what a CTA was seen to pull when 64 - 128 of them stream) and its chain of MMA issues
  // (55 / 68 / 130 cycles each at 64 / 128 / 256 columns), plus 6 us of fixed cost, 1 us for the hand-over
  // and the epilogue, which one warp per 32 rows runs (a quarter of TMEM each): 0.8 us per 32
  // columns and 0.2 us more per peer whose sums it adds. (Without it the tile search, which knows nothing
  // of clusters, took 256-column tiles for 16 x 4096 x 14336: 16 tiles, clusters of 4 = 64 CTAs with a ring
  // of two stages, 60 us where 128 CTAs on 64-column tiles take 26.)
  // (33 - 128 rows: only where K is at least twice N, the few-tile, long-K shapes whose workspace K split was
  // 2 - 3x slower than the vendor library (64 x 4096 x 14336: 51 -> 29 us); with more tiles than that the
  // general search below, tuned on such shapes, stays 5 - 25 % ahead of this model)
  const bool decode_like = (g.m <= 32 || (g.m <= kTileM && (uint64_t)g.k >= 2ull * g.n) || tune.kcluster > 1) && g.m <= kTileM &&
                           !kp.split3 && !i8_long && !g.group_offsets && tune.kcluster != 1 && mode != 1;
  const uint32_t red_rows = g.m <= 32 ? 32u : 128u;   // rows of partial sums a peer hands over: one TMEM quarter, or all four
  auto decode_choice = [&](uint32_t tn, uint32_t* kc_out) {
    const uint64_t tiles = (uint64_t)((g.n + tn - 1) / tn) * g.batch;
    const double a_rows = (double)((g.m + 7u) / 8u * 8u);
    const double kb_bytes = (a_rows + tn) * (double)kRowBytes;
    const double ring0 = (double)(kSmemBudget - kSmemCtrlBytes - kEpiStageBytes - kBiasTileBytes - 1024u);
    const double t_hbm = (double)g.n * g.k * elt * g.b_batch / 6.2e12 * 1e6;
    const double cyc = tn <= 64 ? 55.0 : tn <= 128 ? 68.0 : 130.0;
    double best = 1e300;
    uint32_t best_kc = 1;
    for (uint32_t c = 1; c <= 4; c <<= 1) {
      if (tune.kcluster > 1 && (uint32_t)tune.kcluster != c) continue;
      if (c > 1) {
        const int room = max_active_clusters(g.device_index, dev->sm_count, c == 4 ? 2 : 1);
        if (room <= 0 || num_kb_all < 2 * c) continue;
        if (tune.kcluster <= 1 && (tiles > (uint64_t)room || num_kb_all / c < 8)) continue;
      }
      const double red = c > 1 ? (double)(c - 1) * red_rows * ((tn + 31u) / 32u * 32u) * 4.0 : 0.0;
      const double ring = ring0 - red;
      if (ring < 2.0 * kb_bytes) continue;
      const double bw = std::min(60e9, ring / 2.2e-6);
      const double waves = c > 1 ? 1.0 : (double)((tiles + dev->sm_count - 1) / dev->sm_count);
      const double kb_cta = (double)num_kb_all / c * waves;
      const double t_stream = kb_cta * kb_bytes / bw * 1e6;
      const double t_issue = kb_cta * 4.0 * cyc / 1.8e3;
      const double t_epi = (double)((tn + 31u) / 32u) * (0.8 + 0.2 * (c - 1));
      const double t = std::max(t_stream, std::max(t_hbm, t_issue)) + 6.0 + (c > 1 ? 1.0 : 0.0) + t_epi * waves +
                       3.0 * (waves - 1.0);   // (a further wave restarts the pipeline: about 3 us)
      if (t < best) { best = t; best_kc = c; }
    }
    *kc_out = best_kc;
    return best;
  };
  auto model = [&](bool pm, uint32_t tn) {
    if (decode_like) {
      uint32_t c = 1;
      return pm ? 1e300 : decode_choice(tn, &c);
    }
    const uint64_t tm = pm ? 256 : 128;
    const uint64_t tiles = ((g.m + tm - 1) / tm + (g.group_offsets ? g.groups : 0u)) * ((g.n + tn - 1) / tn) * g.batch;
    const uint64_t workers = pm ? (uint64_t)pairs : (uint64_t)dev->sm_count;
    uint32_t kbs = num_kb_all;
    const uint32_t parts = split_parts(tiles, workers, &kbs);
    if (parts > 1) return kbs * kb_time(pm, tn) + 1.5 + 25.0;
    const uint64_t full = tiles / workers, rem = tiles % workers;
    double t = (double)full * (num_kb_all * kb_time(pm, tn) + 1.5);
    if (rem) {
      const uint32_t c = full ? tail_cut(pm, tn, rem, workers) : 1u;
      t += num_kb_all * kb_time(pm, tn / c) + 1.5;
    }
    return t;
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
  // K-split cluster for problems of at most 32 rows (decode shapes): what bounds them is not HBM but
  // one CTA's chain of MMA issues along K while most SMs have no tile at all. 2 or 4 CTAs (a
  // cluster) share a tile, each walking its own part of K, and the partial sums meet in the leader's
  // shared memory: no workspace, fixed order. Taken when every tile still gets a cluster in one wave
  // and a CTA keeps at least 8 K blocks.
  kp.kc = 1;
  kp.red_bytes = 0;
  if (!pair_mode && decode_like) {
    if (decode_choice(tile_n, &kp.kc) >= 1e300) kp.kc = 1;
    if (kp.kc > 1) kp.red_bytes = (kp.kc - 1) * red_rows * ((tile_n + 31u) / 32u * 32u) * 4u;
  }
  kp.red_q = red_rows / 32u;
  const uint32_t ring_budget = kSmemBudget - kSmemCtrlBytes - kEpiStageBytes - kBiasTileBytes - 1024u - kp.red_bytes;
  kp.map4 = (g.k % kp.kb_elems == 0) ? 1u : 0u;
  if (!tune.map4) kp.map4 = 0;
  kp.ks = 1;
  if (kp.map4) {
    const uint32_t max_ks = kp.b_mn_major ? std::min(4u, 256u / kp.kb_elems) : 4u;   // box rows <= 256
    // (exact-F32 stages hold two parts per operand: two K blocks per stage with a ring of two measured
    // 8 - 14 % faster than one K block per stage with a ring of four, from 1024^3 to 4096^3)
    const uint32_t min_ring = kp.split3 ? 2u : 3u;
    for (uint32_t c = max_ks; c >= 2; c >>= 1)
      if (ring_budget / (kb_bytes * c) >= min_ring && num_kb_all >= c) { kp.ks = c; break; }
    if (tune.ks > 0) {
      const uint32_t c = (uint32_t)tune.ks;
      if ((c == 1 || c == 2 || c == 4) && c <= max_ks && ring_budget / (kb_bytes * c) >= 2) kp.ks = c;
    }
  }
  kp.stage_bytes = kb_bytes * kp.ks;
  kp.tx_bytes = (kp.a_box_rows * kRowBytes + kp.b_tile_bytes) * kp.ks * parts_n * (pair_mode ? 2u : 1u);
  kp.chunk_kb = kp.split3 ? 4u : 0u;   // exact-F32: partial sums of 4 stages (128 values of K)
  if (kp.split3 && tune.f32_chunk > 0) kp.chunk_kb = (uint32_t)tune.f32_chunk;   // (experiments: a multiple of ks)
  if (i8_long) kp.chunk_kb = 512u;     // I8 with long K: 512 K blocks = 65536 values per s32 accumulator
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
  // Rasterisation: tiles are dealt in groups of `group_m` tile rows, column by column, so the rows of
  // A a group needs (group_m x tile_m x K) stay in L2 while B streams past once per group. About
  // 32 MB of A per group measured best on B200 (126 MB L2): 16 tile rows at K = 4096 BF16 (2 % over 8
  // on 16384 x 14336 x 4096, 1 % on 4096^3). A B that fits L2 outright (under 24 MB) is never
  // re-read, and then the smaller group's smaller working set of A wins (groups of 4 against 8: 1 - 2 % at
  // N = 1792, 2 % on I8 4096^3 and on 8192 x 2048 x 8192; against 16: 3 - 4 %).
  {
    const uint64_t row_tile_bytes = (uint64_t)kp.tile_m * g.k * elt * (kp.split3 ? 2u : 1u);
    uint64_t gm = row_tile_bytes ? (32ull << 20) / row_tile_bytes : 16;
    gm = std::min<uint64_t>(16, std::max<uint64_t>(4, gm));
    if ((uint64_t)g.n * g.k * elt * (kp.split3 ? 2u : 1u) <= (24ull << 20)) gm = std::min<uint64_t>(gm, 4);
    kp.group_m = tune.group_m > 0 ? (uint32_t)tune.group_m : (uint32_t)gm;
  }

  // K split of a partly filled wave: with `rem` tiles for `workers` workers each tile is cut into
  // up to workers / rem parts (at least 8 stages each, a multiple of the exact-F32 chunk), so the
  // wave costs 1 / parts of a tile time plus a reduction.
  const uint32_t workers = pair_mode ? (uint32_t)pairs : (uint32_t)dev->sm_count;
  kp.n_full = kp.tiles_total;
  kp.splits = 1;
  kp.kb_per_split = kp.num_kb;
  kp.units_total = kp.tiles_total;
  kp.kc_kbs = kp.num_kb;
  if (kp.kc > 1) {
    // K blocks per CTA of the cluster: whole stages, and every CTA gets at least one block
    uint32_t kbs = (kp.num_kb + kp.kc - 1) / kp.kc;
    kbs = (kbs + kp.ks - 1) / kp.ks * kp.ks;
    while (kp.kc > 1 && (uint64_t)(kp.kc - 1) * kbs >= kp.num_kb) kp.kc >>= 1;
    if (kp.kc > 1) kp.kc_kbs = kbs;
    else kp.red_bytes = 0;   // (the ring was sized with the buffer in mind: it only has room to spare)
  }
  if (kp.kc == 1) {
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
  // Cut of the last wave along N (never together with the K split).
  kp.cut = 1;
  kp.cut_n = tile_n;
  kp.b_rows_cta2 = kp.b_rows_cta;
  kp.tx_bytes2 = kp.tx_bytes;
  if (kp.kc == 1 && kp.splits == 1 && kp.tiles_total > workers) {
    const uint32_t rem = kp.tiles_total % workers;
    const uint32_t c = tail_cut(pair_mode, tile_n, rem, workers);
    if (c > 1) {
      kp.cut = c;
      kp.cut_n = tile_n / c;
      kp.n_full = kp.tiles_total - rem;
      kp.units_total = kp.n_full + rem * c;
      kp.b_rows_cta2 = pair_mode ? kp.cut_n / 2 : kp.cut_n;
      kp.tx_bytes2 = (kp.a_box_rows * kRowBytes + kp.b_rows_cta2 * kRowBytes) * kp.ks * parts_n * (pair_mode ? 2u : 1u);
    }
  }
  cfg.pair_mode = pair_mode;
  cfg.pairs = pairs;
  return NUMR_B200_OK;
}

}  // namespace

int init_gemm_device(int device_index) {
  const DeviceInfo* dev = device_info(device_index);
  if (!dev || !dev->ok)
    return fail(NUMR_B200_ECUDA,
                "device %d is not a usable sm_100 GPU (compute capability major %d); there is no fallback path",
                device_index, dev ? dev->cc_major : -1);
  for (int slot = 0; slot < 3; ++slot) (void)max_active_clusters(device_index, dev->sm_count, slot);
  if (!get_encode_fn()) return fail(NUMR_B200_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
  return NUMR_B200_OK;
}

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

  kp.idesc2 = (kp.idesc & ~(0x3Fu << 17)) | ((kp.cut_n >> 3) << 17);

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
  if (okb && kp.cut > 1 && !kp.b_mn_major)   // a K-major B needs the narrower box of a column slice
    okb = kp.map4 ? encode_map4(&kp.tmB2, dt, elt, g.b, g.k, g.n, (uint64_t)g.b_batch * parts,
                                (uint64_t)g.ldb * elt, kp.b_rows_cta2, kp.ks)
                  : encode_map(&kp.tmB2, dt, elt, g.b, g.k, g.n, (uint64_t)g.b_batch * parts,
                               (uint64_t)g.ldb * elt, kp.b_rows_cta2);
  if (!okb)
    return fail(NUMR_B200_ECUDA, "cuTensorMapEncodeTiled failed for B (ptr %p, pitch %llu B)", g.b,
                (unsigned long long)g.ldb * elt);

  if (g.group_offsets) {
    // bands of row tiles inside one group: about 16 MB of A per band, next to the group's weight in L2
    const uint64_t tile_bytes = (uint64_t)kp.tile_m * g.k * elt * (kp.split3 ? 2u : 1u);
    const int forced_band = tuning().group_m;
    const uint32_t band = forced_band > 0 ? (uint32_t)forced_band
                                           : (uint32_t)std::min<uint64_t>(16, std::max<uint64_t>(2, (16ull << 20) / std::max<uint64_t>(tile_bytes, 1)));
    int pst = launch_group_plan(g.group_offsets, g.groups, g.m, g.group_plan, kp.tiles_m, kp.tile_m, band, g.stream);
    if (pst != NUMR_B200_OK) return pst;
    kp.plan = static_cast<const int4*>(g.group_plan);
  }
  kp.bias = g.bias;
  kp.residual = g.residual;
  kp.out = g.out;
  kp.scale = g.scale;
  kp.act = g.activation;
  kp.bwd = g.epilogue_bwd ? 1u : 0u;
  kp.bias_row = g.bias_per_row ? 1u : 0u;
  static const uint32_t out_bytes[6] = {4, 2, 2, 1, 1, 4};
  const uint32_t ob = out_bytes[g.out_kind];
  kp.vec_ok = ((reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && ((size_t)g.n * ob) % 16 == 0 &&
               ((size_t)(g.ldc ? g.ldc : g.n) * ob) % 16 == 0 &&
               (!g.residual || (reinterpret_cast<uintptr_t>(g.residual) & 15) == 0))
                  ? 1
                  : 0;
  // Output through TMA when its rows are 16-byte aligned: boxes of 32 rows x 128 bytes.
  const uint64_t c_pitch = (uint64_t)(g.ldc ? g.ldc : g.n) * ob;
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
    if (!encode_map(&kp.tmC, cdt, ob, g.out, g.n, g.m, g.batch, c_pitch, 32))
      return fail(NUMR_B200_ECUDA, "cuTensorMapEncodeTiled failed for the output (ptr %p, N %u)", g.out, g.n);
    for (uint32_t i = 0; i < g.n_peer_out; ++i)
      if (!encode_map(&kp.tmCp[i], cdt, ob, g.peer_out[i], g.n, g.m, g.batch, c_pitch, 32))
        return fail(NUMR_B200_ECUDA, "cuTensorMapEncodeTiled failed for the output in peer buffer %u (ptr %p)", i, g.peer_out[i]);
    kp.c_tma = 1;
  }
  kp.n_peers = g.n_peer_out;
  if (g.ldc || g.n_peer_out) {
    // A strided or replicated output is written by the staged TMA stores only (the plain-store paths
    // assume a dense [M, N] output): needs 16-byte aligned rows and tile widths of whole store groups.
    if (g.n_peer_out > 7) return fail(NUMR_B200_EINVAL, "at most 7 peer destinations");
    if (!kp.c_tma || (c_pitch % 16) != 0 || g.group_offsets || kp.tile_n % out_group_of(g.out_kind) != 0)
      return fail(NUMR_B200_EINVAL, "strided / gathered output needs 16-byte aligned rows (N %u, pitch %llu B)", g.n,
                  (unsigned long long)c_pitch);
    for (uint32_t i = 0; i < g.n_peer_out; ++i)
      if (!g.peer_out[i] || (reinterpret_cast<uintptr_t>(g.peer_out[i]) & 15))
        return fail(NUMR_B200_EINVAL, "peer destination %u is NULL or not 16-byte aligned", i);
  }
  kp.status = device_status_ptr();
  if (!kp.status) return fail(NUMR_B200_ECUDA, "cannot resolve the device status word");
  kp.limit_ns = tuning().wait_limit_ns;
  kp.test_hold = tuning().hold_arrival ? 1u : 0u;
  kp.pace_ns = tuning().epi_pace_ns >= 0 ? (uint32_t)tuning().epi_pace_ns : 0u;
  kp.trace = reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(tuning().trace_ptr));

  uint32_t grid = pair_mode ? 2u * std::min<uint32_t>(kp.units_total, (uint32_t)pairs)
                            : std::min<uint32_t>(kp.units_total, (uint32_t)dev->sm_count);
  if (kp.kc > 1) {
    const int room = max_active_clusters(g.device_index, dev->sm_count, kp.kc == 4 ? 2 : 1);
    grid = kp.kc * std::min<uint32_t>(kp.units_total, (uint32_t)std::max(room, 1));
  }
  const size_t smem = (size_t)kp.stages * kp.stage_bytes + kp.red_bytes + kEpiStageBytes + kBiasTileBytes +
                      kSmemCtrlBytes + 1024;
  if (tuning().print_config)
    fprintf(stderr,
            "numr_b200 gemm: %u x %u x %u (batch %u) kind %d out %d | %s tile %u x %u, %u K blocks (%u per stage, %u stages), "
            "tiles %u units %u, K-cluster %u, K-split %u (%u blocks each), N-cut %u, raster group %u, grid %u, smem %zu\n",
            g.m, g.n, g.k, g.batch, g.kind, g.out_kind, pair_mode ? "pair" : "single", kp.tile_m, kp.tile_n, kp.num_kb, kp.ks,
            kp.stages, kp.tiles_total, kp.units_total, kp.kc, kp.splits, kp.kb_per_split, kp.cut, kp.group_m, grid, smem);
  cudaError_t e = cudaErrorInvalidValue;
  const bool pdl = tuning().pdl != 0;
  const int key = g.kind * 16 + g.out_kind;
  switch (key) {
    case KIND_F16 * 16 + OUT_BF16: e = gemm_inst_launch<KIND_F16, OUT_BF16>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_F16 * 16 + OUT_F16: e = gemm_inst_launch<KIND_F16, OUT_F16>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_TF32 * 16 + OUT_F32: e = gemm_inst_launch<KIND_TF32, OUT_F32>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_F8F6F4 * 16 + OUT_F32: e = gemm_inst_launch<KIND_F8F6F4, OUT_F32>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_F8F6F4 * 16 + OUT_BF16: e = gemm_inst_launch<KIND_F8F6F4, OUT_BF16>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_F8F6F4 * 16 + OUT_F16: e = gemm_inst_launch<KIND_F8F6F4, OUT_F16>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_F8F6F4 * 16 + OUT_E4M3: e = gemm_inst_launch<KIND_F8F6F4, OUT_E4M3>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_F8F6F4 * 16 + OUT_E5M2: e = gemm_inst_launch<KIND_F8F6F4, OUT_E5M2>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    case KIND_I8 * 16 + OUT_I32: e = gemm_inst_launch<KIND_I8, OUT_I32>(kp, grid, smem, g.stream, pair_mode, pdl); break;
    default:
      return fail(NUMR_B200_EUNSUPPORTED, "no kernel for MMA kind %d with output kind %d", g.kind,
                  g.out_kind);
  }
  if (e != cudaSuccess)
    return fail(NUMR_B200_ECUDA, "GEMM kernel launch failed: %s", cudaGetErrorString(e));
  return NUMR_B200_OK;
}

}  // namespace nb
