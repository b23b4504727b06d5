/*
 * numr_b200 — C ABI of the B200 (sm_100a) dense-GEMM path for numr.
 *
 * The library replaces the bodies of numr's CUDA matmul launchers
 * (src/runtime/cuda/kernels/loader/*.rs, kernels/gemm_epilogue/launcher.rs,
 * kernels/fp8_matmul.rs) with hand-written tcgen05/TMEM/TMA kernels. Every entry
 * point follows the launchers' contract:
 *   - pointers are raw device addresses of contiguous row-major buffers that the
 *     caller owns (inputs, output and workspace); the library never allocates,
 *     frees or synchronises, and launches only on the stream it is given;
 *   - all per-launch parameters travel by value (safe under CUDA-graph capture);
 *   - every argument is validated on the host and a status is returned before
 *     anything is launched; the text of the last failure on the calling thread is
 *     available from numr_b200_last_error().
 * There is no CPU fallback: on a machine without an sm_100 GPU every compute
 * entry point returns NUMR_B200_ECUDA.
 */
#ifndef NUMR_B200_H
#define NUMR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. 1,2,3,6,7 map onto numr's Error variants (src/error.rs:12-168):
 * InvalidArgument, UnsupportedDType, Internal, ShapeMismatch, DTypeMismatch. */
typedef enum {
  NUMR_B200_OK = 0,
  NUMR_B200_EINVAL = 1,
  NUMR_B200_EUNSUPPORTED = 2,
  NUMR_B200_ECUDA = 3,
  NUMR_B200_EWORKSPACE = 4, /* workspace missing, too small or misaligned */
  NUMR_B200_ETIMEOUT = 5,   /* a bounded device-side wait ran out (see numr_b200_device_status) */
  NUMR_B200_ESHAPE = 6,
  NUMR_B200_EDTYPE = 7
} numr_b200_status;

/* Element types on this path (numr DType, src/dtype/mod.rs). */
typedef enum {
  NUMR_B200_F32 = 0,
  NUMR_B200_BF16 = 1,
  NUMR_B200_F16 = 2,
  NUMR_B200_FP8E4M3 = 3,
  NUMR_B200_FP8E5M2 = 4,
  NUMR_B200_I8 = 5,
  NUMR_B200_I32 = 6,
  /* integer widths without a tensor-core form: exact 128-bit accumulation on the CUDA cores,
   * one saturating store, output of the operands' type (matmul_int.cu:1-104) */
  NUMR_B200_I64 = 7,
  NUMR_B200_I16 = 8,
  NUMR_B200_U8 = 9,
  NUMR_B200_U16 = 10,
  NUMR_B200_U32 = 11,
  NUMR_B200_U64 = 12
} numr_b200_dtype;

/* GemmActivation::code() (src/ops/traits/gemm_epilogue.rs:34-43). */
typedef enum {
  NUMR_B200_ACT_NONE = 0,
  NUMR_B200_ACT_RELU = 1,
  NUMR_B200_ACT_GELU = 2, /* tanh form, 0.7978845608 / 0.044715 */
  NUMR_B200_ACT_SILU = 3,
  NUMR_B200_ACT_SIGMOID = 4,
  NUMR_B200_ACT_TANH = 5,
  /* Added to a code above in numr_b200_gemm_desc.activation: the backward form of the epilogue,
   * out = residual * activation'(scale * acc + bias), the residual operand carrying the incoming
   * gradient (numr's grad_pre, src/runtime/cpu/kernels/gemm_epilogue/backward.rs:183-204). */
  NUMR_B200_ACT_BWD = 16
} numr_b200_activation;

typedef enum {
  NUMR_B200_B_KN = 0, /* B is [K,N] row-major: the launchers' contract */
  NUMR_B200_B_NK = 1  /* B is [N,K] row-major: a transposed view (strides [1,K]) used without a copy */
} numr_b200_b_layout;

typedef enum {
  NUMR_B200_F32_EXACT = 0, /* three TF32 products per term (hi*hi + hi*lo + lo*hi): <= 1e-5 rel. Frobenius */
  NUMR_B200_F32_TF32 = 1   /* operands rounded to TF32 (round-to-nearest): <= 1e-3 rel. Frobenius */
} numr_b200_f32_mode;

/*
 * One GEMM with its fused epilogue:
 *   acc   = sum_k A[bi % a_batch][i,k] * B[bi % b_batch][k,j]     f32 (s32 for I8) accumulation
 *   x     = scale_a*scale_b*acc + bias[j]                          bias optional
 *   y     = activation(x) + residual[bi][i,j]                      residual optional
 *   C[bi][i,j] = cast<out_dtype>(y)                                one rounding (one saturation for I32)
 * Type rules follow src/ops/matmul_dtype.rs:19-100: F32/BF16/F16 keep their type,
 * I8 x I8 gives I32 with an I32 bias that seeds the accumulator, I16/I32/I64/U8/U16/U32/U64 keep
 * their type (128-bit accumulation, bias of the same type seeds it, one saturating store; no
 * activation or residual), FP8 inputs give
 * F32/F16/BF16 (fp8_matmul) or the input FP8 type (plain matmul on FP8 tensors).
 * Activation and residual are rejected for I8, as numr rejects I8 in the epilogue ops.
 */
typedef struct {
  int32_t a_dtype, b_dtype;     /* equal, except FP8E5M2 x FP8E4M3 (fp8_matmul_e5m2) */
  int32_t out_dtype;
  int32_t bias_dtype;           /* = out_dtype for floats; I32 for I8; ignored when bias == NULL */
  uint32_t batch;               /* output batch count (>= 1) */
  uint32_t m, n, k;
  uint32_t a_batch, b_batch;    /* operand batch counts; operand index = bi % count (loader/matmul.rs:284) */
  int32_t b_layout;             /* numr_b200_b_layout */
  int32_t activation;           /* numr_b200_activation */
  int32_t f32_mode;             /* numr_b200_f32_mode; read only when a_dtype == F32 */
  float scale_a, scale_b;       /* FP8 per-tensor scales (ops/traits/fp8_matmul.rs:19-28); 1.0 otherwise */
} numr_b200_gemm_desc;

/* Mirror of what the launch path reads from numr's Tensor<CudaRuntime>
 * (src/tensor/core.rs: ptr() with the view offset applied, shape(), strides() in
 * elements, dtype()). Up to 8 dimensions. */
typedef struct {
  uint64_t ptr;
  int32_t dtype;
  int32_t ndim;
  int64_t shape[8];
  int64_t strides[8];
} numr_b200_tensor;

const char* numr_b200_version(void);

/* Text of the last non-OK status returned on the calling thread (static storage). */
const char* numr_b200_last_error(void);

/* Bytes of caller-provided scratch numr_b200_gemm needs for this problem: TF32
 * rounding / hi-lo split of F32 operands, and a padded copy of any operand whose
 * address or row pitch is not 16-byte aligned (TMA requirement; the reference
 * kernels fall back to scalar loads instead, matmul_wmma_stage.cuh:26-28).
 * `a` and `b` may be NULL, meaning "16-byte aligned". On a machine with an sm_100 GPU the figure also
 * includes optional scratch for splitting the tiles of the kernel's last, partly filled wave along K
 * (32-bit partial sums, combined in a fixed order, so results stay bitwise reproducible); a workspace
 * that covers only the operand preparation is accepted and simply disables that split.
 * Returns 0 when none is needed. */
size_t numr_b200_gemm_workspace_bytes(const numr_b200_gemm_desc* desc, const void* a, const void* b);

/* Launches the GEMM on `cu_stream` (a CUstream / cudaStream_t; NULL = legacy default
 * stream) of the current context. `workspace` must be 256-byte aligned and at least
 * numr_b200_gemm_workspace_bytes() long; it may be NULL when that is 0.
 * Replaces: launch_matmul_kernel / launch_matmul_batched_kernel (loader/matmul.rs:64,284),
 * launch_matmul_bias_kernel (loader/matmul_bias.rs:46,254), launch_gemm_bias_act_kernel and
 * launch_gemm_bias_residual_kernel (kernels/gemm_epilogue/launcher.rs:35,153,278,398),
 * launch_fp8_matmul_e4m3/_e5m2 (kernels/fp8_matmul.rs:51,101,151,204). */
numr_b200_status numr_b200_gemm(const numr_b200_gemm_desc* desc, const void* a, const void* b,
                                const void* bias, const void* residual, void* c, void* workspace,
                                size_t workspace_bytes, void* cu_stream, int device_index);

/* numr_b200_gemm fused with the all-gather of its output over NVLink: for a GEMM whose N is one of
 * `world` equal column blocks of a larger [batch][M][world * N] result (the column-parallel split:
 * every rank holds all of A and its own block of B's columns). Instead of writing a local
 * [M, N] block that a collective then copies around (numr's Communicator::all_gather,
 * src/runtime/communicator/traits.rs:82-94, concatenates along the LEADING dimension, so a
 * re-interleave pass follows it), the epilogue stores every finished tile straight into column block
 * `rank` of EVERY rank's row-major [batch][M][world * N] buffer: c_ptrs[r] is the base address of rank
 * r's buffer as mapped into this process (c_ptrs[rank] this rank's own; the others peer memory, e.g.
 * CUDA IPC or symmetric-memory mappings). Peer buffers are only ever written (tiled bulk stores, no
 * multicast, no load from peer memory). The call does not synchronise ranks: the caller orders "all
 * ranks' kernels finished" before reading a buffer, and "all ranks finished reading" before the next
 * write (a barrier on the stream, numr's Communicator::barrier). Needs N * sizeof(out) to be a
 * multiple of 16 and 16-byte aligned buffers; 1 <= world <= 8. Everything else as numr_b200_gemm. */
numr_b200_status numr_b200_gemm_allgather(const numr_b200_gemm_desc* desc, const void* a, const void* b,
                                          const void* bias, const void* residual, const uint64_t* c_ptrs,
                                          uint32_t world, uint32_t rank, void* workspace,
                                          size_t workspace_bytes, void* cu_stream, int device_index);

/* Bytes of scratch built into the library for numr_b200_gemm_static_scratch. */
#define NUMR_B200_STATIC_SCRATCH_BYTES (16u << 20)
size_t numr_b200_static_scratch_bytes(void);

/* numr_b200_gemm for callers that have no device allocator to ask for a workspace: code that runs
 * inside another framework's stream callback or custom-op hook, a host that is replaying a captured
 * graph with its allocator frozen (numr freezes its own during capture, runtime.rs:427-513), or an
 * embedding that was handed input and output buffers and nothing else. The scratch the GEMM needs
 * (TF32 parts of F32 operands, re-pitched copies of misaligned operands) comes from a fixed
 * NUMR_B200_STATIC_SCRATCH_BYTES (16 MiB) array inside the library's device image instead; every GPU
 * that loads the library carries those 16 MiB until the process exits. Enough for, e.g., an exact-mode
 * F32 GEMM with M*K + K*N <= 2 Mi elements (1024^3), or TF32 mode at twice that.
 *  - Problems that need more scratch are refused with NUMR_B200_EWORKSPACE before anything is launched.
 *  - It calls no cudaMalloc / cudaFree or any other allocating routine; inputs and output are the caller's.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *    device current); make that first call outside any stream capture.
 *  - The integer widths without a tensor-core kernel (I16 ... U64) use no scratch and pass straight through.
 *  - All calls on one device share the one array, and it keeps whatever the previous call left in it;
 *    the GEMM overwrites every byte it later reads, so nothing has to be cleared, but two calls whose
 *    kernels can overlap on the GPU (different streams) race on it: serialise them on one stream.
 * No counterpart in the reference: its launchers always receive allocator-backed buffers. */
numr_b200_status numr_b200_gemm_static_scratch(const numr_b200_gemm_desc* desc, const void* a,
                                               const void* b, const void* bias, const void* residual,
                                               void* c, void* cu_stream, int device_index);

/* Does the library's first-use work for the calling thread's current device, which `device_index`
 * (when >= 0) must name: device query, the kernels' shared-memory attributes, the cluster occupancy
 * query, the addresses of the status word and of the built-in scratch, the NUMR_B200_* switches.
 * Optional (the first launch on a device does the same), but that first-use work calls runtime
 * functions that are not legal inside a stream capture: a caller that captures CUDA graphs calls
 * this once per device beforehand; after it, the entry points only encode tensor maps (host side)
 * and launch. Every entry point that takes a `device_index` returns NUMR_B200_EINVAL when it is
 * >= 0 and differs from the current device (numr binds its context to the thread before launching,
 * src/runtime/cuda/client.rs:128-131). A cudaDeviceReset() discards what this call set up. */
numr_b200_status numr_b200_init(int device_index);

/* Reads and clears the device-side status word of the current device (0 = every
 * bounded wait completed). Synchronises the device; meant for tests and health
 * checks, not for the launch path. */
numr_b200_status numr_b200_device_status(int* kernel_status);

/* Re-reads the NUMR_B200_* environment switches (tile width, CTA pairs, K blocks per stage, K split,
 * small-M dispatch, wait limit). The library reads them once, at its first launch; tests and
 * experiments that change one afterwards call this. Nothing in normal use needs it. No counterpart
 * in the reference (its tile choice has no switches, loader/matmul_config.rs:67-70). */
void numr_b200_reload_tuning(void);

/* ---- launcher mirrors: same names and argument order as the Rust launchers they
 * replace (ctx/stream collapse into cu_stream; a workspace pair is appended). ---- */

/* loader/matmul.rs:64 */
numr_b200_status numr_b200_launch_matmul_kernel(void* cu_stream, int device_index, int32_t dtype,
                                                uint64_t a, uint64_t b, uint64_t c, size_t m,
                                                size_t n, size_t k, void* ws, size_t ws_bytes);
/* loader/matmul.rs:284 */
numr_b200_status numr_b200_launch_matmul_batched_kernel(void* cu_stream, int device_index,
                                                        int32_t dtype, uint64_t a, uint64_t b,
                                                        uint64_t c, size_t batch, size_t m, size_t n,
                                                        size_t k, size_t a_batch, size_t b_batch,
                                                        void* ws, size_t ws_bytes);
/* loader/matmul_bias.rs:46 */
numr_b200_status numr_b200_launch_matmul_bias_kernel(void* cu_stream, int device_index, int32_t dtype,
                                                     uint64_t a, uint64_t b, uint64_t bias,
                                                     uint64_t c, size_t m, size_t n, size_t k,
                                                     void* ws, size_t ws_bytes);
/* loader/matmul_bias.rs:254 */
numr_b200_status numr_b200_launch_matmul_bias_batched_kernel(void* cu_stream, int device_index,
                                                             int32_t dtype, uint64_t a, uint64_t b,
                                                             uint64_t bias, uint64_t c, size_t batch,
                                                             size_t m, size_t n, size_t k,
                                                             size_t a_batch, size_t b_batch, void* ws,
                                                             size_t ws_bytes);
/* kernels/gemm_epilogue/launcher.rs:35 */
numr_b200_status numr_b200_launch_gemm_bias_act_kernel(void* cu_stream, int device_index,
                                                       int32_t dtype, uint64_t a, uint64_t b,
                                                       uint64_t bias, uint64_t c, size_t m, size_t n,
                                                       size_t k, int32_t activation, void* ws,
                                                       size_t ws_bytes);
/* kernels/gemm_epilogue/launcher.rs:153 (A, B, C advance one full matrix per batch) */
numr_b200_status numr_b200_launch_gemm_bias_act_batched_kernel(void* cu_stream, int device_index,
                                                               int32_t dtype, uint64_t a, uint64_t b,
                                                               uint64_t bias, uint64_t c, size_t batch,
                                                               size_t m, size_t n, size_t k,
                                                               int32_t activation, void* ws,
                                                               size_t ws_bytes);
/* kernels/gemm_epilogue/launcher.rs:278 */
numr_b200_status numr_b200_launch_gemm_bias_residual_kernel(void* cu_stream, int device_index,
                                                            int32_t dtype, uint64_t a, uint64_t b,
                                                            uint64_t bias, uint64_t residual,
                                                            uint64_t c, size_t m, size_t n, size_t k,
                                                            void* ws, size_t ws_bytes);
/* kernels/gemm_epilogue/launcher.rs:398 */
numr_b200_status numr_b200_launch_gemm_bias_residual_batched_kernel(
    void* cu_stream, int device_index, int32_t dtype, uint64_t a, uint64_t b, uint64_t bias,
    uint64_t residual, uint64_t c, size_t batch, size_t m, size_t n, size_t k, void* ws,
    size_t ws_bytes);
/* kernels/fp8_matmul.rs:51,101 (batch = 1 for the unbatched form) */
numr_b200_status numr_b200_launch_fp8_matmul_e4m3(void* cu_stream, int device_index,
                                                  int32_t out_dtype, uint64_t a, uint64_t b,
                                                  uint64_t out, float scale_a, float scale_b,
                                                  size_t batch, size_t m, size_t n, size_t k, void* ws,
                                                  size_t ws_bytes);
/* kernels/fp8_matmul.rs:151,204 (A is E5M2, B is E4M3) */
numr_b200_status numr_b200_launch_fp8_matmul_e5m2(void* cu_stream, int device_index,
                                                  int32_t out_dtype, uint64_t a, uint64_t b,
                                                  uint64_t out, float scale_a, float scale_b,
                                                  size_t batch, size_t m, size_t n, size_t k, void* ws,
                                                  size_t ws_bytes);

/* ---- op layer: the validation, shape and dispatch rules of numr's CUDA op impls
 * (src/ops/cuda/{matmul,gemm_epilogue,fp8_matmul}.rs with src/ops/matmul.rs and
 * src/ops/matmul_dtype.rs), over tensor descriptors. The caller allocates `out`
 * (contiguous, shape from the *_out_shape call) and the workspace. ---- */

/* matmul_output_shape / matmul_bias_output_shape (src/ops/matmul.rs:73-102,245-255) with
 * the output dtype rule (matmul_dtype.rs:19-25). `bias` may be NULL. */
numr_b200_status numr_b200_matmul_out_shape(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                            const numr_b200_tensor* bias, int64_t out_shape[8],
                                            int32_t* out_ndim, int32_t* out_dtype);

/* Workspace the op-layer calls below need for these operands (includes gathering
 * non-contiguous views other than the transposed-B view). */
size_t numr_b200_op_workspace_bytes(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                    int32_t out_dtype, int32_t f32_mode);
/* The same for one particular call: `bias` and `residual` are the tensors the op will get (NULL =
 * none). The figure above budgets a gather of a non-contiguous bias and residual whether or not
 * there is one (an extra buffer the size of the output); this one adds them only when needed. */
size_t numr_b200_op_workspace_bytes_for(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                        const numr_b200_tensor* bias, const numr_b200_tensor* residual,
                                        int32_t out_dtype, int32_t f32_mode);

/* MatmulOps::matmul (src/ops/traits/matmul.rs:12; CUDA impl src/ops/cuda/matmul.rs:17-146). */
numr_b200_status numr_b200_matmul(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                  const numr_b200_tensor* out, int32_t f32_mode, void* ws,
                                  size_t ws_bytes, void* cu_stream, int device_index);
/* MatmulOps::matmul_bias (src/ops/traits/matmul.rs:107; src/ops/cuda/matmul.rs:148-288). */
numr_b200_status numr_b200_matmul_bias(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                       const numr_b200_tensor* bias, const numr_b200_tensor* out,
                                       int32_t f32_mode, void* ws, size_t ws_bytes, void* cu_stream,
                                       int device_index);
/* GemmEpilogueOps::matmul_bias_activation (src/ops/traits/gemm_epilogue.rs:66;
 * src/ops/cuda/gemm_epilogue.rs:25-139). */
numr_b200_status numr_b200_matmul_bias_activation(const numr_b200_tensor* a,
                                                  const numr_b200_tensor* b,
                                                  const numr_b200_tensor* bias, int32_t activation,
                                                  const numr_b200_tensor* out, int32_t f32_mode,
                                                  void* ws, size_t ws_bytes, void* cu_stream,
                                                  int device_index);
/* activation(A @ B) without a bias: the form the column-sharded MLP projection uses. The
 * reference has it only inside its grouped GEMM (matmul_wmma.cuh:251); here it is the
 * matmul_bias_activation path with the bias term left out. I8 is rejected as there. */
numr_b200_status numr_b200_matmul_activation(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                             int32_t activation, const numr_b200_tensor* out,
                                             int32_t f32_mode, void* ws, size_t ws_bytes,
                                             void* cu_stream, int device_index);
/* GemmEpilogueOps::matmul_bias_residual (src/ops/traits/gemm_epilogue.rs:105;
 * src/ops/cuda/gemm_epilogue.rs:141-256). */
numr_b200_status numr_b200_matmul_bias_residual(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                                const numr_b200_tensor* bias,
                                                const numr_b200_tensor* residual,
                                                const numr_b200_tensor* out, int32_t f32_mode,
                                                void* ws, size_t ws_bytes, void* cu_stream,
                                                int device_index);
/* Fp8MatmulOps::fp8_matmul / fp8_matmul_e5m2 (src/ops/traits/fp8_matmul.rs:57-92;
 * src/ops/cuda/fp8_matmul.rs:81-214); `a_e5m2` selects the E5M2 x E4M3 form. */
numr_b200_status numr_b200_fp8_matmul(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                      float scale_a, float scale_b, int32_t a_e5m2,
                                      const numr_b200_tensor* out, void* ws, size_t ws_bytes,
                                      void* cu_stream, int device_index);
/* The fused FP8 form, a superset of the reference API (FP8 GEMM + bias + activation + residual):
 * out = cast(act(scale_a*scale_b*acc + bias) + residual); bias/residual carry out's dtype. */
numr_b200_status numr_b200_fp8_matmul_fused(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                            float scale_a, float scale_b,
                                            const numr_b200_tensor* bias, int32_t activation,
                                            const numr_b200_tensor* residual,
                                            const numr_b200_tensor* out, void* ws, size_t ws_bytes,
                                            void* cu_stream, int device_index);

/* ---- grouped (MoE) matmul: GroupedMatmulOps (src/ops/traits/grouped_matmul.rs:31-52; CUDA:
 * src/ops/cuda/grouped_matmul.rs, kernels/grouped_matmul.cu, matmul_wmma.cu:84-140) ----
 * c[offsets[g] .. offsets[g+1]] = act(a[offsets[g] .. offsets[g+1]] @ b[g]) with the offsets ON THE
 * DEVICE (int32, groups + 1 entries, non-decreasing, first 0, last = rows of a). F32 / F16 / BF16.
 * A small kernel turns the offsets into a list of row tiles; the GEMM kernel's tile loop reads
 * it, so nothing is read back to the host. Groups with end <= start or end > rows are skipped (as
 * numr's CPU path does); rows that belong to no group are left as they were.
 *
 * Descriptor level: d->m = rows of a, d->batch = 1, d->a_batch = 1, d->b_batch = groups; d->b_layout
 * says whether each b[g] is [K,N] or [N,K]; no bias, no residual; activation as in the descriptor. */
size_t numr_b200_grouped_gemm_workspace_bytes(const numr_b200_gemm_desc* desc, uint32_t groups,
                                              const void* a, const void* b);
numr_b200_status numr_b200_grouped_gemm(const numr_b200_gemm_desc* desc, uint32_t groups, const void* a,
                                        const void* b, const int32_t* group_offsets, void* c,
                                        void* workspace, size_t workspace_bytes, void* cu_stream,
                                        int device_index);
/* Tensor level: a [rows, k], b [groups, k, n], group_offsets [groups + 1] I32, out [rows, n], all
 * contiguous. `activation` is a numr_b200_activation code (NONE for grouped_matmul). Errors follow
 * validate_grouped (src/ops/cpu/grouped_matmul.rs:13-75): wrong ranks, offsets not I32, dtype
 * mismatch or a dtype other than F32/F16/BF16, wrong offsets length -> EINVAL; k mismatch -> ESHAPE. */
size_t numr_b200_grouped_matmul_workspace_bytes(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                                int32_t f32_mode);
numr_b200_status numr_b200_grouped_matmul(const numr_b200_tensor* a, const numr_b200_tensor* b,
                                          const numr_b200_tensor* group_offsets, int32_t activation,
                                          const numr_b200_tensor* out, int32_t f32_mode, void* ws,
                                          size_t ws_bytes, void* cu_stream, int device_index);

/* ---- backward of the fused epilogue: GemmEpilogueOps::matmul_bias_activation_bwd
 * (src/ops/traits/gemm_epilogue.rs:107-140; src/ops/cuda/gemm_epilogue.rs:258-366; CPU kernel
 * src/runtime/cpu/kernels/gemm_epilogue/backward.rs:136-245) ----
 * grad_pre = grad * activation'(a @ b + bias) (one GEMM with the backward epilogue), d_bias = column
 * sums of grad_pre, d_a = grad_pre @ b^T, d_b = a^T @ grad_pre: three tensor-core GEMMs where the
 * reference runs per-element dot products. 2-D operands: a [M,K], b [K,N] (contiguous, or the
 * transposed view of a contiguous [N,K]), grad [M,N], bias [N]; outputs d_a [M,K], d_b [K,N],
 * d_bias [N], contiguous, of the operands' dtype (F32, F16, BF16). grad_pre is kept in that dtype
 * between the GEMMs (the reference keeps it in f32). */
size_t numr_b200_matmul_bias_activation_bwd_workspace_bytes(const numr_b200_tensor* grad,
                                                            const numr_b200_tensor* a,
                                                            const numr_b200_tensor* b,
                                                            const numr_b200_tensor* bias, int32_t f32_mode);
numr_b200_status numr_b200_matmul_bias_activation_bwd(const numr_b200_tensor* grad, const numr_b200_tensor* a,
                                                      const numr_b200_tensor* b, const numr_b200_tensor* bias,
                                                      int32_t activation, const numr_b200_tensor* d_a,
                                                      const numr_b200_tensor* d_b, const numr_b200_tensor* d_bias,
                                                      int32_t f32_mode, void* ws, size_t ws_bytes,
                                                      void* cu_stream, int device_index);

/* ---- convolutions as GEMM: the im2col + matmul fast paths of numr's CUDA back end
 * (src/ops/cuda/conv1d_im2col.rs:100-157, conv2d_im2col.rs:104-158, conv_transpose1d_gemm.rs:108-162;
 * gather kernels src/runtime/cuda/kernels/{im2col,im2col2d,col_transpose1d}.cu) ----
 * out[n] [C_out, L_out] = W [C_out, C_in*Kh*Kw] @ col[n] + bias[C_out]: one gather kernel writes the
 * column buffer (rows padded to 16 bytes; for F32 directly as the TF32 parts the tensor cores read),
 * the tcgen05 GEMM reads it in place and adds the bias (one value per output channel = per GEMM row)
 * in its epilogue. groups must be 1, dtype F32 / F16 / BF16 (what the reference's GEMM path takes;
 * everything else stays on its direct kernels). Tensors are contiguous NCHW:
 *   conv1d            input [N, C_in, L],    weight [C_out, C_in, K],      out [N, C_out, L_out]
 *   conv2d            input [N, C_in, H, W], weight [C_out, C_in, Kh, Kw], out [N, C_out, H_out, W_out]
 *   conv_transpose1d  input [N, C_in, L],    weight [C_in, C_out, K],      out [N, C_out, L_out]
 * with the resolved paddings of validate_conv1d / validate_conv2d / validate_conv_transpose1d
 * (src/ops/conv_common.rs:146-161,317-334,390-414; conv_transpose_common.rs:52-67,173-199). The 1-D
 * forms use the _w fields and leave the _h fields neutral (in_h = kernel_h = stride_h = dilation_h = 1,
 * pad_top = pad_bottom = 0). `bias` may be NULL. */
typedef struct numr_b200_conv_desc {
  int32_t dtype;                       /* numr_b200_dtype: F32, F16 or BF16 (input, weight, bias and output alike) */
  uint32_t batch, c_in, c_out, groups; /* groups must be 1 */
  uint32_t in_h, in_w;                 /* 1-D forms: in_h = 1, in_w = L */
  uint32_t kernel_h, kernel_w;
  uint32_t stride_h, stride_w;
  uint32_t pad_top, pad_bottom, pad_left, pad_right;
  uint32_t dilation_h, dilation_w;
  uint32_t output_padding;             /* conv_transpose1d only */
  int32_t f32_mode;                    /* numr_b200_f32_mode */
} numr_b200_conv_desc;

typedef enum numr_b200_conv_kind { NUMR_B200_CONV1D = 0, NUMR_B200_CONV2D = 1, NUMR_B200_CONV_TRANSPOSE1D = 2 } numr_b200_conv_kind;

/* Output extents (compute_output_size / compute_transpose_output_size); out_h is 1 for the 1-D forms. */
numr_b200_status numr_b200_conv_out_shape(const numr_b200_conv_desc* desc, int32_t kind, uint32_t* out_h,
                                          uint32_t* out_w);
/* Workspace: the column buffer, a prepared copy of the weight when it cannot be read in place (F32,
 * conv_transpose1d's [C_in, C_out, K] layout, a row pitch that is not a multiple of 16 bytes; `weight`
 * may be NULL = "16-byte aligned") and the optional scratch of the GEMM's K cut. */
size_t numr_b200_conv_workspace_bytes(const numr_b200_conv_desc* desc, int32_t kind, const void* weight);
/* conv1d_im2col (src/ops/cuda/conv1d_im2col.rs:100) */
numr_b200_status numr_b200_conv1d(const numr_b200_conv_desc* desc, const void* input, const void* weight,
                                  const void* bias, void* out, void* workspace, size_t workspace_bytes,
                                  void* cu_stream, int device_index);
/* conv2d_im2col (src/ops/cuda/conv2d_im2col.rs:104) */
numr_b200_status numr_b200_conv2d(const numr_b200_conv_desc* desc, const void* input, const void* weight,
                                  const void* bias, void* out, void* workspace, size_t workspace_bytes,
                                  void* cu_stream, int device_index);
/* conv_transpose1d_gemm (src/ops/cuda/conv_transpose1d_gemm.rs:108) */
numr_b200_status numr_b200_conv_transpose1d(const numr_b200_conv_desc* desc, const void* input,
                                            const void* weight, const void* bias, void* out, void* workspace,
                                            size_t workspace_bytes, void* cu_stream, int device_index);

#ifdef __cplusplus
}
#endif
#endif /* NUMR_B200_H */
