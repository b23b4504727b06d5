// Cycles per 32-column chunk per epilogue warp for the GEMM kernel's staged finisher (finish_to_stage:
// TMEM read, scale + bias + activation (+ residual), conversion, swizzled staging store), BF16 output, with 4
// and with 8 epilogue warps per SM. No MMAs, no TMA stores: the accumulators are whatever TMEM holds.
// Build and run on a B200 (from the repository root):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr -Iinclude \
//        -o epilogue_chunk numr_b200/csrc/microbench/epilogue_chunk.cu && ./epilogue_chunk
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../gemm_kernel.cuh"
using namespace nb;

// stores: 0 = none; 1 = after every 64-column group the staged 4 KB go out as a bulk copy (fence to the async proxy,
// one lane issues, commit) and a buffer is re-used only once its store has read it, as in the GEMM kernel; `bufs`
// staging buffers per warp (1, 2 or 4).
__global__ void __launch_bounds__(320, 1) epi_bench(const __grid_constant__ KParams p, unsigned long long* cycles,
                                                    int iters, int chunks, int n_epi, int stores, int bufs, uint8_t* sink) {
  extern __shared__ __align__(1024) uint8_t stage[];   // n_epi warps x bufs x 4 KB
  __shared__ __align__(16) uint32_t bias_s[256];
  __shared__ uint32_t tmem_slot;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) bias_s[i] = __float_as_uint(0.01f * (float)i);
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_slot), kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp >= 2 && warp < 2 + (uint32_t)n_epi) {
    const uint32_t quarter = warp & 3;
    const uint32_t stage_buf = smem_u32(stage) + (warp - 2) * (uint32_t)bufs * 4096u;
    uint8_t* my_sink = sink + ((size_t)blockIdx.x * 8 + (warp - 2)) * 4096;
    const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
    uint32_t buf_sel = 0;
    const float rb = p.bias_row ? 0.25f : 0.0f;
    const unsigned long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      for (int g0 = 0; g0 < chunks * 32; g0 += 64) {
        const uint32_t buf = stage_buf + buf_sel * 4096u;
        if (stores) {
          if (lane == 0) {
            if (bufs == 1) bulk_wait_group_read<0>(); else if (bufs == 2) bulk_wait_group_read<1>(); else bulk_wait_group_read<3>();
          }
          __syncwarp();
        }
#pragma unroll
        for (int sub = 0; sub < 64; sub += 32) {
          const uint32_t tc0 = g0 + sub;
          uint32_t r[32];
          tmem_ld_32x32(taddr + (tc0 & 255), r);
          tmem_ld_wait();
          const void* res_row = p.residual ? (const __nv_bfloat16*)p.residual + (size_t)(blockIdx.x * 128 + threadIdx.x) * 256 + (tc0 & 255) : nullptr;
          finish_to_stage<OUT_BF16>(p, r, bias_s, tc0 & 255, sub / 8, buf, lane, res_row, p.vec_ok, p.N, rb);
        }
        if (stores) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 4096;" ::"l"(my_sink), "r"(buf) : "memory");
            bulk_commit_group();
          }
        }
        buf_sel = (buf_sel + 1) % (uint32_t)bufs;
      }
    }
    if (lane == 0) bulk_wait_group_read<0>();
    __syncwarp();
    const unsigned long long t1 = clock64();
    if (lane == 0) cycles[blockIdx.x * 8 + (warp - 2)] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

void run(const char* name, int act, int n_epi, unsigned long long* d_cycles, void* res, int stores, int bufs, uint8_t* sink) {
  KParams p;
  memset(&p, 0, sizeof(p));
  p.act = act; p.scale = 1.0f; p.bias = (const void*)1; p.residual = res; p.vec_ok = 1; p.N = 32;
  const int iters = 50, chunks = 8;
  for (int rep = 0; rep < 2; ++rep) {
    cudaMemset(d_cycles, 0, 148 * 8 * 8);
    epi_bench<<<148, 64 + 32 * n_epi, (size_t)n_epi * bufs * 4096>>>(p, d_cycles, iters, chunks, n_epi, stores, bufs, sink);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("%s: %s\n", name, cudaGetErrorString(e)); exit(1); }
  }
  std::vector<unsigned long long> h(148 * 8);
  cudaMemcpy(h.data(), d_cycles, h.size() * 8, cudaMemcpyDeviceToHost);
  std::vector<double> v;
  for (auto c : h) if (c) v.push_back((double)c / (iters * chunks));
  std::sort(v.begin(), v.end());
  printf("%-22s res=%d act=%d warps=%d stores=%d bufs=%d  cycles per 32-column chunk per warp: median %.0f  (min %.0f max %.0f)  -> per SM per tile of 256 cols %.0f cycles\n",
         name, res ? 1 : 0, act, n_epi, stores, bufs, v[v.size() / 2], v.front(), v.back(), v[v.size() / 2] * 8);
}

int main() {
  unsigned long long* d;
  cudaMalloc(&d, 148 * 8 * 8);
  void* res;
  cudaMalloc(&res, (size_t)148 * 512 * 256 * 2);
  cudaMemset(res, 0, (size_t)148 * 512 * 256 * 2);
  uint8_t* sink;
  cudaMalloc(&sink, (size_t)148 * 8 * 4096);
  cudaFuncSetAttribute(epi_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 4 * 4096);
  for (void* r : {(void*)nullptr, res})
    for (int act : {0, 1, 2, 3})   // none, ReLU, GELU, SiLU
      for (int n_epi : {4, 8}) run("finish_to_stage<BF16>", act, n_epi, d, r, 0, 1, sink);
  // with the stores of the GEMM kernel's epilogue, by the number of staging buffers per warp
  for (int act : {0, 3})
    for (int bufs : {1, 2, 4}) run("finish_to_stage<BF16>", act, 4, d, nullptr, 1, bufs, sink);
  return 0;
}
