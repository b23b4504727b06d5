// Cycles per tcgen05.mma.cta_group::2 (clusters of two CTAs, M = 256) for N = 64 / 128 / 256 by K blocks per
// stage and by commit style (two commits, or one commit with .multicast::cluster). No loads: zeroed shared memory.
// Build and run on a B200 (from the repository root):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr -Iinclude \
//        -o mma_issue_pair numr_b200/csrc/microbench/mma_issue_pair.cu && ./mma_issue_pair
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include "../gemm_kernel.cuh"
using namespace nb;

__device__ __forceinline__ void umma_commit_pair_mc(uint32_t bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}

// COMMIT: 0 = two commits (own barrier, peer's barrier), 1 = one multicast commit
template <int COMMIT>
__global__ void __launch_bounds__(192, 1) pair_bench(uint32_t idesc, int stages_n, int ks, unsigned long long* cycles) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint32_t tmem_slot;
  __shared__ uint64_t bars[8];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  for (uint32_t i = threadIdx.x; i < 49152 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem_raw + (smem_base - smem_u32(smem_raw)))[i] = 0;
  if (threadIdx.x == 0) { for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&bars[i]), 1); fence_barrier_init(); }
  if (warp == 1) { tmem_alloc_pair(smem_u32(&tmem_slot), kTmemCols); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 1) {
    if (rank == 0) {
      const uint32_t a_hi32 = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t a_lo_fixed = (16u >> 4) << 16;
      const uint32_t a_units0 = (smem_base & 0x3FFFF) >> 4;
      const uint32_t b_off_units = 16384u >> 4;
      auto desc = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      const uint32_t empty0 = smem_u32(&bars[0]);
      uint32_t stage = 0;
      __syncwarp();
      const unsigned long long t0 = clock64();
      for (int s = 0; s < stages_n; ++s) {
        uint32_t al[4], bl[4];
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {
          al[kk] = a_units0 | a_lo_fixed;
          bl[kk] = (a_units0 + b_off_units) | a_lo_fixed;
        }
        if (elect_one()) {
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            if (kk < (uint32_t)ks) {
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j)
                umma_pair<KIND_F16>(tmem_base, desc(a_hi32, al[kk] + j * 2u), desc(a_hi32, bl[kk] + j * 2u), idesc, (s | kk | j) ? 1u : 0u);
            }
          }
          if constexpr (COMMIT == 0) {
            umma_commit_pair(empty0 + stage * 8u);
            umma_commit_pair(mapa(empty0 + stage * 8u, 1));
          } else {
            umma_commit_pair_mc(empty0 + stage * 8u, (uint16_t)3);
          }
        }
        __syncwarp();
        if (++stage == 4) stage = 0;
      }
      const unsigned long long t1 = clock64();
      if (elect_one()) {
        umma_commit_pair(smem_u32(&bars[7]));
        umma_commit_pair(mapa(smem_u32(&bars[7]), 1));
      }
      __syncwarp();
      if (lane == 0) {
        for (uint32_t spin = 0; spin < (1u << 22) && !mbar_try_wait(smem_u32(&bars[7]), 0); ++spin) {}
      }
      __syncwarp();
      const unsigned long long t2 = clock64();
      if (lane == 0) { cycles[(blockIdx.x >> 1) * 2] = t1 - t0; cycles[(blockIdx.x >> 1) * 2 + 1] = t2 - t0; }
    } else {
      // the peer: wait (bounded) until every MMA that read its shared memory and wrote its TMEM has retired
      if (lane == 0) {
        for (uint32_t spin = 0; spin < (1u << 22) && !mbar_try_wait(smem_u32(&bars[7]), 0); ++spin) {}
      }
      __syncwarp();
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, kTmemCols); }
}

template <int COMMIT>
void run(const char* name, uint32_t n, int ks, unsigned long long* d) {
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
  const int stages_n = 256;
  cudaFuncSetAttribute(pair_bench<COMMIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(148); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = 65536;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  for (int rep = 0; rep < 2; ++rep) {
    cudaError_t le = cudaLaunchKernelEx(&cfg, pair_bench<COMMIT>, idesc, stages_n, ks, d);
    cudaError_t e = cudaDeviceSynchronize();
    if (le != cudaSuccess || e != cudaSuccess) { printf("%s: %s / %s\n", name, cudaGetErrorString(le), cudaGetErrorString(e)); exit(1); }
  }
  std::vector<unsigned long long> h(74 * 2);
  cudaMemcpy(h.data(), d, h.size() * 8, cudaMemcpyDeviceToHost);
  std::vector<double> iss, ret;
  const double mmas = (double)stages_n * ks * 4;
  for (int i = 0; i < 74; ++i) { iss.push_back(h[2 * i] / mmas); ret.push_back(h[2 * i + 1] / mmas); }
  std::sort(iss.begin(), iss.end()); std::sort(ret.begin(), ret.end());
  printf("%-26s N=%3u ks=%d  cycles per MMA: issue %.1f  retire %.1f\n", name, n, ks, iss[37], ret[37]);
}

int main() {
  unsigned long long* d;
  cudaMalloc(&d, 148 * 2 * 8);
  for (uint32_t n : {64u, 128u, 256u})
    for (int ks : {1, 2, 4}) {
      run<0>("pair, two commits", n, ks, d);
      run<1>("pair, multicast commit", n, ks, d);
    }
  return 0;
}
