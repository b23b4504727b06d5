// Cycles per tcgen05.mma (one CTA per SM, M = 128) for N = 64 / 128 / 256, BF16 and TF32, by issue-loop style:
// one thread with fixed descriptors (the floor), the kernel's own loop with 1 / 2 / 4 K blocks per stage, commits
// held back, and the exact-F32 form (three MMAs per step). No loads: the operands are zeroed shared memory.
// Build and run on a B200 (from the repository root):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr -Iinclude \
//        -o mma_issue numr_b200/csrc/microbench/mma_issue.cu && ./mma_issue
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include "../gemm_kernel.cuh"
using namespace nb;

template <int KIND, int STYLE>
__global__ void __launch_bounds__(192, 1) mma_bench(uint32_t idesc, int stages_n, int ks, unsigned long long* cycles, uint32_t* sink, int cb) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint32_t tmem_slot;
  __shared__ uint64_t bars[8];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t i = threadIdx.x; i < 49152 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem_raw + (smem_base - smem_u32(smem_raw)))[i] = 0;
  if (threadIdx.x == 0) { for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&bars[i]), 1); fence_barrier_init(); }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_slot), kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 1) {
    const uint32_t a_hi32 = (1024u >> 4) | (1u << 14) | (2u << 29);
    const uint32_t b_hi32 = a_hi32;
    const uint32_t a_lo_fixed = (16u >> 4) << 16;
    const uint32_t a_units0 = (smem_base & 0x3FFFF) >> 4;
    const uint32_t b_off_units = 16384u >> 4;
    const uint32_t a_kk_units = 0, b_kk_units = 0;   // every K block reads the same (zeroed) bytes
    const uint32_t b_step_units = 2;
    auto desc = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | lo; };
    const uint32_t empty0 = smem_u32(&bars[0]);
    uint32_t stage = 0;
    __syncwarp();
    const unsigned long long t0 = clock64();
    if constexpr (STYLE == 0) {
      // the product's loop: the warp walks in step, one elected lane issues, a commit per stage
      uint32_t a_units = a_units0;
      for (int s = 0; s < stages_n; ++s) {
        uint32_t al[4], bl[4];
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {
          al[kk] = (a_units + kk * a_kk_units) | a_lo_fixed;
          bl[kk] = (a_units + b_off_units + kk * b_kk_units) | a_lo_fixed;
        }
        if (elect_one()) {
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            if (kk < (uint32_t)ks) {
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j)
                umma<KIND>(tmem_base, desc(a_hi32, al[kk] + j * 2u), desc(b_hi32, bl[kk] + j * b_step_units), idesc, (s | kk | j) ? 1u : 0u);
            }
          }
          umma_commit(empty0 + stage * 8u);
        }
        __syncwarp();
        if (++stage == 4) stage = 0;
      }
    } else if constexpr (STYLE == 1) {
      // one thread, fixed descriptors, no commits inside
      if (lane == 0) {
        const uint64_t da = desc(a_hi32, a_units0 | a_lo_fixed), db = desc(b_hi32, (a_units0 + b_off_units) | a_lo_fixed);
        for (int s = 0; s < stages_n; ++s) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < ks * 4) umma<KIND>(tmem_base, da, db, idesc, 1u);
        }
      }
    } else if constexpr (STYLE == 3) {
      // the product's loop, commits held back and issued together every `cb` stages
      uint32_t a_units = a_units0;
      for (int s = 0; s < stages_n; ++s) {
        uint32_t al[4], bl[4];
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {
          al[kk] = (a_units + kk * a_kk_units) | a_lo_fixed;
          bl[kk] = (a_units + b_off_units + kk * b_kk_units) | a_lo_fixed;
        }
        if (elect_one()) {
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            if (kk < (uint32_t)ks) {
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j)
                umma<KIND>(tmem_base, desc(a_hi32, al[kk] + j * 2u), desc(b_hi32, bl[kk] + j * b_step_units), idesc, (s | kk | j) ? 1u : 0u);
            }
          }
          if ((s + 1) % cb == 0)
            for (int c = 0; c < cb; ++c) umma_commit(empty0 + ((stage + 8 - c) & 3) * 8u);
        }
        __syncwarp();
        if (++stage == 4) stage = 0;
      }
    } else {
      // the product's loop with three MMAs per step (exact-F32 form)
      uint32_t a_units = a_units0;
      for (int s = 0; s < stages_n; ++s) {
        uint32_t al[4], bl[4];
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {
          al[kk] = (a_units + kk * a_kk_units) | a_lo_fixed;
          bl[kk] = (a_units + b_off_units + kk * b_kk_units) | a_lo_fixed;
        }
        if (elect_one()) {
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            if (kk < (uint32_t)ks) {
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j) {
                const uint64_t a_hi = desc(a_hi32, al[kk] + j * 2u), a_lo = desc(a_hi32, al[kk] + 256u + j * 2u);
                const uint64_t b_hi = desc(b_hi32, bl[kk] + j * b_step_units), b_lo = desc(b_hi32, bl[kk] + 128u + j * b_step_units);
                umma<KIND>(tmem_base, a_lo, b_hi, idesc, (s | kk | j) ? 1u : 0u);
                umma<KIND>(tmem_base, a_hi, b_lo, idesc, 1u);
                umma<KIND>(tmem_base, a_hi, b_hi, idesc, 1u);
              }
            }
          }
          umma_commit(empty0 + stage * 8u);
        }
        __syncwarp();
        if (++stage == 4) stage = 0;
      }
    }
    const unsigned long long t1 = clock64();   // all issued
    if (elect_one()) {
      umma_commit(smem_u32(&bars[7]));
      for (uint32_t spin = 0; spin < (1u << 22) && !mbar_try_wait(smem_u32(&bars[7]), 0); ++spin) {}
    }
    __syncwarp();
    const unsigned long long t2 = clock64();   // all retired
    if (lane == 0) { cycles[blockIdx.x * 2] = t1 - t0; cycles[blockIdx.x * 2 + 1] = t2 - t0; }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
  if (threadIdx.x == 0 && sink) sink[0] = tmem_base;
}

template <int KIND, int STYLE>
void run(const char* name, uint32_t n, int ks, unsigned long long* d, int cb = 1) {
  const uint32_t fmt = KIND == KIND_TF32 ? 2u : 1u;
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
  const int stages_n = 256;
  cudaFuncSetAttribute(mma_bench<KIND, STYLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
  for (int rep = 0; rep < 2; ++rep) {
    mma_bench<KIND, STYLE><<<148, 192, 65536>>>(idesc, stages_n, ks, d, nullptr, cb);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("%s: %s\n", name, cudaGetErrorString(e)); exit(1); }
  }
  std::vector<unsigned long long> h(148 * 2);
  cudaMemcpy(h.data(), d, h.size() * 8, cudaMemcpyDeviceToHost);
  std::vector<double> iss, ret;
  const double mmas = (double)stages_n * ks * 4 * (STYLE == 2 ? 3 : 1);
  for (int i = 0; i < 148; ++i) { iss.push_back(h[2 * i] / mmas); ret.push_back(h[2 * i + 1] / mmas); }
  std::sort(iss.begin(), iss.end()); std::sort(ret.begin(), ret.end());
  printf("%-38s N=%3u ks=%d cb=%d  cycles per MMA: issue %.1f  retire %.1f\n", name, n, ks, cb, iss[74], ret[74]);
}

int main() {
  unsigned long long* d;
  cudaMalloc(&d, 148 * 2 * 8);
  for (uint32_t n : {64u, 128u, 256u}) {
    run<KIND_F16, 1>("bf16 one thread, fixed descriptors", n, 4, d);
    run<KIND_F16, 0>("bf16 kernel loop", n, 1, d);
    run<KIND_F16, 0>("bf16 kernel loop", n, 2, d);
    run<KIND_F16, 0>("bf16 kernel loop", n, 4, d);
    run<KIND_F16, 3>("bf16 kernel loop, commits held back", n, 1, d, 2);
    run<KIND_TF32, 1>("tf32 one thread, fixed descriptors", n, 4, d);
    run<KIND_TF32, 0>("tf32 kernel loop", n, 1, d);
    run<KIND_TF32, 2>("tf32 kernel loop, 3 MMAs per step", n, 1, d);
    run<KIND_TF32, 2>("tf32 kernel loop, 3 MMAs per step", n, 2, d);
  }
  return 0;
}
