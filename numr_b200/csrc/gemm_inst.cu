// One (MMA kind, output kind) instantiation of the tcgen05 GEMM kernel, chosen by the build with
// -DNB_INST_KIND=<MmaKind> -DNB_INST_OUT=<OutKind>. The kernel template lives in gemm_kernel.cuh.
#include "gemm_kernel.cuh"

#if !defined(NB_INST_KIND) || !defined(NB_INST_OUT)
#error "compile with -DNB_INST_KIND=<0..3> -DNB_INST_OUT=<0..5>"
#endif

namespace nb {
template cudaError_t gemm_inst_launch<NB_INST_KIND, NB_INST_OUT>(const KParams&, uint32_t, size_t, cudaStream_t, bool, bool);
template cudaError_t gemm_inst_set_smem_attr<NB_INST_KIND, NB_INST_OUT>();
template cudaError_t gemm_inst_max_clusters<NB_INST_KIND, NB_INST_OUT>(int*, const cudaLaunchConfig_t*, bool);
}  // namespace nb
