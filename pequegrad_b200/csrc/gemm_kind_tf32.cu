// The tcgen05 GEMM kernels of one instruction kind (see gemm_launch.cuh, gemm_sm100.cu).
#include "gemm_launch.cuh"
#include "gemm_pair.cuh"

namespace pgb {
template int launch_gemm_bn<GEMM_TF32>(int, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, cudaStream_t);
template int launch_gemm_pair<GEMM_TF32>(const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, cudaStream_t);
}  // namespace pgb
