// The tcgen05 GEMM kernels of one instruction kind (see gemm_launch.cuh, gemm_sm100.cu).
#include "gemm_launch.cuh"

namespace pgb {
template int launch_gemm_bn<GEMM_I8>(int, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, cudaStream_t);
}  // namespace pgb
