// Instantiates the col reduce kernels for f16 inputs, 1 input tensor(s).
#include "reduce_col.cuh"

namespace pgb {
template int launch_col_typed<__half, 1>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
}  // namespace pgb
