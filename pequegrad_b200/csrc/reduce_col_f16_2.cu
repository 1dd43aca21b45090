// Instantiates the col reduce kernels for f16 inputs, 2 input tensor(s).
#include "reduce_col.cuh"

namespace pgb {
template int launch_col_typed<__half, 2>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
}  // namespace pgb
