// Instantiates the row reduce kernels for f32 inputs, 2 input tensor(s).
#include "reduce_row.cuh"

namespace pgb {
template int launch_row_typed<float, 2>(ReduceJob &j, bool ident, const ChainProg<float> &chain);
}  // namespace pgb
