// Dispatcher of the row reduce family; the kernels are instantiated in reduce_row_*.cu
// (one translation unit per input type and input count, so they compile in parallel).
#include "reduce_row.cuh"

namespace pgb {

extern template int launch_row_typed<float, 1>(ReduceJob &j, bool ident, const ChainProg<float> &chain);
extern template int launch_row_typed<float, 2>(ReduceJob &j, bool ident, const ChainProg<float> &chain);
extern template int launch_row_typed<__half, 1>(ReduceJob &j, bool ident, const ChainProg<float> &chain);
extern template int launch_row_typed<__half, 2>(ReduceJob &j, bool ident, const ChainProg<float> &chain);

int launch_reduce_row(ReduceJob &j) {
  const CanonReduce &c = j.c;
  if (j.cdtype != PGB_F32) return 0;
  if (c.n_in > 2 || c.nr < 1 || c.nr > 2 || c.nk > 3) return 0;
  if (j.rop == ROP_ARGMAX && c.nr != 1) return 0;
  const int dt = j.in[0].dtype;
  if (dt != PGB_F32 && dt != PGB_F16) return 0;
  bool any1 = false;
  for (int k = 0; k < c.n_in; ++k) {
    if (j.in[k].dtype != dt) return 0;
    const int64_t s = c.rin[k][c.nr - 1];
    if (s != 0 && s != 1) return 0;
    if (s == 1) any1 = true;
  }
  if (!any1) return 0;
  if (c.rsize[c.nr - 1] < 128) return 0;
  ChainProg<float> chain;
  if (!to_chain<float>(j.pro, j.n_pro, chain)) return 0;
  const bool ident = chain.identity && c.n_in == 1;
  if (dt == PGB_F32) return c.n_in == 1 ? launch_row_typed<float, 1>(j, ident, chain) : launch_row_typed<float, 2>(j, ident, chain);
  return c.n_in == 1 ? launch_row_typed<__half, 1>(j, ident, chain) : launch_row_typed<__half, 2>(j, ident, chain);
}

}  // namespace pgb
