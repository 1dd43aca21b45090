// Dispatcher of the col reduce family; the kernels are instantiated in reduce_col_*.cu
// (one translation unit per input type and input count, so they compile in parallel).
#include "reduce_col.cuh"

namespace pgb {

extern template int launch_col_typed<float, 1>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
extern template int launch_col_typed<float, 2>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
extern template int launch_col_typed<__half, 1>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
extern template int launch_col_typed<__half, 2>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);

int launch_reduce_col(ReduceJob &j) {
  const CanonReduce &c = j.c;
  if (j.cdtype != PGB_F32) return 0;
  if (c.n_in > 2 || c.nr > 2 || c.nk < 1 || c.nk > 3) return 0;
  if (j.rop == ROP_ARGMAX && c.nr > 1) return 0;
  const int dt = j.in[0].dtype;
  if (dt != PGB_F32 && dt != PGB_F16) return 0;
  for (int k = 0; k < c.n_in; ++k) if (j.in[k].dtype != dt) return 0;
  // the kept dim that is contiguous in memory for every non-broadcast input;
  // prefer the innermost output dim
  int jd = -1;
  for (int d = c.nk - 1; d >= 0 && jd < 0; --d) {
    bool ok = true, any1 = false;
    for (int k = 0; k < c.n_in; ++k) {
      const int64_t s = c.kin[k][d];
      if (s != 0 && s != 1) ok = false;
      if (s == 1) any1 = true;
    }
    if (ok && any1) jd = d;
  }
  if (jd < 0) return 0;
  if (c.ksize[jd] < 32) return 0;
  ChainProg<float> chain;
  if (!to_chain<float>(j.pro, j.n_pro, chain)) return 0;
  const bool ident = chain.identity && c.n_in == 1;
  if (dt == PGB_F32) return c.n_in == 1 ? launch_col_typed<float, 1>(j, jd, ident, chain) : launch_col_typed<float, 2>(j, jd, ident, chain);
  return c.n_in == 1 ? launch_col_typed<__half, 1>(j, jd, ident, chain) : launch_col_typed<__half, 2>(j, jd, ident, chain);
}

}  // namespace pgb
