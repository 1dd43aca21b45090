// Generic reduce (any rank up to 8, any dtype mix, any program) and the
// second stage of split reductions.
//
// The generic kernel is the semantic twin of the reference's eager kernel
// (csrc/cuda/reduce.cuh:23-98): it walks kept and reduced dims with div/mod,
// but over the canonicalised (merged) dims, with 64-bit offsets (the
// reference indexes with int, csrc/cuda/reduce.cuh:52-67), and it evaluates
// the fused prologue per element. One thread or one warp per output.
#include <type_traits>

#include "reduce_common.cuh"

namespace pgb {

template <typename T, int ROP>
__global__ void __launch_bounds__(256) reduce_generic_kernel(const __grid_constant__ GenParams<T> p) {
  const int G = p.G;
  const int64_t gid = ((int64_t)blockIdx.x * 256 + threadIdx.x) / G;
  const int t = threadIdx.x % G;
  const bool active = gid < p.n_out;
  Acc<T, ROP> acc;
  acc.init();
  if (active) {
    int64_t base[kMaxIn];
    for (int k = 0; k < p.n_in; ++k) base[k] = 0;
    int64_t rem = gid;
    for (int d = p.nk - 1; d >= 0; --d) {
      const int64_t c = rem % p.ksize[d];
      rem /= p.ksize[d];
      for (int k = 0; k < p.n_in; ++k) base[k] += c * p.kin[k][d];
    }
    T v[kMaxInstr];
    for (int64_t i = t; i < p.n_red; i += G) {
      int64_t off[kMaxIn];
      for (int k = 0; k < p.n_in; ++k) off[k] = base[k];
      int64_t r = i;
      for (int d = p.nr - 1; d >= 0; --d) {
        const int64_t c = r % p.rsize[d];
        r /= p.rsize[d];
        for (int k = 0; k < p.n_in; ++k) off[k] += c * p.rin[k][d];
      }
      vm_eval<T>(p.pro, v, (T)0, [&](int k) { return load_as<T>(p.in[k], p.dt[k], off[k]); });
      acc.add(v[p.pro.n - 1], (int)i);
    }
  }
  if (G == 32) warp_combine<T, ROP>(acc);
  if (active && t == 0) finish_output<T>(p.epi, gid, acc.v, acc.i);
}

template <typename T, int ROP>
__global__ void __launch_bounds__(256) reduce_finish_kernel(const T *__restrict__ part_v, const int *__restrict__ part_i, int64_t S,
                                                            int64_t n_out, const __grid_constant__ EpiParams<T> epi) {
  const int64_t o = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (o >= n_out) return;
  Acc<T, ROP> a;
  a.init();
  for (int64_t s = 0; s < S; ++s) a.merge(part_v[s * n_out + o], ROP == ROP_ARGMAX ? part_i[s * n_out + o] : 0);
  finish_output<T>(epi, o, a.v, a.i);
}

template <typename T>
static int finish_typed(ReduceJob &j, const void *part_v, const int *part_i, int64_t S) {
  EpiParams<T> e;
  std::string err = make_epi<T>(j, e);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  const int64_t n_out = j.c.n_out;
  const unsigned grid = (unsigned)((n_out + 255) / 256);
  if (j.rop == ROP_SUM) reduce_finish_kernel<T, ROP_SUM><<<grid, 256, 0, j.stream>>>((const T *)part_v, part_i, S, n_out, e);
  else if (j.rop == ROP_MAX) reduce_finish_kernel<T, ROP_MAX><<<grid, 256, 0, j.stream>>>((const T *)part_v, part_i, S, n_out, e);
  else reduce_finish_kernel<T, ROP_ARGMAX><<<grid, 256, 0, j.stream>>>((const T *)part_v, part_i, S, n_out, e);
  count_launch();
  return check_launch("reduce_finish_kernel");
}

int launch_reduce_finish(ReduceJob &j, const void *part_v, const int *part_i, int64_t S) {
  if (j.cdtype == PGB_F32) return finish_typed<float>(j, part_v, part_i, S);
  if (j.cdtype == PGB_F64) return finish_typed<double>(j, part_v, part_i, S);
  return finish_typed<int>(j, part_v, part_i, S);
}

template <typename T>
static int generic_typed(ReduceJob &j) {
  const CanonReduce &c = j.c;
  GenParams<T> p{};
  p.n_in = c.n_in;
  p.nk = c.nk;
  p.nr = c.nr;
  p.n_out = c.n_out;
  p.n_red = c.n_red;
  for (int d = 0; d < c.nk; ++d) p.ksize[d] = c.ksize[d];
  for (int d = 0; d < c.nr; ++d) p.rsize[d] = c.rsize[d];
  for (int k = 0; k < c.n_in; ++k) {
    p.in[k] = j.in[k].data;
    p.dt[k] = j.in[k].dtype;
    for (int d = 0; d < c.nk; ++d) p.kin[k][d] = c.kin[k][d];
    for (int d = 0; d < c.nr; ++d) p.rin[k][d] = c.rin[k][d];
  }
  p.G = (c.n_red >= 128) ? 32 : 1;
  const int64_t threads = c.n_out * p.G;
  const int64_t grid = (threads + 255) / 256;
  if (grid > 2147483647LL) { set_error("fused_reduce: output too large for the generic kernel"); return PGB_ERR_UNSUPPORTED; }
  char buf[128];
  snprintf(buf, sizeof buf, "generic g=%d grid=%lld nk=%d nr=%d", p.G, (long long)grid, c.nk, c.nr);
  j.desc = buf;
  j.ws_needed = 0;
  if (j.dry_run) return 1;
  to_vm<T>(j.pro, j.n_pro, p.pro);
  std::string err = make_epi<T>(j, p.epi);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  if (j.rop == ROP_SUM) reduce_generic_kernel<T, ROP_SUM><<<(unsigned)grid, 256, 0, j.stream>>>(p);
  else if (j.rop == ROP_MAX) reduce_generic_kernel<T, ROP_MAX><<<(unsigned)grid, 256, 0, j.stream>>>(p);
  else reduce_generic_kernel<T, ROP_ARGMAX><<<(unsigned)grid, 256, 0, j.stream>>>(p);
  count_launch();
  const int st = check_launch("reduce_generic_kernel");
  return st == PGB_OK ? 1 : st;
}

int launch_reduce_generic(ReduceJob &j) {
  if (j.cdtype == PGB_F32) return generic_typed<float>(j);
  if (j.cdtype == PGB_F64) return generic_typed<double>(j);
  return generic_typed<int>(j);
}

}  // namespace pgb
