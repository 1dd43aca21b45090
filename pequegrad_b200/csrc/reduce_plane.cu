// Short-axis reduce, one thread per output: a SHORT reduced axis k (at most 128 elements) over operands that disagree
// on which axis is contiguous. The README fusion case of the reference is exactly this: x read through
// permute(0, 2, 1), so that the innermost KEPT axis j is its contiguous one, against a plain y whose contiguous axis
// is k (README.md:59-63). No single thread mapping reads both with 128-byte requests, so the row and column kernels
// refuse it, and the generic kernel pays 64-bit div / mod and the interpreter per element.
//
// Here thread (plane, j) walks k with every address precomputed: 32-bit offsets, 8 or 16 k steps in flight, 128-bit
// loads for an operand whose k axis is contiguous, the prologue as a decoded chain.
// Consecutive threads read consecutive j of the j-contiguous operand (full requests) and neighbouring short rows of
// the k-contiguous one, whose sectors the L1 serves on the following steps; every byte is fetched from L2 once.
// A shared-memory staging of whole (j, k) planes was tried first and took 26 us on the README case, three times
// the reference's own generated kernel on the same GPU (8 us, thread per output like this one): the problem fits
// the L2, so the staging's barrier and serialised copy loop cost more than the uncoalesced requests they avoid.
#include <type_traits>

#include "reduce_common.cuh"
#include "vec.cuh"

namespace pgb {

namespace {

constexpr int kShortThreads = 256;

template <int NIN>
struct ShortParams {
  const float *in[NIN];
  int64_t bstr[NIN][2];  // element strides of the two outer kept dims
  int32_t jstr[NIN], kstr[NIN];
  int vec4[NIN];         // k contiguous and every row 16-byte aligned: four k steps per load
  int64_t bsize1;        // extent of the inner outer dim
  int64_t n_out;
  int J, K;
  ChainProg<float> pro;
  EpiParams<float> epi;
};

// B = reduced steps whose loads are all issued before the first is used: 16 for short axes with a cheap prologue
// (more would cost so many registers that the README case's 100 000 threads no longer fit the GPU in one wave), else 8.
template <int NIN, int ROP, bool LITE, int B>
__global__ void __launch_bounds__(kShortThreads, B > 8 ? 3 : 4) reduce_short_kernel(const __grid_constant__ ShortParams<NIN> p) {
  // 32-bit index arithmetic (the host checks that the output count fits): a 64-bit division costs more than the loop
  const uint32_t o = blockIdx.x * kShortThreads + threadIdx.x;
  if (o >= (uint32_t)p.n_out) return;
  const int J = p.J, K = p.K;
  const uint32_t plane = o / (uint32_t)J;
  const int j = (int)(o - plane * (uint32_t)J);
  const uint32_t bs1 = (uint32_t)p.bsize1;
  const uint32_t b0 = plane / bs1, b1 = plane - b0 * bs1;
  const float *base[NIN];
#pragma unroll
  for (int k = 0; k < NIN; ++k) base[k] = p.in[k] + (int64_t)b0 * p.bstr[k][0] + (int64_t)b1 * p.bstr[k][1] + (int64_t)j * p.jstr[k];
  ChainRegs<float> cr;
  if (LITE) chain_decode<float>(p.pro, cr);
  Acc<float, ROP> acc;
  acc.init();
  // whole chunks of B steps without any clamping, then the remainder four steps at a time (K = 20: 16 + 4 exactly)
  auto chunk = [&](auto cb_c, int k0) {
    constexpr int CB = decltype(cb_c)::value;
    float w[NIN][CB], run[CB];
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
      if (p.vec4[k]) {
#pragma unroll
        for (int v = 0; v < CB; v += 4) {
          // K % 4 == 0 here, so a vector never straddles the end of the row
          const float4 t = __ldg(reinterpret_cast<const float4 *>(base[k] + (k0 + v)));
          w[k][v] = t.x; w[k][v + 1] = t.y; w[k][v + 2] = t.z; w[k][v + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < CB; ++e) w[k][e] = __ldg(base[k] + (int64_t)min(k0 + e, K - 1) * p.kstr[k]);
      }
    }
    if (LITE) chain_eval_fast<float, NIN, CB>(cr, w, run);
    else chain_eval<float, NIN, CB>(p.pro, w, run);
#pragma unroll
    for (int e = 0; e < CB; ++e)
      if (k0 + e < K) acc.add_stream(run[e], k0 + e);
  };
  int k0 = 0;
#pragma unroll 1
  for (; k0 + B <= K; k0 += B) chunk(std::integral_constant<int, B>{}, k0);
#pragma unroll 1
  for (; k0 < K; k0 += 4) chunk(std::integral_constant<int, 4>{}, k0);
  finish_output<float>(p.epi, o, acc.v, acc.i);
}

template <int NIN>
int launch_short(ReduceJob &j, const ChainProg<float> &chain) {
  const CanonReduce &c = j.c;
  ShortParams<NIN> p{};
  const int jd = c.nk - 1;
  const int64_t J = c.ksize[jd], K = c.rsize[0];
  p.J = (int)J;
  p.K = (int)K;
  p.n_out = c.n_out;
  p.bsize1 = jd >= 1 ? c.ksize[jd - 1] : 1;
  for (int k = 0; k < NIN; ++k) {
    const int64_t sj = c.kin[k][jd], sk = c.rin[k][0];
    if (sj > 2147483647LL / 4 || sk > 2147483647LL / 256) return 0;
    p.in[k] = (const float *)j.in[k].data;
    p.jstr[k] = (int32_t)sj;
    p.kstr[k] = (int32_t)sk;
    bool v4 = sk == 1 && K % 4 == 0 && sj % 4 == 0 && (reinterpret_cast<uintptr_t>(p.in[k]) & 15) == 0;
    for (int q = 0; q < 2; ++q) {
      const int d = jd - 2 + q;
      p.bstr[k][q] = d >= 0 ? c.kin[k][d] : 0;
      if (d >= 0 && c.kin[k][d] % 4) v4 = false;
    }
    p.vec4[k] = v4 ? 1 : 0;
  }
  const int64_t grid = (c.n_out + kShortThreads - 1) / kShortThreads;
  if (c.n_out > 2147483647LL - kShortThreads) return 0;
  char buf[160];
  snprintf(buf, sizeof buf, "short nin=%d J=%lld K=%lld outputs=%lld grid=%lld %s", NIN, (long long)J, (long long)K, (long long)c.n_out, (long long)grid,
           chain.lite ? "chain" : "chain-full");
  j.desc = buf;
  j.ws_needed = 0;
  if (j.dry_run) return 1;
  p.pro = chain;
  std::string err = make_epi<float>(j, p.epi);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  auto go = [&](auto rop_c) {
    constexpr int ROP = decltype(rop_c)::value;
    // a short axis that is a multiple of four goes in one pass, every load of the row in flight at once (K = 20: as
    // many as the reference's fully unrolled generated kernel has)
    if (chain.lite && K == 20) reduce_short_kernel<NIN, ROP, true, 20><<<(unsigned)grid, kShortThreads, 0, j.stream>>>(p);
    else if (chain.lite && K == 24) reduce_short_kernel<NIN, ROP, true, 24><<<(unsigned)grid, kShortThreads, 0, j.stream>>>(p);
    else if (chain.lite && K == 12) reduce_short_kernel<NIN, ROP, true, 12><<<(unsigned)grid, kShortThreads, 0, j.stream>>>(p);
    else if (chain.lite && K <= 32) reduce_short_kernel<NIN, ROP, true, 16><<<(unsigned)grid, kShortThreads, 0, j.stream>>>(p);
    else if (chain.lite) reduce_short_kernel<NIN, ROP, true, 8><<<(unsigned)grid, kShortThreads, 0, j.stream>>>(p);
    else reduce_short_kernel<NIN, ROP, false, 8><<<(unsigned)grid, kShortThreads, 0, j.stream>>>(p);
  };
  if (j.rop == ROP_SUM) go(std::integral_constant<int, ROP_SUM>{});
  else if (j.rop == ROP_MAX) go(std::integral_constant<int, ROP_MAX>{});
  else go(std::integral_constant<int, ROP_ARGMAX>{});
  count_launch();
  const int st = check_launch("reduce_short_kernel");
  return st == PGB_OK ? 1 : st;
}

}  // namespace

// 1 launched (or planned), 0 not this kernel's case, < 0 error. Takes what the row and column kernels refused: two
// fp32 operands, one short reduced axis, a chain prologue, at most three kept dims; and only when one operand's
// innermost kept axis is its contiguous one (so that the requests of a warp are whole lines for at least that one).
int launch_reduce_plane(ReduceJob &j) {
  const CanonReduce &c = j.c;
  if (j.cdtype != PGB_F32 || c.n_in != 2 || c.nr != 1 || c.nk < 1 || c.nk > 3) return 0;
  bool any_j1 = false;
  for (int k = 0; k < c.n_in; ++k) {
    if (j.in[k].dtype != PGB_F32) return 0;
    if (c.kin[k][c.nk - 1] == 1) any_j1 = true;
  }
  const int64_t J = c.ksize[c.nk - 1], K = c.rsize[0];
  if (!any_j1 || K < 2 || K > 128 || J < 8) return 0;
  ChainProg<float> chain;
  if (!to_chain<float>(j.pro, j.n_pro, chain)) return 0;
  return launch_short<2>(j, chain);
}

}  // namespace pgb
