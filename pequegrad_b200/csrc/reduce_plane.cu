// Plane reduce: a SHORT reduced axis k next to the innermost kept axis j, where the (j, k) plane of every input is
// one contiguous block of memory but the inputs disagree on its orientation: [k][j] for one (j contiguous), [j][k]
// for another (k contiguous). The README fusion case of the reference is exactly this, x read through
// permute(0, 2, 1) against a plain y (README.md:59-63): no single thread mapping reads both operands coalesced, so
// the row and column kernels refuse it, and the generated kernel of the reference reads y with an 80-byte stride
// between threads (README.md:110-111).
//
// Here a CTA takes G whole planes of every input (all other kept dims are a batch), copies them to shared memory
// with coalesced 128-bit loads in memory order (the [j][k] orientation with an odd row pitch, so that the strided
// reads below hit distinct banks), and then thread (g, j) walks k: prologue chain, accumulate, epilogue, one
// coalesced store. Each input is read once, in full lines.
#include "reduce_common.cuh"
#include "vec.cuh"

namespace pgb {

namespace {

constexpr int kPlaneThreads = 256;
constexpr int kPlaneSmem = 48 * 1024;

template <int NIN>
struct PlaneParams {
  const float *in[NIN];
  int kj[NIN];             // 1: plane stored [k][j] (j contiguous); 0: stored [j][k] (k contiguous)
  int vec[NIN];            // planes can be fetched with 128-bit loads
  int64_t bstr[NIN][2];    // element strides of the two outer kept dims
  int64_t bsize1;          // extent of the inner one of them
  int64_t nplanes;
  int J, K, G, pitch;      // pitch: shared-memory row pitch of a [j][k] plane (odd)
  ChainProg<float> pro;
  EpiParams<float> epi;
};

template <int NIN, int ROP>
__global__ void __launch_bounds__(kPlaneThreads) reduce_plane_kernel(const __grid_constant__ PlaneParams<NIN> p) {
  extern __shared__ __align__(16) float sm[];
  const int J = p.J, K = p.K, G = p.G, JK = J * K;
  const int plane_words[2] = {J * p.pitch, JK};  // by orientation: [j][k] padded, [k][j] as in memory
  const int64_t plane0 = (int64_t)blockIdx.x * G;
  const int g_here = (int)min((int64_t)G, p.nplanes - plane0);
  float *base_sm[NIN];
  {
    float *cur = sm;
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
      base_sm[k] = cur;
      cur += (size_t)G * ((plane_words[p.kj[k]] + 3) & ~3);
    }
  }
  // stage the planes
#pragma unroll
  for (int k = 0; k < NIN; ++k) {
    const int pw = (plane_words[p.kj[k]] + 3) & ~3;
    for (int g = 0; g < g_here; ++g) {
      const int64_t pl = plane0 + g;
      const int64_t b1 = pl % p.bsize1, b0 = pl / p.bsize1;
      const float *src = p.in[k] + b0 * p.bstr[k][0] + b1 * p.bstr[k][1];
      float *dst = base_sm[k] + (size_t)g * pw;
      if (p.vec[k]) {
        for (int v = threadIdx.x; v < JK / 4; v += kPlaneThreads) {
          const float4 t = __ldg(reinterpret_cast<const float4 *>(src) + v);
          if (p.kj[k]) {
            reinterpret_cast<float4 *>(dst)[v] = t;
          } else {
            const float e[4] = {t.x, t.y, t.z, t.w};
            const int m = v * 4;
            int jj = m / K, kk = m - jj * K;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              dst[jj * p.pitch + kk] = e[i];
              if (++kk == K) { kk = 0; ++jj; }
            }
          }
        }
      } else {
        for (int m = threadIdx.x; m < JK; m += kPlaneThreads) {
          const float t = __ldg(src + m);
          if (p.kj[k]) dst[m] = t;
          else { const int jj = m / K; dst[jj * p.pitch + (m - jj * K)] = t; }
        }
      }
    }
  }
  __syncthreads();
  // thread -> (plane of the group, j); J > 256 loops over j
  const int per = G > 1 ? J : kPlaneThreads;
  for (int j0 = 0; j0 < J; j0 += per) {
    const int g = G > 1 ? (int)threadIdx.x / J : 0;
    const int j = G > 1 ? (int)threadIdx.x - g * J : j0 + (int)threadIdx.x;
    if (g >= g_here || j >= J) continue;
    Acc<float, ROP> acc;
    acc.init();
    const float *pl[NIN];
#pragma unroll
    for (int k = 0; k < NIN; ++k) pl[k] = base_sm[k] + (size_t)g * ((plane_words[p.kj[k]] + 3) & ~3);
    for (int k0 = 0; k0 < K; k0 += 4) {
      float w[NIN][4], run[4];
#pragma unroll
      for (int k = 0; k < NIN; ++k) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kk = min(k0 + e, K - 1);
          w[k][e] = p.kj[k] ? pl[k][kk * J + j] : pl[k][j * p.pitch + kk];
        }
      }
      chain_eval<float, NIN, 4>(p.pro, w, run);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (k0 + e < K) acc.add_stream(run[e], k0 + e);
    }
    finish_output<float>(p.epi, (plane0 + g) * J + j, acc.v, acc.i);
  }
}

template <int NIN>
int launch_plane(ReduceJob &j, const ChainProg<float> &chain) {
  const CanonReduce &c = j.c;
  PlaneParams<NIN> p{};
  const int jd = c.nk - 1;
  const int64_t J = c.ksize[jd], K = c.rsize[0];
  p.J = (int)J;
  p.K = (int)K;
  p.pitch = (int)(K | 1);
  size_t per_group = 0;
  bool mixed = false;
  for (int k = 0; k < NIN; ++k) {
    const int64_t sj = c.kin[k][jd], sk = c.rin[k][0];
    if (sj == 1 && sk == J) p.kj[k] = 1;
    else if (sj == K && sk == 1) p.kj[k] = 0;
    else return 0;
    if (p.kj[k] != p.kj[0]) mixed = true;
    p.in[k] = (const float *)j.in[k].data;
    bool vec = (J * K) % 4 == 0 && (reinterpret_cast<uintptr_t>(p.in[k]) & 15) == 0;
    for (int q = 0; q < 2; ++q) {
      const int d = jd - 2 + q;
      p.bstr[k][q] = d >= 0 ? c.kin[k][d] : 0;
      if (d >= 0 && c.kin[k][d] % 4) vec = false;
    }
    p.vec[k] = vec ? 1 : 0;
    per_group += (size_t)(((p.kj[k] ? J * K : J * p.pitch) + 3) & ~3) * sizeof(float);
  }
  // one orientation for all inputs is the row or the column kernel's case
  if (!mixed) return 0;
  p.bsize1 = jd >= 1 ? c.ksize[jd - 1] : 1;
  p.nplanes = c.n_out / J;
  int G = J >= kPlaneThreads ? 1 : (int)(kPlaneThreads / J);
  while (G > 1 && per_group * G > (size_t)kPlaneSmem) --G;
  if (per_group * G > (size_t)kPlaneSmem) return 0;
  p.G = G;
  const int64_t grid = (p.nplanes + G - 1) / G;
  if (grid > 2147483647LL) return 0;
  char buf[160];
  snprintf(buf, sizeof buf, "plane nin=%d J=%lld K=%lld planes=%lld per_cta=%d grid=%lld", NIN, (long long)J, (long long)K, (long long)p.nplanes, G,
           (long long)grid);
  j.desc = buf;
  j.ws_needed = 0;
  if (j.dry_run) return 1;
  p.pro = chain;
  std::string err = make_epi<float>(j, p.epi);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  const size_t smem = per_group * G;
  if (j.rop == ROP_SUM) reduce_plane_kernel<NIN, ROP_SUM><<<(unsigned)grid, kPlaneThreads, smem, j.stream>>>(p);
  else if (j.rop == ROP_MAX) reduce_plane_kernel<NIN, ROP_MAX><<<(unsigned)grid, kPlaneThreads, smem, j.stream>>>(p);
  else reduce_plane_kernel<NIN, ROP_ARGMAX><<<(unsigned)grid, kPlaneThreads, smem, j.stream>>>(p);
  count_launch();
  const int st = check_launch("reduce_plane_kernel");
  return st == PGB_OK ? 1 : st;
}

}  // namespace

// 1 launched (or planned), 0 not this kernel's case, < 0 error.
int launch_reduce_plane(ReduceJob &j) {
  const CanonReduce &c = j.c;
  if (j.cdtype != PGB_F32 || c.n_in != 2 || c.nr != 1 || c.nk < 1 || c.nk > 3) return 0;
  for (int k = 0; k < c.n_in; ++k)
    if (j.in[k].dtype != PGB_F32) return 0;
  const int64_t J = c.ksize[c.nk - 1], K = c.rsize[0];
  if (K < 2 || K > 128 || J < 8 || J * K > 8192) return 0;
  ChainProg<float> chain;
  if (!to_chain<float>(j.pro, j.n_pro, chain)) return 0;
  return launch_plane<2>(j, chain);
}

}  // namespace pgb
