#pragma once
// Row reduce: the innermost reduced dim is contiguous in memory.
// Replaces the eager reduce kernel for this layout (one 64-thread block per
// output with a per-element div/mod walk, csrc/cuda/reduce.cuh:23-98) and the
// JIT reduce kernel's serial per-thread loop (csrc/compiler/ir.cpp:1527-1535).
//
// A group of G threads (one warp, or a whole 256-thread CTA) owns one work
// item = one output row, or one slice of it when rows are split across CTAs.
// Every thread keeps kBatch elements per input in flight as 128-bit loads,
// runs the prologue over the batch, and accumulates; groups combine with
// warp shuffles (+ shared memory across warps).
#include <cstdlib>
#include <type_traits>

#include "reduce_common.cuh"
#include "vec.cuh"

namespace pgb {

template <typename T, typename InT, int NIN, int ROP, int MODE, int V, int G>
__global__ void __launch_bounds__(256) reduce_row_kernel(const __grid_constant__ RowParams<T, NIN> p) {
  // MODE 0: no prologue; 1: short chain of cheap binary ops, decoded into registers, 16-element batches; 2: any chain, one small batch at a time
  constexpr int B = (MODE == 2) ? (V > 4 ? V : 4) : kBatch;
  constexpr int U = B / V;
  ChainRegs<T> cr;
  if (MODE == 1) chain_decode<T>(p.pro, cr);
  // MODE 3: the commonest prologue, x * a + b with two roundings, hard-wired
  const T aff_a = p.pro.imm[0][1], aff_b = p.pro.imm[1][1];
  constexpr int GPB = 256 / G;
  // All index arithmetic is 32-bit (the host checks that the counts fit):
  // 64-bit divisions cost hundreds of instructions per thread, which a thread
  // that only streams a few dozen elements cannot amortise.
  const uint32_t g = threadIdx.x / G, t = threadIdx.x % G;
  const uint32_t item = blockIdx.x * GPB + g;
  const uint32_t S = (uint32_t)p.S, n_out = (uint32_t)p.n_out;
  const bool active = item < n_out * S;

  Acc<T, ROP> acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i].init();

  uint32_t row = 0, s = 0;
  if (active) {
    if (S == 1) row = item;
    else { row = item / S; s = item - row * S; }
    uint32_t k0 = 0, k1 = 0, k2 = row;
    if (p.nk >= 2) {
      const uint32_t ks2 = (uint32_t)p.ksize2, ks1 = (uint32_t)p.ksize1;
      k2 = row % ks2;
      const uint32_t tmp = row / ks2;
      k1 = tmp;
      if (p.nk >= 3) { k1 = tmp % ks1; k0 = tmp / ks1; }
    }
    const InT *base[NIN];
#pragma unroll
    for (int k = 0; k < NIN; ++k)
      base[k] = (const InT *)p.in[k] + (int64_t)k0 * p.kstr[k][0] + (int64_t)k1 * p.kstr[k][1] + (int64_t)k2 * p.kstr[k][2];
    const uint32_t C = (uint32_t)p.C, chunk = (uint32_t)p.chunk, nchunks = (uint32_t)p.nchunks;
    const uint32_t nseg = (uint32_t)p.R1 * nchunks;
    uint32_t seg_lo = 0, seg_hi = nseg;
    if (S > 1) {
      seg_lo = (uint32_t)((uint64_t)s * nseg / S);
      seg_hi = (uint32_t)((uint64_t)(s + 1) * nseg / S);
    }
    for (uint32_t seg = seg_lo; seg < seg_hi; ++seg) {
      uint32_t r1 = seg, cc = 0;
      if (nchunks > 1) { r1 = seg / nchunks; cc = seg - r1 * nchunks; }
      const uint32_t c_lo = cc * chunk;
      const uint32_t c_end = min(C, c_lo + chunk);
      const InT *rowp[NIN];
#pragma unroll
      for (int k = 0; k < NIN; ++k) rowp[k] = base[k] + (int64_t)r1 * p.r1str[k];
      // rows whose length is no multiple of the vector width: whole vectors here, the last few elements below
      const uint32_t c_hi = (V > 1) ? c_end - (c_end % V) : c_end;  // c_lo is a multiple of V
      for (uint32_t c0 = c_lo + t * V; c0 < c_hi; c0 += G * V * U) {
        T w[NIN][B];
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
          if (p.cstr[k] != 0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint32_t c = c0 + u * G * V;
              T tmpv[V];
              if (c < c_hi) load_vec<T, InT, V>(rowp[k] + c, tmpv);
              else {
#pragma unroll
                for (int e = 0; e < V; ++e) tmpv[e] = (T)0;
              }
#pragma unroll
              for (int e = 0; e < V; ++e) w[k][u * V + e] = tmpv[e];
            }
          } else {
            const T b = to_compute<T, InT>(__ldg(rowp[k]));
#pragma unroll
            for (int e = 0; e < B; ++e) w[k][e] = b;
          }
        }
        T run[B];
        if (MODE == 0) {
#pragma unroll
          for (int e = 0; e < B; ++e) run[e] = w[0][e];
        } else if (MODE == 3) {
#pragma unroll
          for (int e = 0; e < B; ++e) run[e] = w[0][e] * aff_a + aff_b;
        } else if (MODE == 1) {
          chain_eval_fast<T, NIN, B>(cr, w, run);
        } else {
          chain_eval<T, NIN, B>(p.pro, w, run);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t c = c0 + u * G * V;
          if (c < c_hi) {
#pragma unroll
            for (int e = 0; e < V; ++e) acc[(u * V + e) & 3].add_stream(run[u * V + e], (int)(c + e));
          }
        }
      }
      if (V > 1 && c_hi + t < c_end) {  // the ragged end: one element per thread, through the same prologue
        const uint32_t c = c_hi + t;
        T w[NIN][B];
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
          const T b = to_compute<T, InT>(__ldg(rowp[k] + (p.cstr[k] != 0 ? c : 0u)));
#pragma unroll
          for (int e = 0; e < B; ++e) w[k][e] = b;
        }
        T run[B];
        if (MODE == 0) run[0] = w[0][0];
        else if (MODE == 3) run[0] = w[0][0] * aff_a + aff_b;
        else if (MODE == 1) chain_eval_fast<T, NIN, B>(cr, w, run);
        else chain_eval<T, NIN, B>(p.pro, w, run);
        acc[0].add_stream(run[0], (int)c);
      }
    }
  }
#pragma unroll
  for (int i = 1; i < 4; ++i) acc[0].merge(acc[i].v, acc[i].i);
  warp_combine<T, ROP>(acc[0]);
  if (G > 32) {
    constexpr int WPG = G / 32 > 0 ? G / 32 : 1;  // warps per group
    __shared__ T sv[8];
    __shared__ int si[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = acc[0].v; si[warp] = acc[0].i; }
    __syncthreads();
    if (warp % WPG == 0) {  // the first warp of each group combines the group's warps
      Acc<T, ROP> a;
      a.init();
      if (lane < WPG) { a.v = sv[warp + lane]; a.i = si[warp + lane]; }
      warp_combine<T, ROP>(a);
      acc[0] = a;
    }
  }
  if (active && t == 0) {
    if (p.S == 1) finish_output<T>(p.epi, row, acc[0].v, acc[0].i);
    else {
      p.part_v[(int64_t)s * p.n_out + row] = acc[0].v;
      if (ROP == ROP_ARGMAX) p.part_i[(int64_t)s * p.n_out + row] = acc[0].i;
    }
  }
}

// ---------------------------------------------------------------------------
template <typename InT, int NIN>
int launch_row_typed(ReduceJob &j, bool ident, const ChainProg<float> &chain) {
  using T = float;
  const CanonReduce &c = j.c;
  constexpr int VFULL = 16 / (int)sizeof(InT);
  RowParams<T, NIN> p{};
  const int ri = c.nr - 1;  // inner reduced dim
  p.C = c.rsize[ri];
  p.R1 = (c.nr == 2) ? c.rsize[0] : 1;
  p.n_out = c.n_out;
  bool vec = p.C >= VFULL;  // a ragged end is read element by element
  for (int k = 0; k < NIN; ++k) {
    p.in[k] = j.in[k].data;
    p.cstr[k] = c.rin[k][ri];
    p.r1str[k] = (c.nr == 2) ? c.rin[k][0] : 0;
    // right-align kept dims into 3 slots
    for (int d = 0; d < 3; ++d) p.kstr[k][d] = 0;
    for (int d = 0; d < c.nk; ++d) p.kstr[k][3 - c.nk + d] = c.kin[k][d];
    if (p.cstr[k] == 1) {
      if ((reinterpret_cast<uintptr_t>(p.in[k]) & 15) != 0) vec = false;
      for (int d = 0; d < 3; ++d) if (p.kstr[k][d] % VFULL) vec = false;
      if (p.r1str[k] % VFULL) vec = false;
    }
  }
  int64_t ks[3] = {1, 1, 1};
  for (int d = 0; d < c.nk; ++d) ks[3 - c.nk + d] = c.ksize[d];
  p.ksize1 = ks[1];
  p.ksize2 = ks[2];
  p.nk = c.nk;

  // work partition
  const int64_t per_row = p.R1 * p.C;
  // threads per row: a warp for short rows, half a CTA for medium ones (two rows per CTA
  // halve the per-row combine cost), a whole CTA beyond
  const int G = (per_row <= 2048) ? 32 : (per_row <= 16384 ? 128 : 256);
  const int V = vec ? VFULL : 1;
  int64_t S = 1;
  p.chunk = p.C;
  p.nchunks = 1;
  const int64_t want_items = (int64_t)sm_count() * 16;
  if (G == 256 && p.n_out < want_items / 4) {
    int64_t s_want = (want_items + p.n_out - 1) / p.n_out;
    int64_t s_max = per_row / 16384;
    S = std::max<int64_t>(1, std::min(s_want, s_max));
    if (S > 1) {
      int64_t nch = (S + p.R1 - 1) / p.R1;
      const int64_t gran = (int64_t)G * kBatch;
      int64_t chunk = (p.C + nch - 1) / nch;
      chunk = (chunk + gran - 1) / gran * gran;
      p.chunk = chunk;
      p.nchunks = (p.C + chunk - 1) / chunk;
      S = std::min(S, p.R1 * p.nchunks);
    }
  }
  p.S = S;
  const int64_t items = p.n_out * S;
  const int gpb = 256 / G;
  const int64_t grid = (items + gpb - 1) / gpb;
  if (grid > 2147483647LL || items > 2147483647LL || per_row > 2147483647LL || p.C + p.chunk > 2147483647LL) return 0;
  const size_t ws = (S > 1) ? (size_t)(S * p.n_out) * (sizeof(T) + (j.rop == ROP_ARGMAX ? sizeof(int) : 0)) : 0;
  j.ws_needed = ws;
  char buf[256];
  snprintf(buf, sizeof buf, "row in=%s nin=%d %s g=%d vec=%d split=%lld grid=%lld C=%lld R1=%lld", dtype_name(j.in[0].dtype), NIN,
           ident ? "ident" : (chain.affine && NIN == 1 ? "chain-affine" : (chain.lite ? "chain" : "chain-full")), G, V, (long long)S, (long long)grid, (long long)p.C, (long long)p.R1);
  j.desc = buf;
  if (j.dry_run) return 1;

  void *ws_ptr = nullptr;
  bool own_ws = false;
  if (ws) {
    if (j.workspace) {
      if (j.workspace_bytes < ws) { set_error("fused_reduce: workspace too small"); return PGB_ERR_WORKSPACE; }
      ws_ptr = j.workspace;
    } else if (j.no_alloc) {
      set_error("fused_reduce: this call may not allocate and was given no workspace for its partial results");
      return PGB_ERR_WORKSPACE;
    } else {
      if (cudaMallocAsync(&ws_ptr, ws, j.stream) != cudaSuccess) { set_error("fused_reduce: workspace allocation failed"); return PGB_ERR_CUDA; }
      own_ws = true;
    }
    p.part_v = (T *)ws_ptr;
    p.part_i = (int *)((char *)ws_ptr + (size_t)(S * p.n_out) * sizeof(T));
  }
  p.pro = chain;
  std::string err = make_epi<T>(j, p.epi);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }

  auto go = [&](auto rop_c, auto ident_c, auto v_c, auto g_c) {
    constexpr int ROP = decltype(rop_c)::value;
    constexpr int MD = decltype(ident_c)::value;
    constexpr int VV = decltype(v_c)::value;
    constexpr int GG = decltype(g_c)::value;
    reduce_row_kernel<T, InT, NIN, ROP, MD, VV, GG><<<(unsigned)grid, 256, 0, j.stream>>>(p);
  };
  auto by_g = [&](auto rop_c, auto ident_c, auto v_c) {
    if (G == 32) go(rop_c, ident_c, v_c, std::integral_constant<int, 32>{});
    else if (G == 128) go(rop_c, ident_c, v_c, std::integral_constant<int, 128>{});
    else go(rop_c, ident_c, v_c, std::integral_constant<int, 256>{});
  };
  auto by_v = [&](auto rop_c, auto ident_c) {
    if (V == 1) by_g(rop_c, ident_c, std::integral_constant<int, 1>{});
    else by_g(rop_c, ident_c, std::integral_constant<int, VFULL>{});
  };
  auto by_ident = [&](auto rop_c) {
    if constexpr (NIN == 1) {
      if (ident) { by_v(rop_c, std::integral_constant<int, 0>{}); return; }
      if (chain.affine) { by_v(rop_c, std::integral_constant<int, 3>{}); return; }
    }
    if (chain.lite) by_v(rop_c, std::integral_constant<int, 1>{});
    else by_v(rop_c, std::integral_constant<int, 2>{});
  };
  if (j.rop == ROP_SUM) by_ident(std::integral_constant<int, ROP_SUM>{});
  else if (j.rop == ROP_MAX) by_ident(std::integral_constant<int, ROP_MAX>{});
  else by_ident(std::integral_constant<int, ROP_ARGMAX>{});
  count_launch();
  int st = check_launch("reduce_row_kernel");
  if (st == PGB_OK && S > 1) st = launch_reduce_finish(j, p.part_v, p.part_i, S);
  if (own_ws) cudaFreeAsync(ws_ptr, j.stream);
  return st == PGB_OK ? 1 : st;
}

}  // namespace pgb
