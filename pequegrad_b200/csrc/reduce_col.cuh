#pragma once
// Column reduce: a KEPT dim is the memory-contiguous one and the reduced dims
// are strided (axis 0 of a matrix, the middle axis of a 3-D tensor, permuted
// views of either). The reference handles these with the same one-block-per-
// output kernel, whose consecutive threads then read addresses a whole row
// apart (csrc/cuda/reduce.cuh:52-71).
//
// A CTA is 32 x 8 threads: x owns V consecutive columns (one 128-bit load),
// y strides over the reduced rows, kBatch/V rows in flight per thread. The 8
// partial rows are combined through shared memory and written with one
// coalesced store per column tile. When the contiguous kept dim is not the
// innermost dim of the OUTPUT (a permuted view), `jout` carries its output
// stride and the stores scatter; L2 merges them.
#include <type_traits>

#include "reduce_common.cuh"
#include "vec.cuh"

// Resident CTAs per SM asked of the compiler for the one-input fp32 kernels without a program to interpret (no
// prologue, or x * a + b). The kernel is bound by the loads it keeps in flight, so residency is worth more than
// registers: at six CTAs (40 registers, no spill in sum / max, 12 bytes in argmax) the 36-case sweep runs at
// 6573 GB/s, against 6022 at four CTAs (62 registers), 6382 at five and 6493 at eight (32 registers). The
// interpreting and 16-bit instantiations would spill and keep four.
#ifndef PGB_COL_MINB
#define PGB_COL_MINB 6
#endif
namespace pgb {

template <typename T, typename InT, int NIN, int ROP, int MODE, int V>
__global__ void __launch_bounds__(256, NIN == 1 ? (((MODE == 0 || MODE == 3) && sizeof(InT) == 4) ? PGB_COL_MINB : 4) : 2) reduce_col_kernel(const __grid_constant__ ColParams<T, NIN> p) {
  // MODE 0: no prologue; 1: short chain of cheap binary ops, decoded into registers, 16-element batches; 2: any chain, one small batch at a time
  constexpr int B = (MODE == 2) ? (V > 4 ? V : 4) : kBatch;
  constexpr int U = B / V;
  ChainRegs<T> cr;
  if (MODE == 1) chain_decode<T>(p.pro, cr);
  // MODE 3: the commonest prologue, x * a + b with two roundings, hard-wired
  const T aff_a = p.pro.imm[0][1], aff_b = p.pro.imm[1][1];
  constexpr int TY = 8;
  constexpr int TILE = 32 * V;
  // 32-bit index arithmetic throughout (the host checks that the counts fit)
  const uint32_t x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const uint32_t ntiles = (uint32_t)p.ntiles, S = (uint32_t)p.S, bsize1 = (uint32_t)p.bsize1;
  uint32_t bid = blockIdx.x;
  uint32_t tile = bid, s = 0, batch = 0, b0 = 0, b1 = 0;
  if (ntiles != gridDim.x) {  // grid = tiles x splits x batch, tiles fastest
    tile = bid % ntiles;
    bid /= ntiles;
    batch = bid;
    if (S > 1) { s = bid % S; batch = bid / S; }
    b1 = batch;
    if (bsize1 != (uint32_t)p.nbatch) { b1 = batch % bsize1; b0 = batch / bsize1; }
  }
  const uint32_t J = (uint32_t)p.J;
  const uint32_t j = tile * TILE + x * V;
  const bool col_ok = j < J;

  Acc<T, ROP> acc[V];
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e].init();

  const uint32_t R = (uint32_t)p.R;
  const uint32_t r_lo = s * (uint32_t)p.rows_per_split;
  const uint32_t r_hi = min(R, r_lo + (uint32_t)p.rows_per_split);
  if (col_ok) {
    const InT *base[NIN];
#pragma unroll
    for (int k = 0; k < NIN; ++k)
      base[k] = (const InT *)p.in[k] + (int64_t)b0 * p.bstr[k][0] + (int64_t)b1 * p.bstr[k][1] + (int64_t)j * p.jstr[k];
    const bool one_rdim = p.R0 == 1;
    const uint32_t R1 = (uint32_t)p.R1;
    for (uint32_t rb = r_lo + y; rb < r_hi; rb += TY * U) {
      T w[NIN][B];
#pragma unroll
      for (int k = 0; k < NIN; ++k) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t r = rb + u * TY;
          T tmpv[V];
          if (r < r_hi) {
            int64_t off;
            if (one_rdim) off = (int64_t)r * p.rstr[k][1];
            else { const uint32_t r0 = r / R1; off = (int64_t)r0 * p.rstr[k][0] + (int64_t)(r - r0 * R1) * p.rstr[k][1]; }
            if (p.jstr[k] != 0) load_vec<T, InT, V>(base[k] + off, tmpv);
            else {
              const T b = to_compute<T, InT>(__ldg(base[k] + off));
#pragma unroll
              for (int e = 0; e < V; ++e) tmpv[e] = b;
            }
          } else {
#pragma unroll
            for (int e = 0; e < V; ++e) tmpv[e] = (T)0;
          }
#pragma unroll
          for (int e = 0; e < V; ++e) w[k][u * V + e] = tmpv[e];
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
        const uint32_t r = rb + u * TY;
        if (r < r_hi) {
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e].add_stream(run[u * V + e], (int)r);
        }
      }
    }
  }
  __shared__ T sv[TY][TILE];
  __shared__ int si[ROP == ROP_ARGMAX ? TY : 1][TILE];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    sv[y][x * V + e] = acc[e].v;
    if (ROP == ROP_ARGMAX) si[y][x * V + e] = acc[e].i;
  }
  __syncthreads();
  for (int col = threadIdx.x; col < TILE; col += 256) {
    const uint32_t jj = tile * TILE + col;
    if (jj >= J) break;
    Acc<T, ROP> a;
    a.init();
#pragma unroll
    for (int yy = 0; yy < TY; ++yy) a.merge(sv[yy][col], ROP == ROP_ARGMAX ? si[yy][col] : 0);
    const int64_t o = (int64_t)b0 * p.bout[0] + (int64_t)b1 * p.bout[1] + (int64_t)jj * p.jout;
    if (p.S == 1) finish_output<T>(p.epi, o, a.v, a.i);
    else {
      p.part_v[(int64_t)s * p.n_out + o] = a.v;
      if (ROP == ROP_ARGMAX) p.part_i[(int64_t)s * p.n_out + o] = a.i;
    }
  }
  if (p.S == 1 || p.tickets == nullptr) return;  // a finish kernel combines the partials
  // Split reduction without a second launch: every CTA of a column tile takes a ticket once its partials are
  // visible; whoever draws the last one combines the S partials of the tile, in split order (the same order, hence
  // the same bits, as the finish kernel). Nobody waits. atomicInc wraps the counter back to zero for the next launch.
  __shared__ bool is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicInc(p.tickets + (batch * ntiles + tile), S - 1) == S - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int col = threadIdx.x; col < TILE; col += 256) {
    const uint32_t jj = tile * TILE + col;
    if (jj >= J) break;
    const int64_t o = (int64_t)b0 * p.bout[0] + (int64_t)b1 * p.bout[1] + (int64_t)jj * p.jout;
    Acc<T, ROP> a;
    a.init();
    for (uint32_t ss = 0; ss < S; ++ss) a.merge(__ldcg(p.part_v + (int64_t)ss * p.n_out + o), ROP == ROP_ARGMAX ? __ldcg(p.part_i + (int64_t)ss * p.n_out + o) : 0);
    finish_output<T>(p.epi, o, a.v, a.i);
  }
}

// ---------------------------------------------------------------------------
template <typename InT, int NIN>
int launch_col_typed(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain) {
  using T = float;
  const CanonReduce &c = j.c;
  constexpr int VFULL = 16 / (int)sizeof(InT);
  ColParams<T, NIN> p{};
  // output strides of the kept dims (the output is contiguous in kept order)
  int64_t kout[PGB_MAX_DIMS];
  {
    int64_t acc = 1;
    for (int d = c.nk - 1; d >= 0; --d) { kout[d] = acc; acc *= c.ksize[d]; }
  }
  p.J = c.ksize[jd];
  p.jout = kout[jd];
  int bd[2] = {-1, -1};
  {
    int nb = 0;
    for (int d = 0; d < c.nk; ++d) if (d != jd) bd[nb++] = d;
    if (nb == 1) { bd[1] = bd[0]; bd[0] = -1; }  // right-align
  }
  int64_t bs[2] = {1, 1};
  for (int q = 0; q < 2; ++q) {
    if (bd[q] >= 0) { bs[q] = c.ksize[bd[q]]; p.bout[q] = kout[bd[q]]; }
    else p.bout[q] = 0;
  }
  p.bsize1 = bs[1];
  p.nbatch = bs[0] * bs[1];
  p.R0 = (c.nr == 2) ? c.rsize[0] : 1;
  p.R1 = (c.nr >= 1) ? c.rsize[c.nr - 1] : 1;
  p.R = p.R0 * p.R1;
  p.n_out = c.n_out;
  bool vec = (p.J % VFULL) == 0;
  for (int k = 0; k < NIN; ++k) {
    p.in[k] = j.in[k].data;
    p.jstr[k] = c.kin[k][jd];
    for (int q = 0; q < 2; ++q) p.bstr[k][q] = bd[q] >= 0 ? c.kin[k][bd[q]] : 0;
    p.rstr[k][0] = (c.nr == 2) ? c.rin[k][0] : 0;
    p.rstr[k][1] = (c.nr >= 1) ? c.rin[k][c.nr - 1] : 0;
    if (p.jstr[k] == 1) {
      if ((reinterpret_cast<uintptr_t>(p.in[k]) & 15) != 0) vec = false;
      for (int q = 0; q < 2; ++q) if (p.bstr[k][q] % VFULL) vec = false;
      for (int q = 0; q < 2; ++q) if (p.rstr[k][q] % VFULL) vec = false;
    }
  }
  const int V = vec ? VFULL : 1;
  p.ntiles = (p.J + 32 * V - 1) / (32 * V);
  const int64_t ctas = p.ntiles * p.nbatch;
  const int64_t want = (int64_t)sm_count() * 16;
  int64_t S = 1;
  if (ctas < want) {
    int64_t s_want = (want + ctas - 1) / ctas;
    const int64_t s_max = std::max<int64_t>(1, p.R / 64);
    // Very few column tiles (a tall matrix reduced over its rows: 8 to 64 tiles in the sweep and its shards): one wave
    // of about four CTAs per SM, each with a long run of rows, beats sixteen short ones, whose fixed costs (start-up,
    // shared-memory combine, partial store, ticket) are paid sixteen times per SM. Measured on [8192, 8192] /
    // [8192, 4096] / [8192, 1024], L2 flushed: 51.3 -> 50.2 us, 34.9 -> 30.8 us, 20.5 -> 17.5 us (argmax 55.4 -> 51.3,
    // 41.0 -> 32.8, 28.7 -> 20.5); one CTA more than a wave holds (14 x 64 = 896 > 888) costs 25 %.
    if (s_want >= 8) s_want = std::max<int64_t>(1, (int64_t)sm_count() * 4 / ctas);
    S = std::max<int64_t>(1, std::min(s_want, s_max));
  }
  p.rows_per_split = (p.R + S - 1) / S;
  S = (p.R + p.rows_per_split - 1) / p.rows_per_split;
  if (S < 1) S = 1;
  p.S = S;
  const int64_t grid = ctas * S;
  if (grid > 2147483647LL || p.R > 2147483647LL - 64 || p.J > 2147483647LL - 1024) return 0;
  const size_t ws = (S > 1) ? (size_t)(S * p.n_out) * (sizeof(T) + (j.rop == ROP_ARGMAX ? sizeof(int) : 0)) : 0;
  j.ws_needed = ws;
  char buf[256];
  snprintf(buf, sizeof buf, "col in=%s nin=%d %s vec=%d split=%lld grid=%lld J=%lld jout=%lld R=%lld batch=%lld", dtype_name(j.in[0].dtype),
           NIN, ident ? "ident" : (chain.affine && NIN == 1 ? "chain-affine" : (chain.lite ? "chain" : "chain-full")), V, (long long)S, (long long)grid, (long long)p.J, (long long)p.jout, (long long)p.R,
           (long long)p.nbatch);
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
  p.tickets = (S > 1) ? split_tickets(j.stream, ctas) : nullptr;
  std::string err = make_epi<T>(j, p.epi);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }

  auto go = [&](auto rop_c, auto ident_c, auto v_c) {
    constexpr int ROP = decltype(rop_c)::value;
    constexpr int MD = decltype(ident_c)::value;
    constexpr int VV = decltype(v_c)::value;
    reduce_col_kernel<T, InT, NIN, ROP, MD, VV><<<(unsigned)grid, 256, 0, j.stream>>>(p);
  };
  auto by_v = [&](auto rop_c, auto ident_c) {
    if (V == 1) go(rop_c, ident_c, std::integral_constant<int, 1>{});
    else go(rop_c, ident_c, std::integral_constant<int, VFULL>{});
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
  int st = check_launch("reduce_col_kernel");
  if (st == PGB_OK && S > 1 && !p.tickets) st = launch_reduce_finish(j, p.part_v, p.part_i, S);
  if (own_ws) cudaFreeAsync(ws_ptr, j.stream);
  return st == PGB_OK ? 1 : st;
}

}  // namespace pgb
