// Epilogue role of the tcgen05 GEMM: one warp drains 32 TMEM lanes (32 rows of
// the tile) of each finished accumulator, applies the fused epilogue and stores.
// The epilogue's shape (activation, bias, residual) is a template parameter, chosen
// once per kernel, so the per-element code has no branches and no dead code in it.
// Latency is hidden in three places: the tile's column operands (dequant scale,
// bias) are fetched into shared memory BEFORE the warp waits for the accumulator;
// the TMEM load of chunk c+1 is in flight while chunk c is processed; and the
// accumulator itself is double-buffered against the MMA warp.
#pragma once
#include "gemm_epilogue_tma.cuh"
#include "gemm_kernel.cuh"

namespace pgb {

template <int KIND, int ACT, bool BIAS, bool RES>
struct EpiChunk {
  const GemmParams &p;
  uint32_t *stage;
  const float *stash;  // [0,256) scale, [256,512) bias of this tile's columns
  int lane, row0, row, n0, bz;
  bool out_vec, acc_vec, want_max;
  float &local_max;

  __device__ __forceinline__ void run(const uint32_t (&v)[32], int c0) const {
    const GemmEpilogue &e = p.epi;
    const bool full_chunk = n0 + c0 + 32 <= p.N;
    const int n_left = row < p.M ? min(32, p.N - n0 - c0) : 0;
    if (e.acc_out) {
      int32_t *dst = e.acc_out + (int64_t)row0 * e.ld_acc + n0 + c0;
      if (full_chunk && acc_vec) stage_and_store<32>(stage, v, (uint8_t *)dst, e.ld_acc * 4, row0, p.M, lane);
      else store_tail<4>(v, (uint8_t *)dst, e.ld_acc * 4, lane, n_left);
    }
    if (!e.out && !want_max) return;
    float res[RES ? 32 : 1];
    if (RES) {
      // the residual is this thread's own row segment: 32 consecutive elements
      const int64_t roff = (int64_t)(bz / p.nb1) * e.res_batch0 + (int64_t)(bz % p.nb1) * e.res_batch + (int64_t)row * e.res_ld + n0 + c0;
#pragma unroll
      for (int i = 0; i < 32; ++i) res[RES ? i : 0] = i < n_left ? load_as<float>(e.residual, e.res_dtype, roff + i) : 0.f;
    }
    const float alpha = e.alpha;
    uint32_t f[32];
    // column operands come from the warp's stash as 128-bit broadcast reads (every lane the same address)
    float sc[KIND == GEMM_I8 ? 32 : 1], bi[BIAS ? 32 : 1];
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      if (KIND == GEMM_I8) {
        const float4 s4 = *reinterpret_cast<const float4 *>(stash + c0 + i);
        sc[KIND == GEMM_I8 ? i : 0] = s4.x; sc[KIND == GEMM_I8 ? i + 1 : 0] = s4.y;
        sc[KIND == GEMM_I8 ? i + 2 : 0] = s4.z; sc[KIND == GEMM_I8 ? i + 3 : 0] = s4.w;
      }
      if (BIAS) {
        const float4 b4 = *reinterpret_cast<const float4 *>(stash + 256 + c0 + i);
        bi[BIAS ? i : 0] = b4.x; bi[BIAS ? i + 1 : 0] = b4.y; bi[BIAS ? i + 2 : 0] = b4.z; bi[BIAS ? i + 3 : 0] = b4.w;
      }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float x;
      if (KIND == GEMM_I8) x = __fmul_rn((float)(int)v[i], sc[KIND == GEMM_I8 ? i : 0]);
      else x = __uint_as_float(v[i]) * alpha;
      if (BIAS) x = __fadd_rn(x, bi[BIAS ? i : 0]);
      if (ACT == ACT_RELU) x = x > 0.f ? x : 0.f;
      if (ACT == ACT_GELU_TANH) x = gelu_tanh(x);
      if (RES) x = __fadd_rn(x, res[RES ? i : 0]);
      f[i] = __float_as_uint(x);
    }
    if (want_max) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < n_left) local_max = fmaxf(local_max, fabsf(__uint_as_float(f[i])));
    }
    if (!e.out) return;
    const int64_t off0 = (int64_t)(bz / p.nb1) * e.out_batch0 + (int64_t)(bz % p.nb1) * e.out_batch + (int64_t)row0 * e.ldc + n0 + c0;
    if (e.out_dtype == PGB_F32) {
      float *dst = (float *)e.out + off0;
      if (full_chunk && out_vec) stage_and_store<32>(stage, f, (uint8_t *)dst, e.ldc * 4, row0, p.M, lane);
      else store_tail<4>(f, (uint8_t *)dst, e.ldc * 4, lane, n_left);
    } else {
      const bool is_h = e.out_dtype == PGB_F16;
      uint32_t h[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float lo = __uint_as_float(f[2 * i]), hi = __uint_as_float(f[2 * i + 1]);
        const uint16_t l16 = is_h ? __half_as_ushort(__float2half_rn(lo)) : __bfloat16_as_ushort(__float2bfloat16_rn(lo));
        const uint16_t h16 = is_h ? __half_as_ushort(__float2half_rn(hi)) : __bfloat16_as_ushort(__float2bfloat16_rn(hi));
        h[i] = (uint32_t)l16 | ((uint32_t)h16 << 16);
      }
#pragma unroll
      for (int i = 16; i < 32; ++i) h[i] = 0;
      uint16_t *dst = (uint16_t *)e.out + off0;
      if (full_chunk && out_vec) stage_and_store<16>(stage, h, (uint8_t *)dst, e.ldc * 2, row0, p.M, lane);
      else store_tail<2>(h, (uint8_t *)dst, e.ldc * 2, lane, n_left);
    }
  }
};

template <int KIND, int BN, int ACT, bool BIAS, bool RES>
__device__ __noinline__ void gemm_epilogue_tiles(const GemmParams &p, uint32_t tmem_base, uint32_t *stage, float *stash, int half, uint64_t *acc_full,
                                                 uint64_t *acc_empty, volatile int *abort_flag, int q, int lane, int num_tiles,
                                                 int tiles_per_batch) {
  const GemmEpilogue &e = p.epi;
  float a_scale = e.a_scale;
  if (KIND == GEMM_I8 && e.a_scale_dev) {
    // activation scale from the running absmax: max(amax, 1e-6) / 127, same fp32 ops as the host formula
    a_scale = fmaxf(__ldg(e.a_scale_dev), 1e-6f) / 127.0f;
  }
  float local_max = 0.f;
  const int out_es = e.out_dtype == PGB_F32 ? 4 : 2;
  // vector stores need 16-byte aligned rows
  const bool out_vec = e.out && ((reinterpret_cast<uintptr_t>(e.out) & 15) == 0) && ((e.ldc * out_es) % 16 == 0) &&
                       ((e.out_batch * out_es) % 16 == 0) && ((e.out_batch0 * out_es) % 16 == 0);
  const bool acc_vec = e.acc_out && ((reinterpret_cast<uintptr_t>(e.acc_out) & 15) == 0) && ((e.ld_acc & 3) == 0);
  const bool want_max = e.absmax != nullptr;
  int it = 0;
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
    const int bz = tile / tiles_per_batch, rem = tile - bz * tiles_per_batch;
    const int m0 = (rem / p.tiles_n) * kBM, n0 = (rem % p.tiles_n) * BN;
    const int buf = it & 1;
    // column operands of this tile, fetched while the MMAs are still running
    __syncwarp();
    constexpr int HALF = BN >= 64 ? BN / 2 : BN;  // columns per epilogue warp of a lane group
    const int cbeg = half * HALF, cend = min(cbeg + HALF, BN);
    for (int c = cbeg + lane; c < cend; c += 32) {
      const int col = n0 + c;
      const bool okc = col < p.N;
      if (KIND == GEMM_I8) stash[c] = e.col_scale ? __fmul_rn(a_scale, okc ? __ldg(e.col_scale + col) : 0.f) : a_scale;
      if (BIAS) stash[256 + c] = (okc && e.bias) ? load_as<float>(e.bias, e.bias_dtype, col) : 0.f;
    }
    __syncwarp();
    bool ok = true;
    if (lane == 0) ok = mbar_wait(&acc_full[buf], (it >> 1) & 1, abort_flag, p.spin_limit);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) {
      if (lane == 0) report_error(p, abort_flag, 3);
      break;
    }
    tc_fence_after();
    const int row0 = m0 + q * 32;
    EpiChunk<KIND, ACT, BIAS, RES> chunk{p, stage, stash, lane, row0, row0 + lane, n0, bz, out_vec, acc_vec, want_max, local_max};
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
    const int lim = min(cend, p.N - n0);  // end of this warp's columns that exist (warp-uniform)
    uint32_t va[32], vb[32];
    if (cbeg < lim) tmem_ld32_issue(taddr + cbeg, va);
    for (int c0 = cbeg; c0 < lim; c0 += 64) {
      tmem_ld_wait();
      if (c0 + 32 < lim) tmem_ld32_issue(taddr + c0 + 32, vb);
      chunk.run(va, c0);
      if (c0 + 32 < lim) {
        tmem_ld_wait();
        if (c0 + 64 < lim) tmem_ld32_issue(taddr + c0 + 64, va);
        chunk.run(vb, c0 + 32);
      }
    }
    // this warp is done reading the accumulator: hand the buffer back to the MMA warp
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&acc_empty[buf]);
  }
  if (want_max) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, m));
    // non-negative floats order like their bit patterns
    if (lane == 0 && local_max > 0.f) atomicMax(reinterpret_cast<unsigned int *>(e.absmax), __float_as_uint(local_max));
  }
}

// Chooses the specialisation once per kernel. TMA_EPI kernels hold only the TMA-store epilogues (p.out_tma = the
// output's element size), the others only the plain-store one above.
// ew = epilogue warp 0..15: TMEM lane quadrant q = warp % 4, column group ew / 4.
template <int KIND, int BN, bool TMA_EPI>
__device__ __forceinline__ void gemm_epilogue_warp(const GemmParams &p, const CUtensorMap *omap, const CUtensorMap *rmap, uint32_t tmem_base,
                                                   uint8_t *stage_base, float *stash_base, uint64_t *res_bar, int ew, uint64_t *acc_full,
                                                   uint64_t *acc_empty, volatile int *abort_flag, int q, int lane, int num_tiles,
                                                   int tiles_per_batch) {
#define PGB_EPI_TMA(ACT, BIAS, RES, OES)                                                                                                \
  gemm_epilogue_tma<KIND, BN, ACT, BIAS, RES, OES>(p, omap, rmap, tmem_base, stage_base + ew * kStoreBoxBytes, stash_base, res_bar, ew >> 2, acc_full, \
                                                   acc_empty, abort_flag, q, lane, num_tiles, tiles_per_batch)
#define PGB_EPI(ACT, BIAS, RES)                                                                                           \
  do {                                                                                                                    \
    if constexpr (TMA_EPI) {                                                                                              \
      if constexpr (KIND != GEMM_I8) {                                                                                    \
        if (p.out_tma == 2) { PGB_EPI_TMA(ACT, BIAS, RES, 2); break; }                                                    \
      } else if constexpr (BN == 256) {                                                                                   \
        if (p.out_tma == 1) { PGB_EPI_TMA(ACT, BIAS, RES, 1); break; }                                                    \
      }                                                                                                                   \
      PGB_EPI_TMA(ACT, BIAS, RES, 4);                                                                                     \
    } else if (ew < kPlainWarps) {                                                                                        \
      gemm_epilogue_tiles<KIND, BN, ACT, BIAS, RES>(p, tmem_base, reinterpret_cast<uint32_t *>(stage_base + ew * kPlainStageBytes), \
                                                    stash_base + ew * 512, ew >> 2, acc_full, acc_empty, abort_flag, q, lane, num_tiles, \
                                                    tiles_per_batch);                                                     \
    } else {                                                                                                              \
      gemm_epilogue_idle(p, acc_full, acc_empty, abort_flag, lane, num_tiles);                                            \
    }                                                                                                                     \
  } while (0)
  const bool bias = p.epi.bias != nullptr, res = p.epi.residual != nullptr;
  const int act = p.epi.act;
  if (KIND == GEMM_I8) {
    if (act == ACT_RELU) { if (bias) PGB_EPI(ACT_RELU, true, false); else PGB_EPI(ACT_RELU, false, false); }
    else { if (bias) PGB_EPI(ACT_NONE, true, false); else PGB_EPI(ACT_NONE, false, false); }
  } else {
    if (act == ACT_GELU_TANH) { if (res) PGB_EPI(ACT_GELU_TANH, true, true); else PGB_EPI(ACT_GELU_TANH, true, false); }
    else if (act == ACT_RELU) { if (res) PGB_EPI(ACT_RELU, true, true); else PGB_EPI(ACT_RELU, true, false); }
    else if (res) { PGB_EPI(ACT_NONE, true, true); }
    else if (bias) { PGB_EPI(ACT_NONE, true, false); }
    else { PGB_EPI(ACT_NONE, false, false); }
  }
#undef PGB_EPI
#undef PGB_EPI_TMA
}

}  // namespace pgb
