// Epilogue of the tcgen05 GEMM for outputs that TMA can store (16-byte aligned base and pitches):
// each epilogue warp drains 32 TMEM lanes (32 rows) of the finished accumulator 32 columns at a
// time, applies the fused epilogue in registers, writes its rows into a 32-row box in shared
// memory (swizzled, so the 16-byte writes of a warp hit 32 distinct banks) and one lane issues a
// TMA tile store of the box. The tensor map clips ragged bottom / right edges.
// Sixteen epilogue warps: four per TMEM lane quadrant, each with a quarter of the tile's columns, so
// that every scheduler has four warps to hide the TMEM-load, shared-memory and store latencies of
// one another (two warps per scheduler ran at a quarter of the issue rate). A box is 32 rows x 64
// bytes (64B swizzle): 16 fp32, 32 16-bit or 64 int8 columns, 2 KB per warp, which leaves room for a
// fourth stage in the operand ring. The tile's dequant scales and biases sit in shared memory once
// per CTA. The residual (laid out like the output) comes through the TMA unit into the same box.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_kernel.cuh"
#include "gemm_pair_ptx.cuh"

namespace pgb {

__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool is_h) {
  if (is_h) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
  const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&b);
}

// Barrier of the four warps (one per TMEM lane quadrant) that share a column group. Ids 1..4; id 0 is __syncthreads.
__device__ __forceinline__ void group_barrier(int group) { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }

template <int KIND, int BN, int ACT, bool BIAS, bool RES, int OES>
__device__ __noinline__ void gemm_epilogue_tma(const GemmParams &p, const CUtensorMap *omap, const CUtensorMap *rmap, uint32_t tmem_base,
                                               uint8_t *stage, float *stash, uint64_t *res_bar, int group, uint64_t *acc_full, uint64_t *acc_empty,
                                               volatile int *abort_flag, int q, int lane, int num_tiles, int tiles_per_batch) {
  constexpr int COLS = BN / kEpiGroups;  // columns per epilogue warp: 64 or 32
  const GemmEpilogue &e = p.epi;
  float a_scale = e.a_scale;
  if (KIND == GEMM_I8 && e.a_scale_dev) {
    // activation scale from the running absmax: max(amax, 1e-6) / 127, same fp32 ops as the host formula
    a_scale = fmaxf(__ldg(e.a_scale_dev), 1e-6f) / 127.0f;
  }
  float local_max = 0.f;
  const bool want_max = e.absmax != nullptr;
  const bool is_h = e.out_dtype == PGB_F16;
  const bool no_out = e.out == nullptr;
  const float alpha = e.alpha;
  float rq_s = 1.f, rq_r = 1.f, rq_thr = 0.f;
  if (OES == 1) {
    rq_s = fmaxf(__ldg(e.requant_absmax), 1e-6f) / 127.0f;
    rq_r = 1.0f / rq_s;
    rq_thr = 0.49999f * rq_s;
  }
  const int cbeg = group * COLS, cend = cbeg + COLS;
  // the tile's column operands, one copy per CTA: [0,256) dequant scale, [256,512) bias; this group owns [cbeg, cend)
  float *sc_stash = stash + cbeg, *bi_stash = stash + 256 + cbeg;
  // 64-byte box rows with the 64B swizzle: 16-byte piece j of row r sits at piece j ^ ((r >> 1) & 3)
  uint8_t *rowp = stage + lane * 64;
  const int sw = (lane >> 1) & 3;
  bool dead = false;  // a wait ran out: keep taking part in the group barriers, do nothing else
  uint32_t res_phase = 0;  // parity of this warp's residual barrier
  // CTAs per tile: one, or a pair that shares a 256-row tile (this CTA computes rows m_off .. m_off + 127 of it, and
  // hands its accumulator back on the barrier of the pair's leader, which issues the MMAs of both)
  const int psh = p.pair - 1;
  const int m_off = (int)(blockIdx.x & psh) * kBM;
  const uint32_t leader_empty = psh ? map_to_cta(smem_u32(acc_empty), 0) : 0u;
  auto release_acc = [&](int buf) {
    if (psh) mbar_arrive_cluster(leader_empty + 8u * (uint32_t)buf);
    else mbar_arrive(&acc_empty[buf]);
  };
  int it = 0;
  for (int tile = blockIdx.x >> psh; tile < num_tiles; tile += gridDim.x >> psh, ++it) {
    const int bz = tile / tiles_per_batch, rem = tile - bz * tiles_per_batch;
    const int m0 = (rem / p.tiles_n) * (kBM << psh) + m_off, n0 = (rem % p.tiles_n) * BN;
    const int zb = bz % p.nb1, wb = bz / p.nb1;
    const int buf = it & 1;
    // Column operands of this tile, fetched while the MMAs are still running. The four warps of the group each
    // fetch a quarter of the group's columns; the barriers keep a fast warp from overwriting what a slow one still reads.
    group_barrier(group);
    if (lane < COLS / 4) {
      const int c = q * (COLS / 4) + lane, col = n0 + cbeg + c;
      const bool okc = col < p.N;
      if (KIND == GEMM_I8) sc_stash[c] = e.col_scale ? __fmul_rn(a_scale, okc ? __ldg(e.col_scale + col) : 0.f) : a_scale;
      if (BIAS) bi_stash[c] = (okc && e.bias) ? load_as<float>(e.bias, e.bias_dtype, col) : 0.f;
    }
    group_barrier(group);
    if (dead) continue;
    const int row0 = m0 + q * 32, row = row0 + lane;
    const bool row_ok = row < p.M;
    const int lim = min(cend, p.N - n0);  // end of this warp's columns that exist (warp-uniform)
    if (RES && lane == 0 && row0 < p.M) {
      // this warp's share of the residual tile goes to L2 through the TMA unit while the MMAs still run
      for (int c = cbeg; c < lim; c += 64 / OES) tma_prefetch_4d(rmap, n0 + c, row0, zb, wb);
    }
    bool ok = true;
    if (lane == 0) ok = mbar_wait(&acc_full[buf], (it >> 1) & 1, abort_flag, p.spin_limit);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) {
      if (lane == 0) report_error(p, abort_flag, 3);
      dead = true;
      continue;
    }
    tc_fence_after();
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
    const bool store = !no_out && row0 < p.M;  // else only the absmax is wanted, or the whole warp is below the bottom edge
    bool released = false;
    for (int c0 = cbeg; c0 < lim; c0 += 32) {
      uint32_t v[32];
      // The residual box (same 32 rows x 64 bytes as the output box) is fetched by the TMA unit into the warp's box while
      // the accumulator chunk is loaded and processed. (Loading it with ordinary global loads cost ~0.4 us per MB of
      // residual whatever the access pattern: with nearly all of the SM's memory carved out as shared memory, the
      // load / store unit's miss path is a trickle.)
      auto res_request = [&](int col) {
        if (lane == 0) {
          tma_store_wait_read<0>();  // the previous store of this warp has read the box
          mbar_expect_tx(res_bar, kStoreBoxBytes);
          tma_load_4d(stage, rmap, col, row0, zb, wb, res_bar);
        }
      };
      auto res_arrived = [&]() -> bool {
        bool got = true;
        if (lane == 0) got = mbar_wait(res_bar, res_phase, abort_flag, p.spin_limit);
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        res_phase ^= 1u;
        return got;
      };
      if (RES && store) res_request(n0 + c0);
      tmem_ld32_issue(taddr + c0, v);
      tmem_ld_wait();
      if (c0 + 32 >= lim) {
        // every TMEM load of this tile has landed in registers: hand the buffer back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) release_acc(buf);
        released = true;
      }
      float x[32];
      const float *sc = sc_stash + (c0 - cbeg), *bi = bi_stash + (c0 - cbeg);
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f), b4 = s4;
        if (KIND == GEMM_I8) s4 = *reinterpret_cast<const float4 *>(sc + i);  // 128-bit broadcast reads
        if (BIAS) b4 = *reinterpret_cast<const float4 *>(bi + i);
        const float s[4] = {s4.x, s4.y, s4.z, s4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float t;
          if (KIND == GEMM_I8) t = __fmul_rn((float)(int)v[i + k], s[k]);
          else t = __uint_as_float(v[i + k]) * alpha;
          if (BIAS) t = __fadd_rn(t, b[k]);
          if (ACT == ACT_RELU) t = t > 0.f ? t : 0.f;
          if (ACT == ACT_GELU_TANH) t = gelu_tanh(t);
          x[i + k] = t;
        }
      }
      if (want_max && row_ok) {
#pragma unroll
        for (int i = 0; i < 32; ++i) local_max = fmaxf(local_max, fabsf(x[i]));
      }
      if (!store) continue;
      // a box may be refilled once the previous store of this warp has read it
      auto begin_box = [&]() {
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
      };
      auto end_box = [&](int col) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          tma_store_4d(omap, stage, col, row0, zb, wb);
          tma_store_commit();
        }
      };
      if (OES == 4) {
        // 32 fp32 columns = two boxes of 16
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          if (hb == 1 && n0 + c0 + 16 >= p.N) break;  // the second half lies beyond the right edge
          if (RES) {
            if (hb == 1) res_request(n0 + c0 + 16);
            if (!res_arrived()) { if (lane == 0) report_error(p, abort_flag, 5); dead = true; break; }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 rv = *reinterpret_cast<const uint4 *>(rowp + ((j ^ sw) << 4));
              x[hb * 16 + 4 * j] += __uint_as_float(rv.x); x[hb * 16 + 4 * j + 1] += __uint_as_float(rv.y);
              x[hb * 16 + 4 * j + 2] += __uint_as_float(rv.z); x[hb * 16 + 4 * j + 3] += __uint_as_float(rv.w);
            }
          } else {
            begin_box();
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4 *>(rowp + ((j ^ sw) << 4)) =
                make_uint4(__float_as_uint(x[hb * 16 + 4 * j]), __float_as_uint(x[hb * 16 + 4 * j + 1]), __float_as_uint(x[hb * 16 + 4 * j + 2]),
                           __float_as_uint(x[hb * 16 + 4 * j + 3]));
          end_box(n0 + c0 + hb * 16);
        }
        if (dead) break;
      } else if (OES == 2) {
        if (RES) {
          if (!res_arrived()) { if (lane == 0) report_error(p, abort_flag, 5); dead = true; break; }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 rv = *reinterpret_cast<const uint4 *>(rowp + ((j ^ sw) << 4));
            const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float2 f;
              if (is_h) f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
              else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[k]));
              x[8 * j + 2 * k] += f.x;
              x[8 * j + 2 * k + 1] += f.y;
            }
          }
        } else {
          begin_box();
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4 *>(rowp + ((j ^ sw) << 4)) =
              make_uint4(pack2(x[8 * j], x[8 * j + 1], is_h), pack2(x[8 * j + 2], x[8 * j + 3], is_h), pack2(x[8 * j + 4], x[8 * j + 5], is_h),
                         pack2(x[8 * j + 6], x[8 * j + 7], is_h));
        end_box(n0 + c0);
      } else {
        // int8 requantisation for the next layer (the exact rounding of v / s_next): two chunks fill a box
        const int sub = ((c0 - cbeg) >> 5) & 1;
        if (sub == 0) begin_box();
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          bool recheck = false;
          uint32_t w[4];
#pragma unroll
          for (int g = 0; g < 4; ++g)
            w[g] = quant_i8_fast4<ACT == ACT_RELU>(x[16 * j + 4 * g], x[16 * j + 4 * g + 1], x[16 * j + 4 * g + 2], x[16 * j + 4 * g + 3], rq_s, rq_r,
                                                   rq_thr, recheck);
          if (recheck) {  // some value sits next to a rounding boundary (about one in 60 000): the IEEE division decides
#pragma unroll
            for (int g = 0; g < 4; ++g)
              w[g] = quant_i8_pack4(x[16 * j + 4 * g], x[16 * j + 4 * g + 1], x[16 * j + 4 * g + 2], x[16 * j + 4 * g + 3], rq_s, rq_r);
          }
          *reinterpret_cast<uint4 *>(rowp + (((sub * 2 + j) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (sub == 1 || c0 + 32 >= lim) end_box(n0 + c0 - sub * 32);
      }
    }
    if (!released) {  // none of this warp's columns exist in this tile
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release_acc(buf);
    }
  }
  // shared memory must outlive the reads of the last stores
  if (lane == 0) tma_store_wait_all();
  if (want_max) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, m));
    // non-negative floats order like their bit patterns
    if (lane == 0 && local_max > 0.f) atomicMax(reinterpret_cast<unsigned int *>(e.absmax), __float_as_uint(local_max));
  }
}

// A warp with no share of the tile in the plain-store epilogue still takes part in the accumulator hand-over.
static __device__ __noinline__ void gemm_epilogue_idle(const GemmParams &p, uint64_t *acc_full, uint64_t *acc_empty, volatile int *abort_flag, int lane,
                                                int num_tiles) {
  int it = 0;
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
    const int buf = it & 1;
    bool ok = true;
    if (lane == 0) ok = mbar_wait(&acc_full[buf], (it >> 1) & 1, abort_flag, p.spin_limit);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) {
      if (lane == 0) report_error(p, abort_flag, 3);
      break;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&acc_empty[buf]);
  }
}

}  // namespace pgb
