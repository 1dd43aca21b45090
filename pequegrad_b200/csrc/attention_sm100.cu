// Fused scaled-dot-product attention (forward) for head dim 64 on the 5th-generation tensor cores.
//
// Replaces the composite of the reference's GPT-2 block (examples/gpt2.py:168-186): scores = q @ k^T / sqrt(d),
// additive causal mask, softmax (pequegrad/ops.py:259-267), att @ v, which runs as four kernel chains and
// materialises the [B, H, T, T] scores twice. Here the scores never leave the SM:
//   one CTA per (batch, head, block of 128 query rows); keys and values stream in blocks of 64
//   warp 0      TMA producer: Q once, then K and V blocks into two rings (128B swizzle, per-CTA loads only)
//   warp 1      allocates TMEM and issues tcgen05.mma (one thread):
//                 S = Q K^T    128 x 64 x 64, fp32 in TMEM
//                 O += P V     128 x 64 x 64, fp32 in TMEM; V is read as an MN-major operand, so it needs no transpose
//   warps 2-5   softmax: thread = query row. tcgen05.ld the row of S, mask, online max / sum with exp2 on the
//               SFU, rescale the row of O in TMEM when its max outgrew the exponent reference by 2^8, write P (16-bit) to shared memory in the
//               K-major 128B-swizzled operand layout for the PV MMA; at the end O / sum -> global
// Three CTAs fit per SM (65 KB of shared memory and 128 TMEM columns each), so one CTA's MMAs and loads run
// under the others' exponentials: the kernel is bound by its softmax warps, and three per scheduler hide the
// TMEM, barrier and SFU latencies of one another better than two did. Every wait is bounded; a timeout sets the device error word and the CTA drains.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "gemm_ptx.cuh"
#include "reduce_common.cuh"

namespace pgb {

constexpr int kQB = 128;  // query rows per CTA
constexpr int kKB = 64;   // keys per block
constexpr int kHD = 64;   // head dim
constexpr int kKStages = 2, kVStages = 2;
constexpr int kAttnThreads = 320;  // producer warp, MMA warp, eight softmax warps
constexpr int kQBytes = kQB * kHD * 2, kKVBytes = kKB * kHD * 2, kPBytes = kQB * kKB * 2;
constexpr int kAttnSmem = kQBytes + (kKStages + kVStages) * kKVBytes + kPBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + 2 * 2 * kQB * 4 /*half-row maxima, two phases*/;
constexpr int kAttnTmemCols = 128;  // S [0,64), O [64,128)
constexpr int kAttnCtasPerSm = 3;
constexpr float kLazyRescale = 8.0f;  // log2 of the largest p allowed before a row's exponent reference moves

struct AttnParams {
  int T, Tk, H, B, n_qblk;
  int causal;
  int is_half;  // 1 = f16, 0 = bf16
  float c;      // scale * log2(e)
  void *out;
  int64_t o_row, o_head, o_batch;  // output strides in elements
  int *err;
};

// f16 / bf16 instruction descriptor, M = 128, N = 64, fp32 accumulate; bit 16 = B operand is MN-major
__device__ __forceinline__ uint32_t attn_idesc(bool is_half, bool b_mn_major) {
  uint32_t d = 0;
  const uint32_t fmt = is_half ? 0u : 1u;
  d |= 1u << 4;
  d |= fmt << 7;
  d |= fmt << 10;
  if (b_mn_major) d |= 1u << 16;
  d |= (uint32_t)(64 >> 3) << 17;
  d |= (uint32_t)(128 >> 4) << 24;
  return d;
}

__device__ __forceinline__ float ex2f(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t ua, ub, uc, ud;
  memcpy(&ua, &a, 8); memcpy(&ub, &b, 8); memcpy(&uc, &c, 8);
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(ud) : "l"(ua), "l"(ub), "l"(uc));
  float2 d;
  memcpy(&d, &ud, 8);
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t ua, ub, ud;
  memcpy(&ua, &a, 8); memcpy(&ub, &b, 8);
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(ud) : "l"(ua), "l"(ub));
  float2 d;
  memcpy(&d, &ud, 8);
  return d;
}

__device__ __forceinline__ uint32_t pack_pair(float lo, float hi, bool is_h) {
  if (is_h) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
  const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&b);
}

// 64-thread named barrier of the two softmax warps that share TMEM lane quadrant `quad` (ids 1..4; 0 is __syncthreads)
__device__ __forceinline__ void pair_sync(int quad) {
  switch (quad) {
    case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
  }
}

__device__ __forceinline__ void attn_fail(const AttnParams &p, volatile int *abort_flag, int role) {
  *abort_flag = 1;
  atomicCAS(p.err, 0, ((8 + role) << 16) | (int)(blockIdx.x & 0xffff));
}

__global__ void __launch_bounds__(kAttnThreads, kAttnCtasPerSm) attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                        const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v,
                                                                        const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  uint8_t *q_s = smem;
  uint8_t *k_s = q_s + kQBytes;
  uint8_t *v_s = k_s + kKStages * kKVBytes;
  uint8_t *p_s = v_s + kVStages * kKVBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(p_s + kPBytes);
  uint64_t *q_full = bars;                   // [1]
  uint64_t *k_full = bars + 1;               // [kKStages]
  uint64_t *k_empty = k_full + kKStages;     // [kKStages]
  uint64_t *v_full = k_empty + kKStages;     // [kVStages]
  uint64_t *v_empty = v_full + kVStages;     // [kVStages]
  uint64_t *s_full = v_empty + kVStages;     // [1]  MMA -> softmax
  uint64_t *s_free = s_full + 1;             // [1]  softmax -> MMA (4 warps): S is in registers
  uint64_t *p_full = s_free + 1;             // [1]  softmax -> MMA (4 warps): P written, O rescaled
  uint64_t *pv_done = p_full + 1;            // [1]  MMA -> softmax: P and V consumed, O updated
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(pv_done + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  int *dead = const_cast<int *>(abort_flag) + 1;
  float *xch = reinterpret_cast<float *>(p_s + kPBytes + 256);  // [phase][column half][row]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy query blocks (those with the most keys under a causal mask) are scheduled first
  const int qb = p.n_qblk - 1 - (int)(blockIdx.x % p.n_qblk);
  const int bh = (int)(blockIdx.x / p.n_qblk);
  const int h = bh % p.H, b = bh / p.H;
  const int q0 = qb * kQB;
  int n_kb = (p.Tk + kKB - 1) / kKB;
  if (p.causal) n_kb = min(n_kb, (min(q0 + kQB, p.T) - 1) / kKB + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kKStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < kVStages; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(s_free, 8);
    mbar_init(p_full, 8);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    *dead = *(volatile int *)p.err != 0;  // an earlier launch failed and the host has not cleared the word: do nothing
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kAttnTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (*dead) {
    // one decision for the whole CTA (read by one thread before the barrier): the pair barriers below need every
    // softmax warp or none
  } else if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      mbar_expect_tx(q_full, kQBytes);
      tma_load_4d(q_s, &map_q, 0, q0, h, b, q_full);
      for (int j = 0; j < n_kb; ++j) {
        const int ks = j % kKStages, vs = j % kVStages;
        if (!mbar_wait(&k_empty[ks], ((j / kKStages) & 1) ^ 1, abort_flag)) { attn_fail(p, abort_flag, 1); break; }
        mbar_expect_tx(&k_full[ks], kKVBytes);
        tma_load_4d(k_s + ks * kKVBytes, &map_k, 0, j * kKB, h, b, &k_full[ks]);
        if (!mbar_wait(&v_empty[vs], ((j / kVStages) & 1) ^ 1, abort_flag)) { attn_fail(p, abort_flag, 2); break; }
        mbar_expect_tx(&v_full[vs], kKVBytes);
        tma_load_4d(v_s + vs * kKVBytes, &map_v, 0, j * kKB, h, b, &v_full[vs]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = attn_idesc(p.is_half != 0, false), idesc_pv = attn_idesc(p.is_half != 0, true);
      const uint64_t dq = make_kmajor_sw128_desc(smem_u32(q_s)), dp = make_kmajor_sw128_desc(smem_u32(p_s));
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (!ok) attn_fail(p, abort_flag, 3);
      // S(j) = Q K(j)^T; the single S buffer is free once the softmax warps hold S(j-1) in registers
      auto issue_s = [&](int j) -> bool {
        const int ks = j % kKStages;
        if (!mbar_wait(&k_full[ks], (j / kKStages) & 1, abort_flag)) { attn_fail(p, abort_flag, 4); return false; }
        if (!mbar_wait(s_free, (j & 1) ^ 1, abort_flag)) { attn_fail(p, abort_flag, 5); return false; }
        tc_fence_after();
        const uint64_t dk = make_kmajor_sw128_desc(smem_u32(k_s + ks * kKVBytes));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) tc_mma<GEMM_F16>(tmem_base, dq + 2 * kk, dk + 2 * kk, idesc_s, kk != 0);
        tc_commit(&k_empty[ks]);
        tc_commit(s_full);
        return true;
      };
      if (ok && n_kb > 0) ok = issue_s(0);
      for (int j = 0; j < n_kb && ok; ++j) {
        if (j + 1 < n_kb) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int vs = j % kVStages;
        if (!mbar_wait(p_full, j & 1, abort_flag)) { attn_fail(p, abort_flag, 6); break; }
        if (!mbar_wait(&v_full[vs], (j / kVStages) & 1, abort_flag)) { attn_fail(p, abort_flag, 7); break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(v_s + vs * kKVBytes);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // 16 keys per MMA: 32 bytes along P's rows, 16 rows of V
          tc_mma<GEMM_F16>(tmem_base + 64u, dp + 2 * kk, make_mnmajor_sw128_desc(v_addr + kk * 2048, 1024), idesc_pv, (j | kk) != 0);
        tc_commit(&v_empty[vs]);
        tc_commit(pv_done);
      }
    }
  } else {
    // Two warps share each TMEM lane quadrant (a warp reaches lanes 32 * (warp % 4) .. + 31): thread = (query row,
    // half of the block's 64 keys). The halves exchange their maxima through shared memory once per block (a
    // 64-thread named barrier per quadrant) so that both use the same exponent reference; the row sums stay
    // per half until the end. Eight softmax warps per CTA, three CTAs per SM: six warps per scheduler to hide
    // the TMEM, barrier and SFU latencies of one another.
    const int quad = warp & 3;              // TMEM lanes 32*quad .. +31
    const int ch = (warp - 2) >> 2;         // column half: keys [32*ch, 32*ch + 32) of the block, O columns likewise
    const int row = quad * 32 + lane, qrow = q0 + row;
    const bool is_h = p.is_half != 0;
    const float c = p.c;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + (uint32_t)(ch * 32), o_addr = lane_addr + 64u + (uint32_t)(ch * 32);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kb; ++j) {
      // A warp that gave up keeps meeting its partner at the pair barrier, once per block, so that neither is ever
      // left waiting there: every softmax warp passes exactly n_kb + 1 pair barriers, whatever happened.
      if (ok) {
        if (lane == 0) ok = mbar_wait(s_full, j & 1, abort_flag);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok && lane == 0) attn_fail(p, abort_flag, 8);
      }
      if (!ok) { pair_sync(quad); continue; }
      tc_fence_after();
      uint32_t sa[32];
      tmem_ld32_issue(s_addr, sa);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      float s[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(sa[i]);
      const int key0 = j * kKB + ch * 32;
      if ((p.causal && j * kKB + kKB - 1 > q0) || j * kKB + kKB > p.Tk) {  // block-uniform: only edge blocks pay for the mask
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = key0 + i;
          if ((p.causal && key > qrow) || key >= p.Tk) s[i] = -INFINITY;
        }
      }
      // three-input max, two independent chains
      float mq[2];
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        mq[g] = max3(s[16 * g], s[16 * g + 1], s[16 * g + 2]);
#pragma unroll
        for (int i = 3; i + 1 < 16; i += 2) mq[g] = max3(mq[g], s[16 * g + i], s[16 * g + i + 1]);
        mq[g] = fmaxf(mq[g], s[16 * g + 15]);
      }
      float mx = fmaxf(mq[0], mq[1]);
      float *xj = xch + (j & 1) * (2 * kQB);
      xj[ch * kQB + row] = mx;
      pair_sync(quad);
      mx = fmaxf(mx, xj[(ch ^ 1) * kQB + row]);
      // `m` is the reference point of the exponents, not the exact running max: it moves only when the row's max
      // outgrew it by more than kLazyRescale in the log2 domain (or on the row's first finite score). Until then
      // p <= 2^kLazyRescale, harmless in the fp32 sum, the fp32 accumulator and 16-bit P, and O / l is the same
      // quotient whatever the reference point; the rescale of O in tensor memory becomes a rare event.
      const float m_cand = fmaxf(m, mx);
      const bool grow = (m_cand - m) * c > kLazyRescale;  // -inf -> finite is +inf > threshold; -inf -> -inf is NaN: false
      const float m_new = grow ? m_cand : m;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row with no key yet: every p is 0
      const float alpha = grow ? ex2f((m - m_use) * c) : 1.0f;
      const float mc = m_use * c;
      // exponent arguments and the row sum on the packed fp32 pipe (two lanes of work per instruction)
      const float2 c2 = make_float2(c, c), nmc2 = make_float2(-mc, -mc);
      float2 sq[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 t = fma2(make_float2(s[i], s[i + 1]), c2, nmc2);
        const float2 pp = make_float2(ex2f(t.x), ex2f(t.y));
        sq[(i >> 1) & 3] = add2(sq[(i >> 1) & 3], pp);  // four independent partial sums
        pk[i >> 1] = pack_pair(pp.x, pp.y, is_h);
      }
      const float2 s01 = add2(sq[0], sq[1]), s23 = add2(sq[2], sq[3]);
      const float sum = (s01.x + s01.y) + (s23.x + s23.y);
      l = l * alpha + sum;
      m = m_new;
      if (j > 0) {
        // PV(j-1) must have consumed P and updated O before either is touched
        if (lane == 0) ok = mbar_wait(pv_done, (j - 1) & 1, abort_flag);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) { if (lane == 0) attn_fail(p, abort_flag, 9); continue; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
          // some row of this warp moved its reference: O_row *= 2^((m_old - m_new) c), this warp's 32 columns
          uint32_t o[32];
          tmem_ld32_issue(o_addr, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(o_addr, o);
          tmem_st_wait();
        }
      }
      // P half row -> shared memory, K-major with the 128B swizzle: 16-byte chunk i of row r sits at chunk i ^ (r & 7)
      uint8_t *prow = p_s + row * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4 *>(prow + (((ch * 4 + i) ^ (row & 7)) << 4)) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && n_kb > 0) {
      if (lane == 0) ok = mbar_wait(pv_done, (n_kb - 1) & 1, abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok && lane == 0) attn_fail(p, abort_flag, 10);
    }
    // the two halves of a row add their sums (both were kept against the same reference); failed or not, every
    // softmax warp comes here
    float *xl = xch + (n_kb & 1) * (2 * kQB);
    xl[ch * kQB + row] = l;
    pair_sync(quad);
    l += xl[(ch ^ 1) * kQB + row];
    if (ok) {
      tc_fence_after();
      const float inv = n_kb > 0 ? 1.0f / l : 0.f;
      uint8_t *orow = reinterpret_cast<uint8_t *>(p.out) + ((int64_t)b * p.o_batch + (int64_t)h * p.o_head + (int64_t)qrow * p.o_row) * 2;
      uint32_t o[32];
      if (n_kb > 0) {
        tmem_ld32_issue(o_addr, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
      if (qrow < p.T) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k)
            w[k] = pack_pair(__uint_as_float(o[8 * i + 2 * k]) * inv, __uint_as_float(o[8 * i + 2 * k + 1]) * inv, is_h);
          *reinterpret_cast<uint4 *>(orow + ch * 64 + i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kAttnTmemCols);
}

// ---- host side ---------------------------------------------------------------
// q, k, v, out: [B, H, T, 64] views with a contiguous head dim; *_str = strides in elements of the
// batch, head and row dims. Rows and all strides must be multiples of 8 elements (16 bytes).
int run_attention(const void *q, const void *k, const void *v, void *out, int is_half, int64_t B, int64_t H, int64_t T, int64_t Tk,
                  const int64_t q_str[3], const int64_t k_str[3], const int64_t v_str[3], const int64_t o_str[3], float scale, int causal,
                  cudaStream_t stream) {
  if (B <= 0 || H <= 0 || T <= 0) return PGB_OK;
  if (!(scale > 0.f) || !std::isfinite(scale)) { set_error("attention: the scale must be positive and finite"); return PGB_ERR_INVALID_ARG; }
  const int64_t n_qblk = (T + kQB - 1) / kQB;
  if (T > 2147483647LL / 2 || Tk > 2147483647LL / 2 || B * H * n_qblk > 2147483647LL) {
    set_error("attention: problem too large for one launch");
    return PGB_ERR_UNSUPPORTED;
  }
  const void *ptrs[4] = {q, k, v, out};
  const int64_t *strs[4] = {q_str, k_str, v_str, o_str};
  for (int i = 0; i < 4; ++i) {
    if ((reinterpret_cast<uintptr_t>(ptrs[i]) & 15) || strs[i][0] % 8 || strs[i][1] % 8 || strs[i][2] % 8 || strs[i][2] < kHD) {
      set_error("attention: q, k, v and out must be 16-byte aligned with row, head and batch pitches that are multiples of 16 bytes");
      return PGB_ERR_UNSUPPORTED;
    }
  }
  const CUtensorMapDataType dt = is_half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap mq, mk, mv;
  auto encode = [&](CUtensorMap *m, const void *ptr, const int64_t str[3], int64_t rows, uint32_t box_rows) {
    // a dim of extent 1 still needs a valid stride
    const uint64_t dims[4] = {(uint64_t)kHD, (uint64_t)rows, (uint64_t)H, (uint64_t)B};
    const uint64_t row_b = (uint64_t)str[2] * 2;
    const uint64_t head_b = H > 1 ? (uint64_t)str[1] * 2 : row_b * (uint64_t)rows;
    const uint64_t batch_b = B > 1 ? (uint64_t)str[0] * 2 : head_b * (uint64_t)H;
    const uint64_t strides[3] = {row_b, head_b, batch_b};
    const uint32_t box[4] = {(uint32_t)kHD, box_rows, 1, 1};
    return encode_map_4d(m, dt, ptr, dims, strides, box);
  };
  if (!encode(&mq, q, q_str, T, kQB) || !encode(&mk, k, k_str, Tk, kKB) || !encode(&mv, v, v_str, Tk, kKB)) {
    set_error("attention: cuTensorMapEncodeTiled failed");
    return PGB_ERR_CUDA;
  }
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] { attr_err = cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem); });
  if (attr_err != cudaSuccess) {
    set_error(std::string("attention: cannot raise the shared-memory limit: ") + cudaGetErrorString(attr_err));
    return PGB_ERR_CUDA;
  }
  AttnParams p{};
  p.T = (int)T;
  p.Tk = (int)Tk;
  p.H = (int)H;
  p.B = (int)B;
  p.n_qblk = (int)n_qblk;
  p.causal = causal ? 1 : 0;
  p.is_half = is_half ? 1 : 0;
  p.c = scale * 1.4426950408889634f;
  p.out = out;
  p.o_batch = o_str[0];
  p.o_head = o_str[1];
  p.o_row = o_str[2];
  p.err = gemm_error_word();
  if (!p.err) { set_error("attention: cannot resolve the device error word"); return PGB_ERR_CUDA; }
  attention_fwd_kernel<<<(unsigned)(B * H * n_qblk), kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, p);
  count_launch();
  return check_launch("attention_fwd_kernel");
}

}  // namespace pgb
