// Fused scaled-dot-product attention (forward) for head dim 64 on the 5th-generation tensor cores.
//
// Replaces the composite of the reference's GPT-2 block (examples/gpt2.py:168-186): scores = q @ k^T / sqrt(d),
// additive causal mask, softmax (pequegrad/ops.py:259-267), att @ v, which runs as four kernel chains and
// materialises the [B, H, T, T] scores twice. Here the scores never leave the SM.
//
// Work item = (batch, head, block of 128 query rows); keys and values stream in blocks of 128. The kernel is
// persistent: two CTAs per SM, each walking its share of the items (heaviest first under a causal mask), and
// every role keeps its own running block counter, so the loads and the MMAs of the next item start while the
// softmax of the current one is still running.
//   warps 0-3   softmax, one warp per TMEM lane quadrant: thread = query row, all 128 keys of the block.
//               tcgen05.ld the row of S, mask, max, exponent arguments in fp32 (packed f32x2 FMAs), exp2 on the
//               SFU for three pairs out of four and as a cubic on the FMA pipe for the fourth, row sum in
//               registers, then P as 16-bit pairs straight back into tensor memory (tcgen05.st): no shared-memory
//               round trip for P, no exchange between threads. The row of O is rescaled in tensor memory only when
//               its max outgrew the exponent reference by 2^8. An item's epilogue (O / l -> global) runs inside the
//               first block of the NEXT item, when the PV it needs has long finished.
//   warp 4      TMA producer: Q per item, K and V blocks through two-stage rings (128B swizzle, per-CTA loads only)
//   warp 5      allocates TMEM and issues tcgen05.mma (one thread):
//                 S = Q K^T    128 x 128 x 64, fp32 in TMEM, one block ahead of the softmax
//                 O += P V     128 x 64 x 128: P is the A operand read from tensor memory, V an MN-major
//                              shared-memory operand (no transpose)
// TMEM per CTA: S [0,128), P [128,192), O [192,256). What the earlier forms of this kernel taught: with P staged in
// shared memory the SM's shared-memory bandwidth was its busiest resource (MMA operand reads + P writes + TMA
// writes = 150 KB per 128 x 128 block); eight softmax warps splitting every row in halves spent a named barrier
// and an exchange per block and ran pairwise in lockstep on the same SFU; one CTA per item paid its pipeline fill
// and drain (about 8 us) ten times per SM. Every wait is bounded; a timeout sets the device error word and the
// CTA drains.
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

constexpr int kQB = 128;   // query rows per CTA
constexpr int kKB = 128;   // keys per block
constexpr int kHD = 64;    // head dim
constexpr int kKStages = 2, kVStages = 2;
constexpr int kAttnThreads = 192;  // four softmax warps, producer warp, MMA warp
constexpr int kQBytes = kQB * kHD * 2, kKVBytes = kKB * kHD * 2;
constexpr int kAttnSmem = kQBytes + (kKStages + kVStages) * kKVBytes + 256 /*barriers*/ + 1024 /*alignment slack*/;
constexpr int kAttnTmemCols = 256;  // S [0,128), P [128,192) (16-bit pairs), O [192,256)
constexpr uint32_t kColP = 128, kColO = 192;
constexpr int kAttnCtasPerSm = 2;
constexpr uint32_t kAttnPolls = 1u << 20;  // polls per wait before a role gives up
constexpr float kLazyRescale = 8.0f;  // log2 of the largest p allowed before a row's exponent reference moves

struct AttnParams {
  int T, Tk, H, B, n_qblk;
  int causal;
  float c;      // scale * log2(e)
  void *out;
  int64_t o_row, o_head, o_batch;  // output strides in elements
  int *err;
  uint32_t polls;   // polls per wait before a role gives up
  int skip_loads;   // failure-detection drill: the producer loads nothing
  int snake;        // item rounds alternate direction (see attn_item)
};

// f16 / bf16 instruction descriptor, M = 128, fp32 accumulate; bit 16 = B operand is MN-major
__device__ __forceinline__ uint32_t attn_idesc(bool is_half, bool b_mn_major, int n) {
  uint32_t d = 0;
  const uint32_t fmt = is_half ? 0u : 1u;
  d |= 1u << 4;
  d |= fmt << 7;
  d |= fmt << 10;
  if (b_mn_major) d |= 1u << 16;
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(128 >> 4) << 24;
  return d;
}

__device__ __forceinline__ float ex2f(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
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
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M = 128 rows = lanes, 16-bit elements two per column) is read from
// tensor memory
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 2^x for a pair of exponent arguments on the FMA pipe instead of the SFU: n = round(x) taken from the low mantissa
// bits of x + 1.5 * 2^23, f = x - n in [-0.5, 0.5], a cubic for 2^f (relative error 7.5e-5, a sixth of the rounding
// of a 16-bit P), and n added into the exponent field. x below -126 is clamped (the result is then 2^-126, nothing in P).
__device__ __forceinline__ float2 ex2_fma2(float2 x) {
  const float kMagic = 12582912.f;
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 r = add2(x, make_float2(kMagic, kMagic));
  const float2 n = add2(r, make_float2(-kMagic, -kMagic));
  const float2 f = add2(x, make_float2(-n.x, -n.y));
  float2 q = fma2(make_float2(0.05517144873738289f, 0.05517144873738289f), f, make_float2(0.2426108419895172f, 0.2426108419895172f));
  q = fma2(q, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
  q = fma2(q, f, make_float2(0.9999281167984009f, 0.9999281167984009f));
  return make_float2(__uint_as_float(__float_as_uint(q.x) + (__float_as_uint(r.x) << 23)), __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(r.y) << 23)));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <bool HALF>
__device__ __forceinline__ uint32_t out_pair(float lo, float hi) {
  uint32_t r;
  if (HALF) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
      "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
// Bounded wait. try_wait lets the hardware park the thread for a short while instead of spinning through the issue
// slots that the softmax warps need. (A suspend-time hint of 2 us was measured and is slower.)
__device__ __forceinline__ bool attn_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t polls) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < polls; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  return false;
}

// role: 0 Q buffer, 1 K ring, 2 V ring (producer); 3 Q, 4 K, 5 S buffer, 6 P, 7 V (MMA issuer); 8 S, 9 PV, 10 last PV
// (softmax). The error word carries 16 + role.
__device__ __forceinline__ void attn_fail(const AttnParams &p, volatile int *abort_flag, int role) {
  *abort_flag = 1;
  atomicCAS(p.err, 0, ((16 + role) << 16) | (int)(blockIdx.x & 0xffff));
}

struct AttnTile {
  int h, b, q0, n_kb;
};
// Work item `id` of the launch: query block and (batch, head). Heavy query blocks (those with the most keys under
// a causal mask) come first, so that the persistent CTAs, which take items gridDim.x apart, end together.
__device__ __forceinline__ AttnTile attn_tile(const AttnParams &p, int id) {
  const int bhn = p.B * p.H;
  const int qb = p.n_qblk - 1 - id / bhn, bh = id % bhn;
  AttnTile t;
  t.h = bh % p.H;
  t.b = bh / p.H;
  t.q0 = qb * kQB;
  t.n_kb = (p.Tk + kKB - 1) / kKB;
  if (p.causal) t.n_kb = min(t.n_kb, (min(t.q0 + kQB, p.T) - 1) / kKB + 1);
  return t;
}

// The item this CTA takes in round r. With few rounds (`snake`: at most three items per CTA) the rounds alternate
// direction over the CTAs, so that the CTAs that took the heaviest items first take the lightest next: 20.6 against
// 24.2 us for 4 x 12 heads of 1024 causal tokens. With many rounds the plain order is faster although it balances
// the key blocks per CTA worse (51 against 48 for 32 x 12 heads: 113 against 116 us).
__device__ __forceinline__ int attn_item(const AttnParams &p, int r) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  return r * G + ((p.snake && (r & 1)) ? G - 1 - c : c);
}

template <bool HALF>
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
  uint64_t *bars = reinterpret_cast<uint64_t *>(v_s + kVStages * kKVBytes);
  uint64_t *q_full = bars;                   // [1]
  uint64_t *q_empty = bars + 1;              // [1]  MMA -> producer: the item's last S was computed
  uint64_t *k_full = q_empty + 1;            // [kKStages]
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = p.B * p.H * p.n_qblk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < kKStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int st = 0; st < kVStages; ++st) { mbar_init(&v_full[st], 1); mbar_init(&v_empty[st], 1); }
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    *dead = *(volatile int *)p.err != 0;  // an earlier launch failed and the host has not cleared the word: do nothing
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) tmem_alloc(tmem_slot, kAttnTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Every role walks the same list of items (attn_item) and, inside an item, its key blocks, with its own running
  // block counter g: ring stages and barrier parities follow g, not the item, so the producer and the MMA thread run
  // ahead into the next item while the softmax warps still finish the current one (the next Q arrives under the last
  // block's softmax, and the next item's first S is ready when that softmax ends).
  if (*dead) {
    // an earlier kernel's wait ran out and nobody has cleared the word: nothing runs (one decision for the whole CTA)
  } else if (warp == 4) {
    if (lane == 0 && !p.skip_loads) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      uint32_t g = 0, it = 0;
      bool ok = true;
      for (int r = 0, id; (id = attn_item(p, r)) < n_items && ok; ++r) {
        const AttnTile t = attn_tile(p, id);
        if (t.n_kb == 0) continue;
        // the single Q buffer is free once the previous item's last S = Q K^T has been computed
        if (!attn_wait(q_empty, (it & 1) ^ 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 0); break; }
        mbar_expect_tx(q_full, kQBytes);
        tma_load_4d(q_s, &map_q, 0, t.q0, t.h, t.b, q_full);
        ++it;
        for (int j = 0; j < t.n_kb; ++j, ++g) {
          const uint32_t ks = g % kKStages;
          if (!attn_wait(&k_empty[ks], ((g / kKStages) & 1) ^ 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 1); ok = false; break; }
          mbar_expect_tx(&k_full[ks], kKVBytes);
          tma_load_4d(k_s + ks * kKVBytes, &map_k, 0, j * kKB, t.h, t.b, &k_full[ks]);
          const uint32_t vs = g % kVStages;
          if (!attn_wait(&v_empty[vs], ((g / kVStages) & 1) ^ 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 2); ok = false; break; }
          mbar_expect_tx(&v_full[vs], kKVBytes);
          tma_load_4d(v_s + vs * kKVBytes, &map_v, 0, j * kKB, t.h, t.b, &v_full[vs]);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc_s = attn_idesc(HALF, false, kKB), idesc_pv = attn_idesc(HALF, true, kHD);
      const uint64_t dq = make_kmajor_sw128_desc(smem_u32(q_s));
      // two cursors over the same block sequence: S runs one block ahead of PV, across item boundaries
      int s_r = 0, s_id = attn_item(p, 0), s_j = 0, s_n = 0;
      uint32_t s_g = 0, s_it = 0;
      auto s_seek = [&]() {  // moves the S cursor to the next item that has key blocks
        while (s_id < n_items) {
          s_n = attn_tile(p, s_id).n_kb;
          if (s_n > 0) return;
          s_id = attn_item(p, ++s_r);
        }
        s_n = 0;
      };
      s_seek();
      // S(g) = Q K(g)^T; the single S buffer is free once the softmax warps hold S(g-1) in registers
      auto issue_s = [&]() -> bool {
        if (s_j == 0 && !attn_wait(q_full, s_it & 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 3); return false; }
        const uint32_t ks = s_g % kKStages;
        if (!attn_wait(&k_full[ks], (s_g / kKStages) & 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 4); return false; }
        if (!attn_wait(s_free, (s_g & 1) ^ 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 5); return false; }
        tc_fence_after();
        const uint64_t dk = make_kmajor_sw128_desc(smem_u32(k_s + ks * kKVBytes));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) tc_mma<GEMM_F16>(tmem_base, dq + 2 * kk, dk + 2 * kk, idesc_s, kk != 0);
        tc_commit(&k_empty[ks]);
        tc_commit(s_full);
        ++s_g;
        if (++s_j == s_n) {  // the item's last S: Q may be replaced
          tc_commit(q_empty);
          ++s_it;
          s_j = 0;
          s_id = attn_item(p, ++s_r);
          s_seek();
        }
        return true;
      };
      bool ok = true;
      if (s_id < n_items) ok = issue_s();
      uint32_t g = 0;
      for (int r = 0, id; (id = attn_item(p, r)) < n_items && ok; ++r) {
        const int n_kb = attn_tile(p, id).n_kb;
        for (int j = 0; j < n_kb && ok; ++j, ++g) {
          // S runs one block ahead of PV, across item boundaries too: the softmax warps go straight from an item's
          // last block to the next item's first
          if (s_id < n_items) {
            ok = issue_s();
            if (!ok) break;
          }
          // P(g) arrives only after the softmax warps have read the previous item's O and row sums, so the first
          // PV of an item may overwrite them
          if (!attn_wait(p_full, g & 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 6); ok = false; break; }
          const uint32_t vs = g % kVStages;
          if (!attn_wait(&v_full[vs], (g / kVStages) & 1, abort_flag, p.polls)) { attn_fail(p, abort_flag, 7); ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)  // 16 keys per MMA: 8 columns of P (two keys each), 16 rows of V
            tc_mma_ts(tmem_base + kColO, tmem_base + kColP + kk * 8, make_mnmajor_sw128_desc(smem_u32(v_s + vs * kKVBytes) + kk * 2048, 1024), idesc_pv, (j | kk) != 0);
          tc_commit(&v_empty[vs]);
          tc_commit(pv_done);
        }
      }
    }
  } else {
    // One softmax warp per TMEM lane quadrant (a warp reaches lanes 32 * (warp % 4) .. + 31): thread = query row, all
    // 128 keys of the block. No exchange between threads anywhere: the row's max, exponent reference and sum live in
    // this thread's registers.
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const float c = p.c;
    const float2 c2 = make_float2(c, c);
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr, o_addr = lane_addr + kColO, p_addr = lane_addr + kColP;
    uint32_t g = 0;
    bool ok = true;
    // O / l -> global for this thread's row of item `oid`
    auto write_out = [&](int oid, float lsum) {
      const AttnTile ot = attn_tile(p, oid);
      const int orow_i = ot.q0 + row;
      uint8_t *orow = reinterpret_cast<uint8_t *>(p.out) + ((int64_t)ot.b * p.o_batch + (int64_t)ot.h * p.o_head + (int64_t)orow_i * p.o_row) * 2;
      const float inv = 1.0f / lsum;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {  // 16 columns at a time: few registers next to the block's scores
        uint32_t o[16];
        tmem_ld16_issue(o_addr + q4 * 16, o);
        tmem_ld_wait();
        if (orow_i < p.T) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              w[k] = out_pair<HALF>(__uint_as_float(o[8 * i + 2 * k]) * inv, __uint_as_float(o[8 * i + 2 * k + 1]) * inv);
            *reinterpret_cast<uint4 *>(orow + q4 * 32 + i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      tc_fence_before();
    };
    // The epilogue of an item is deferred into the first block of the next one: by the time that block's P is
    // ready, the previous item's last PV has long finished, so nobody waits for it; O is only overwritten by the
    // PV that this block's P releases.
    int prev_id = -1;
    float l_prev = 0.f;
    for (int r = 0, id; (id = attn_item(p, r)) < n_items; ++r) {
      const AttnTile t = attn_tile(p, id);
      const int qrow = t.q0 + row;
      if (t.n_kb == 0) {  // no keys at all (Tk == 0, so for every item): zeros
        if (qrow < p.T) {
          uint8_t *orow = reinterpret_cast<uint8_t *>(p.out) + ((int64_t)t.b * p.o_batch + (int64_t)t.h * p.o_head + (int64_t)qrow * p.o_row) * 2;
#pragma unroll
          for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4 *>(orow + i * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < t.n_kb; ++j, ++g) {
        if (ok) {
          // every lane polls (one broadcast read of the barrier per poll): no shuffle, no divergent branch
          ok = __all_sync(0xffffffffu, attn_wait(s_full, g & 1, abort_flag, p.polls));
          if (!ok && lane == 0) attn_fail(p, abort_flag, 8);
        }
        if (!ok) continue;
        tc_fence_after();
        uint32_t sa[4][32];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) tmem_ld32_issue(s_addr + q4 * 32, sa[q4]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
        float s[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) s[i] = __uint_as_float(sa[i >> 5][i & 31]);
        const int key0 = j * kKB;
        // warp-uniform: only blocks whose keys reach past one of this warp's rows' diagonal, or past the last key, mask
        if ((p.causal && key0 + kKB - 1 > t.q0 + quad * 32) || key0 + kKB > p.Tk) {
          int lim = p.Tk - 1 - key0;                     // last valid element of this thread's 128
          if (p.causal) lim = min(lim, qrow - key0);
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i > lim) s[i] = -INFINITY;
        }
        // three-input max, eight independent chains
        float mq[8];
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
          mq[q8] = max3(s[16 * q8], s[16 * q8 + 1], s[16 * q8 + 2]);
#pragma unroll
          for (int i = 3; i + 1 < 16; i += 2) mq[q8] = max3(mq[q8], s[16 * q8 + i], s[16 * q8 + i + 1]);
          mq[q8] = fmaxf(mq[q8], s[16 * q8 + 15]);
        }
        const float mx = fmaxf(max3(mq[0], mq[1], mq[2]), max3(max3(mq[3], mq[4], mq[5]), mq[6], mq[7]));
        // `m` is the reference point of the exponents, not the exact running max: it moves only when the row's max
        // outgrew it by more than kLazyRescale in the log2 domain (or on the row's first finite score). Until then
        // p <= 2^kLazyRescale, harmless in the fp32 accumulators and in 16-bit P, and O / l is the same quotient
        // whatever the reference point; the rescale of O in tensor memory becomes a rare event.
        const float m_cand = fmaxf(m, mx);
        const bool grow = (m_cand - m) * c > kLazyRescale;  // -inf -> finite is +inf > threshold; -inf -> -inf is NaN: false
        const float m_new = grow ? m_cand : m;
        const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row with no key yet: every p is 0
        const float alpha = grow ? ex2f((m - m_use) * c) : 1.0f;
        const float nmc = -m_use * c;
        const float2 nmc2 = make_float2(nmc, nmc);
        m = m_new;
        if (g > 0) {
          // PV(g-1) must have consumed P and updated O before either is touched (it was released a whole block ago)
          ok = __all_sync(0xffffffffu, attn_wait(pv_done, (g - 1) & 1, abort_flag, p.polls));
          if (!ok) { if (lane == 0) attn_fail(p, abort_flag, 9); continue; }
          tc_fence_after();
          if (j == 0 && prev_id >= 0) {
            write_out(prev_id, l_prev);
          } else if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
            // some row of this warp moved its reference: O_row *= 2^((m_old - m_new) c)
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint32_t o[16];
              tmem_ld16_issue(o_addr + q4 * 16, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st16(o_addr + q4 * 16, o);
            }
            tmem_st_wait();
          }
        }
        // P row -> tensor memory, two keys per 32-bit column (the A operand of the PV MMA), 64 keys at a time
        float2 sq[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            const float2 e = fma2(make_float2(s[64 * half + i], s[64 * half + i + 1]), c2, nmc2);
            // every fourth pair takes its exponentials on the FMA pipe: the SFU (16 results per clock per SM) is the
            // unit this kernel keeps busiest, and a quarter is what the spare issue slots pay for (a third measured slower)
            const float2 pp = ((i >> 1) & 3) == 3 ? ex2_fma2(e) : make_float2(ex2f(e.x), ex2f(e.y));
            sq[(i >> 1) & 3] = add2(sq[(i >> 1) & 3], pp);  // independent partial row sums
            pk[i >> 1] = out_pair<HALF>(pp.x, pp.y);
          }
          tmem_st32(p_addr + half * 32, pk);
        }
        {
          const float2 s01 = add2(sq[0], sq[1]), s23 = add2(sq[2], sq[3]);
          l = l * alpha + ((s01.x + s01.y) + (s23.x + s23.y));
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
      prev_id = id;
      l_prev = l;
    }
    if (prev_id >= 0 && ok) {  // the last item's epilogue
      ok = __all_sync(0xffffffffu, attn_wait(pv_done, (g - 1) & 1, abort_flag, p.polls));
      if (!ok && lane == 0) attn_fail(p, abort_flag, 10);
      if (ok) {
        tc_fence_after();
        write_out(prev_id, l_prev);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, kAttnTmemCols);
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
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(attention_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
    if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(attention_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
  });
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
  p.c = scale * 1.4426950408889634f;
  p.out = out;
  p.o_batch = o_str[0];
  p.o_head = o_str[1];
  p.o_row = o_str[2];
  p.err = gemm_error_word();
  uint32_t drill_polls = 0;
  take_next_wait_test(&drill_polls, &p.skip_loads);
  p.polls = drill_polls ? drill_polls : kAttnPolls;
  if (!p.err) { set_error("attention: cannot resolve the device error word"); return PGB_ERR_CUDA; }
  const unsigned grid = (unsigned)std::min<int64_t>(B * H * n_qblk, (int64_t)kAttnCtasPerSm * sm_count());
  p.snake = B * H * n_qblk <= 3 * (int64_t)grid ? 1 : 0;
  if (is_half) attention_fwd_kernel<true><<<grid, kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, p);
  else attention_fwd_kernel<false><<<grid, kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, p);
  count_launch();
  return check_launch("attention_fwd_kernel");
}

}  // namespace pgb
