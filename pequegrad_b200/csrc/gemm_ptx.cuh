// PTX wrappers for the tensor-core GEMM kernels: mbarriers, TMA tile loads,
// TMEM allocation, tcgen05 MMA / commit / load, shared-memory matrix descriptors.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm.hpp"

namespace pgb {

constexpr uint32_t kSpinLimit = 1u << 20;  // polls per wait before a role gives up

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false if the barrier did not flip within the limit or
// another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *tmap, int x, int y, int z, int w, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
      : "memory");
}
// Asks the TMA unit to bring a tile into L2 (no shared-memory destination, nothing to wait for).
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap *tmap, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  if (KIND == GEMM_I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if (KIND == GEMM_TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 lanes x 32 columns of 32-bit: thread t of the warp receives lane (base + t), columns c .. c+31
// The load is asynchronous: the registers are valid only after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
        "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The mirror image: thread t of the warp writes lane (base + t), columns c .. c+31. Complete after tmem_st_wait().
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
      "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
      "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are one 128-byte
// swizzle atom wide: 8-row groups are 1024 bytes apart (stride byte offset),
// leading byte offset is 1 (unused for swizzled K-major), version 1 (Blackwell),
// layout type 2 = SWIZZLE_128B. Field positions as in the PTX matrix-descriptor
// format: start address [0,14), LBO [16,30), SBO [32,46), version [46,48), layout [61,64),
// addresses and offsets in units of 16 bytes.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Descriptor of an MN-major tile (the M or N dim is contiguous, K runs across rows) stored as rows of one
// 128-byte swizzle atom: row k holds 64 16-bit elements of the M/N dim, 8-row groups are 1024 bytes apart
// (stride byte offset = the K-direction group stride); the leading byte offset would separate 64-element
// atoms along M/N and is not used by a 64-wide tile.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// TMA tile store shared -> global (bulk async group of the issuing thread). The tensor map clips the box
// at the tensor's extents, so ragged right / bottom edges need no special case.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *tmap, const void *smem_src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tmap), "r"(smem_u32(smem_src)),
               "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of this thread's bulk groups still have to READ their shared-memory source
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// makes this thread's generic-proxy writes to shared memory visible to the async proxy (TMA)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// clip(rint(x / s), -127, 127) with the IEEE quotient's rounding, r = RN(1 / s). The quotient comes from one
// Newton step on x * r (within one ulp of x / s); only when that lands within 1e-4 of a rounding boundary,
// or is not finite, does the IEEE division run. (div.rn itself takes a slow path for zero numerators,
// which is half of a ReLU output.)
__device__ __forceinline__ float quant_i8_exact(float x, float s, float r) {
  const float y0 = x * r;
  const float y = fmaf(fmaf(-y0, s, x), r, y0);
  float k = rintf(y);
  if (!(fabsf(y - k) <= 0.4999f)) k = rintf(__fdiv_rn(x, s));
  return fminf(fmaxf(k, -127.f), 127.f);
}
__device__ __forceinline__ uint32_t quant_i8_pack4(float a, float b, float c, float d, float s, float r) {
  return ((uint32_t)(uint8_t)(int8_t)(int)quant_i8_exact(a, s, r)) | ((uint32_t)(uint8_t)(int8_t)(int)quant_i8_exact(b, s, r) << 8) |
         ((uint32_t)(uint8_t)(int8_t)(int)quant_i8_exact(c, s, r) << 16) | ((uint32_t)(uint8_t)(int8_t)(int)quant_i8_exact(d, s, r) << 24);
}
// The cheap route to the same four bytes, for the common case: k = rint(clamp(x * r)) by adding 1.5 * 2^23 (the sum's low
// mantissa byte is k in two's complement, rounding is to nearest even), then the residual x - k * s from one fused
// multiply-add certifies k: |x - k s| <= 0.49999 s means x / s is at least 1e-5 away from the rounding boundaries, farther
// than the rounding of the fp32 quotient can move it (4e-6 for |k| < 128), so rint of the IEEE quotient is the same k.
// Anything else (a boundary, a clamped value, NaN) raises `recheck` and the caller redoes the group with quant_i8_pack4.
// NONNEG: the values are outputs of a ReLU, so only the upper clamp is needed.
template <bool NONNEG>
__device__ __forceinline__ uint32_t quant_i8_fast4(float a, float b, float c, float d, float s, float r, float thr, bool &recheck) {
  const float kMagic = 12582912.f;  // 1.5 * 2^23
  const float x[4] = {a, b, c, d};
  uint32_t t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float y = fminf(x[i] * r, 127.f);
    if (!NONNEG) y = fmaxf(y, -127.f);
    const float ti = y + kMagic;
    const float kf = ti - kMagic;
    recheck |= !(fabsf(fmaf(-kf, s, x[i])) <= thr);
    t[i] = __float_as_uint(ti);
  }
  const uint32_t lo = __byte_perm(t[0], t[1], 0x0040), hi = __byte_perm(t[2], t[3], 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
  // (pequegrad/ops.py:109-118, 159-164). tanh is the hardware approximation (relative error about 2^-11),
  // inside the 16-bit tolerance of the outputs this feeds.
  const float z = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(z));  // one SFU operation per element
  const float hx = 0.5f * x;
  return fmaf(hx, t, hx);
}

}  // namespace pgb
