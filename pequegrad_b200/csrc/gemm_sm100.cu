// Dense contractions on the 5th-generation tensor cores: tcgen05.mma with the
// accumulator in TMEM, operands staged in shared memory by TMA (no multicast),
// mbarrier pipeline, warp-specialised roles. Two instantiations of one kernel:
//   kind::i8   int8 x int8 -> int32   (quantized linear, fused dequant + bias + ReLU)
//   kind::f16  f16 / bf16 -> f32      (matmul / linear with bias, ReLU / GELU, residual)
//
// Replaces MatMul::dispatch_cuda (cuBLAS strided-batched GEMM with a handle
// created and destroyed per call, and fp16 ACCUMULATION for half inputs,
// csrc/cuda/matmul.cu:72-163) and FusedLinearBiasAct::dispatch_cuda (CUTLASS 2.x
// Sm75 tiles, csrc/cuda/other.cu:19-166). The reference has no int8 path.
//
// Both operands are K-major: A is [M, K] and B is [N, K], K contiguous
// (a Linear weight is passed as its transpose, prepared once). One CTA computes
// one 128 x BN tile of C:
//   warp 0     TMA producer: 128-byte-wide K slabs of A and B per stage, 128B swizzle
//   warp 1     allocates TMEM, issues tcgen05.mma (one elected thread), commits
//   warps 2-5  epilogue: tcgen05.ld the accumulator (one row per thread), apply
//              the fused epilogue, store
// Every wait is bounded: on a timeout the kernel records an error word that
// pgb_device_error() reads, skips the rest of its work and frees its TMEM.
#include <cuda.h>

#include <mutex>

#include "gemm.hpp"
#include "reduce_common.cuh"

namespace pgb {

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kSlabBytes = 128;  // bytes of K per stage = one 128B swizzle atom row
constexpr int kStages = 3;
constexpr int kTileABytes = kBM * kSlabBytes;
constexpr int kTileBBytes = kBN * kSlabBytes;
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kGemmThreads = 192;
constexpr int kGemmSmem = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kSpinLimit = 1u << 20;  // polls per wait before a role gives up

static __device__ int g_gemm_error;  // 0 = ok; else (role << 16) | block index bits

struct GemmParams {
  int M, N, K;  // K in elements
  int num_kb;   // K slabs
  GemmEpilogue epi;
};

// ---- PTX wrappers -----------------------------------------------------------
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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *tmap, int x, int y, int z, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
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
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 lanes x 32 columns of 32-bit: thread t of the warp receives lane (base + t), columns c .. c+31
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

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

// Instruction descriptor: c format [4,6) (1 = f32, 2 = s32), a format [7,10), b format [10,13)
// (f16 kinds: 0 f16, 1 bf16; i8: 1 = signed), a/b major [15],[16] (0 = K-major),
// N >> 3 at [17,23), M >> 4 at [24,29).
template <int KIND>
__device__ __forceinline__ uint32_t make_idesc() {
  uint32_t d = 0;
  const uint32_t cfmt = (KIND == GEMM_I8) ? 2u : 1u;
  const uint32_t abfmt = (KIND == GEMM_F16) ? 0u : 1u;  // i8 signed = 1, bf16 = 1, f16 = 0
  d |= cfmt << 4;
  d |= abfmt << 7;
  d |= abfmt << 10;
  d |= (uint32_t)(kBN >> 3) << 17;
  d |= (uint32_t)(kBM >> 4) << 24;
  return d;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), tanh(z) = 2 / (1 + exp(-2z)) - 1
  // (pequegrad/ops.py:109-118, 159-164)
  const float z = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = 2.0f / (1.0f + expf(-2.0f * z)) - 1.0f;
  return 0.5f * x * (1.0f + t);
}

template <int KIND>
__global__ void __launch_bounds__(kGemmThreads) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                 const __grid_constant__ CUtensorMap tmap_b,
                                                                 const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128B-swizzled tiles
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  uint8_t *tiles = smem;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
  uint64_t *full = bars;               // [kStages]
  uint64_t *empty = bars + kStages;    // [kStages]
  uint64_t *acc_full = bars + 2 * kStages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  // a kernel of an earlier launch gave up on a wait: do nothing until the host has read and cleared the error
  if (*(volatile int *)&g_gemm_error != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * kBM, bz = blockIdx.z;
  constexpr int ES = (KIND == GEMM_I8) ? 1 : 2;
  constexpr int SLAB_ELEMS = kSlabBytes / ES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kBN);  // kBN fp32 / int32 columns x 128 lanes
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
      uint32_t phase = 0;
      int s = 0;
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_gemm_error, 0, (1 << 16) | (blockIdx.x & 0xffff));
          break;
        }
        mbar_expect_tx(&full[s], kStageBytes);
        uint8_t *sa = tiles + s * kStageBytes;
        tma_load_3d(sa, &tmap_a, kb * SLAB_ELEMS, m0, bz, &full[s]);
        tma_load_3d(sa + kTileABytes, &tmap_b, kb * SLAB_ELEMS, n0, bz, &full[s]);
        if (++s == kStages) { s = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc<KIND>();
      uint32_t phase = 0;
      int s = 0;
      bool ok = true;
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!mbar_wait(&full[s], phase, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_gemm_error, 0, (2 << 16) | (blockIdx.x & 0xffff));
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(tiles + s * kStageBytes);
        const uint64_t da = make_kmajor_sw128_desc(sa), db = make_kmajor_sw128_desc(sa + kTileABytes);
#pragma unroll
        for (int kk = 0; kk < kSlabBytes / 32; ++kk)  // one MMA consumes 32 bytes of K: +2 in 16-byte units
          tc_mma<KIND>(tmem_base, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
        tc_commit(&empty[s]);  // frees the stage when these MMAs have read it
        if (++s == kStages) { s = 0; phase ^= 1; }
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    // epilogue: warp w may read TMEM lanes 32*(w%4) .. +31
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    const GemmEpilogue &e = p.epi;
    bool ok = true;
    if (lane == 0) ok = mbar_wait(acc_full, 0, abort_flag);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) {
      if (lane == 0) { *abort_flag = 1; atomicCAS(&g_gemm_error, 0, (3 << 16) | (blockIdx.x & 0xffff)); }
    } else {
      tc_fence_after();
      float a_scale = e.a_scale;
      if (KIND == GEMM_I8 && e.a_scale_dev) {
        // activation scale from the running absmax: max(amax, 1e-6) / 127, same fp32 ops as the host formula
        a_scale = fmaxf(__ldg(e.a_scale_dev), 1e-6f) / 127.0f;
      }
      float local_max = 0.f;
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);  // all lanes: sync.aligned
        if (row < p.M && n0 + c0 < p.N) {
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = n0 + c0 + i;
            float x;
            if (KIND == GEMM_I8) {
              const float sc = (e.col_scale && col < p.N) ? __fmul_rn(a_scale, __ldg(e.col_scale + col)) : a_scale;
              x = __fmul_rn((float)(int)v[i], sc);
            } else {
              x = __uint_as_float(v[i]);
            }
            if (e.bias && col < p.N) x = __fadd_rn(x, load_as<float>(e.bias, e.bias_dtype, col));
            if (e.act == ACT_RELU) x = x > 0.f ? x : 0.f;
            else if (e.act == ACT_GELU_TANH) x = gelu_tanh(x);
            if (e.residual && col < p.N)
              x = __fadd_rn(x, load_as<float>(e.residual, e.res_dtype, (int64_t)bz * e.res_batch + (int64_t)row * e.res_ld + col));
            f[i] = x;
            if (col < p.N) local_max = fmaxf(local_max, fabsf(x));
          }
          const bool full_chunk = n0 + c0 + 32 <= p.N;
          if (e.acc_out) {
            int32_t *dst = e.acc_out + (int64_t)row * e.ld_acc + n0 + c0;
            if (full_chunk && (e.ld_acc & 3) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) *reinterpret_cast<int4 *>(dst + i) = make_int4((int)v[i], (int)v[i + 1], (int)v[i + 2], (int)v[i + 3]);
            } else {
              for (int i = 0; i < 32 && n0 + c0 + i < p.N; ++i) dst[i] = (int)v[i];
            }
          }
          if (e.out) {
            const int64_t off = (int64_t)bz * e.out_batch + (int64_t)row * e.ldc + n0 + c0;
            if (e.out_dtype == PGB_F32) {
              float *dst = (float *)e.out + off;
              if (full_chunk && (e.ldc & 3) == 0 && (e.out_batch & 3) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4 *>(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
              } else {
                for (int i = 0; i < 32 && n0 + c0 + i < p.N; ++i) dst[i] = f[i];
              }
            } else {
              const bool is_h = e.out_dtype == PGB_F16;
              uint16_t *dst = (uint16_t *)e.out + off;
              if (full_chunk && (e.ldc & 7) == 0 && (e.out_batch & 7) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint32_t w[4];
#pragma unroll
                  for (int h = 0; h < 4; ++h) {
                    uint16_t lo, hi;
                    if (is_h) { lo = __half_as_ushort(__float2half_rn(f[i + 2 * h])); hi = __half_as_ushort(__float2half_rn(f[i + 2 * h + 1])); }
                    else { lo = __bfloat16_as_ushort(__float2bfloat16_rn(f[i + 2 * h])); hi = __bfloat16_as_ushort(__float2bfloat16_rn(f[i + 2 * h + 1])); }
                    w[h] = (uint32_t)lo | ((uint32_t)hi << 16);
                  }
                  *reinterpret_cast<uint4 *>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
                }
              } else {
                for (int i = 0; i < 32 && n0 + c0 + i < p.N; ++i)
                  dst[i] = is_h ? __half_as_ushort(__float2half_rn(f[i])) : __bfloat16_as_ushort(__float2bfloat16_rn(f[i]));
              }
            }
          }
        }
      }
      if (e.absmax) {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, m));
        // non-negative floats order like their bit patterns
        if (lane == 0 && local_max > 0.f) atomicMax(reinterpret_cast<unsigned int *>(e.absmax), __float_as_uint(local_max));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kBN);
}

// ---- activation quantisation (per tensor, dynamic) ---------------------------
// absmax: one pass, atomicMax on the bit pattern. quantize: q = clip(rint(x / s), -127, 127),
// s = max(absmax, 1e-6) / 127, true fp32 division, round half to even.
__global__ void __launch_bounds__(256) absmax_f32_kernel(const float *__restrict__ x, int64_t n, float *out) {
  float m = 0.f;
  const int64_t stride = (int64_t)gridDim.x * 256 * 4;
  for (int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(x + i));
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    } else {
      for (int64_t j = i; j < n; ++j) m = fmaxf(m, fabsf(x[j]));
    }
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, k));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int *>(out), __float_as_uint(m));
}

__global__ void __launch_bounds__(256) quantize_i8_kernel(const float *__restrict__ x, int64_t n, const float *__restrict__ absmax,
                                                          float scale_host, int8_t *__restrict__ q) {
  const float s = absmax ? fmaxf(__ldg(absmax), 1e-6f) / 127.0f : scale_host;
  const int64_t stride = (int64_t)gridDim.x * 256 * 16;
  for (int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 16; i < n; i += stride) {
    if (i + 15 < n) {
      uint32_t w[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const float4 v = __ldcs(reinterpret_cast<const float4 *>(x + i + 4 * g));
        const float f[4] = {v.x, v.y, v.z, v.w};
        uint32_t pk = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float r = rintf(__fdiv_rn(f[e], s));
          r = fminf(fmaxf(r, -127.f), 127.f);
          pk |= ((uint32_t)(uint8_t)(int8_t)(int)r) << (8 * e);
        }
        w[g] = pk;
      }
      *reinterpret_cast<uint4 *>(q + i) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      for (int64_t j = i; j < n; ++j) {
        float r = rintf(__fdiv_rn(x[j], s));
        r = fminf(fmaxf(r, -127.f), 127.f);
        q[j] = (int8_t)(int)r;
      }
    }
  }
}

// ---- host side ---------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// [batch, rows, K] K-major operand -> 3-D tensor map with a {128 bytes of K, box_rows, 1} box, 128B swizzle
static int make_operand_map(CUtensorMap *map, const void *ptr, int kind, int64_t rows, int64_t K, int64_t ld_elems, int64_t batch,
                            int64_t batch_stride_elems, int box_rows, const char *what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("matmul: cuTensorMapEncodeTiled is not available from this driver"); return PGB_ERR_CUDA; }
  const int es = kind == GEMM_I8 ? 1 : 2;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld_elems * es) % 16 || (batch > 1 && (batch_stride_elems * es) % 16)) {
    set_error(std::string("matmul: operand ") + what + " must be 16-byte aligned with row and batch pitches that are multiples of 16 bytes");
    return PGB_ERR_UNSUPPORTED;
  }
  const CUtensorMapDataType dt = kind == GEMM_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                 : (kind == GEMM_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)(ld_elems * es), (cuuint64_t)((batch > 1 ? batch_stride_elems : rows * ld_elems) * es)};
  const cuuint32_t box[3] = {(cuuint32_t)(kSlabBytes / es), (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, dt, 3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(std::string("matmul: cuTensorMapEncodeTiled failed for operand ") + what + " (code " + std::to_string((int)r) + ")");
    return PGB_ERR_CUDA;
  }
  return PGB_OK;
}

static int ensure_smem_attr() {
  static std::once_flag once;
  static cudaError_t err = cudaSuccess;
  std::call_once(once, [] {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<GEMM_I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<GEMM_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<GEMM_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    err = e;
  });
  if (err != cudaSuccess) { set_error(std::string("matmul: cannot raise the shared-memory limit: ") + cudaGetErrorString(err)); return PGB_ERR_CUDA; }
  return PGB_OK;
}

// a: [batch, M, K], b: [batch, N, K] (batch stride 0 = shared weights), both K contiguous.
int run_gemm_tc(int kind, const void *a, int64_t lda, int64_t a_batch, const void *b, int64_t ldb, int64_t b_batch, int64_t M, int64_t N,
                int64_t K, int64_t batch, const GemmEpilogue &epi, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return PGB_OK;
  if (K <= 0) { set_error("matmul: empty contraction dim"); return PGB_ERR_INVALID_ARG; }
  if (M > 2147483647LL || N > 2147483647LL || K > 2147483647LL || (M + kBM - 1) / kBM > 65535 || batch > 65535) {
    set_error("matmul: problem too large for one launch");
    return PGB_ERR_UNSUPPORTED;
  }
  int st = ensure_smem_attr();
  if (st != PGB_OK) return st;
  CUtensorMap ma, mb;
  st = make_operand_map(&ma, a, kind, M, K, lda, batch, a_batch, kBM, "A");
  if (st != PGB_OK) return st;
  // a weight shared by every batch entry is described with batch extent 1 and always addressed at z = 0
  if (b_batch == 0 && batch > 1) { set_error("matmul: batched A with an unbatched B: flatten the batch into M"); return PGB_ERR_UNSUPPORTED; }
  st = make_operand_map(&mb, b, kind, N, K, ldb, batch, b_batch, kBN, "B");
  if (st != PGB_OK) return st;
  GemmParams p{};
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  const int es = kind == GEMM_I8 ? 1 : 2;
  p.num_kb = (int)((K * es + kSlabBytes - 1) / kSlabBytes);
  p.epi = epi;
  dim3 grid((unsigned)((N + kBN - 1) / kBN), (unsigned)((M + kBM - 1) / kBM), (unsigned)batch);
  if (kind == GEMM_I8) gemm_tc_kernel<GEMM_I8><<<grid, kGemmThreads, kGemmSmem, stream>>>(ma, mb, p);
  else if (kind == GEMM_F16) gemm_tc_kernel<GEMM_F16><<<grid, kGemmThreads, kGemmSmem, stream>>>(ma, mb, p);
  else gemm_tc_kernel<GEMM_BF16><<<grid, kGemmThreads, kGemmSmem, stream>>>(ma, mb, p);
  count_launch();
  return check_launch("gemm_tc_kernel");
}

int run_absmax_f32(const float *x, int64_t n, float *out, cudaStream_t stream) {
  if (cudaMemsetAsync(out, 0, sizeof(float), stream) != cudaSuccess) { set_error("absmax: memset failed"); return PGB_ERR_CUDA; }
  if (n <= 0) return PGB_OK;
  int64_t grid = (n + 1023) / 1024;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (grid > cap) grid = cap;
  absmax_f32_kernel<<<(unsigned)grid, 256, 0, stream>>>(x, n, out);
  count_launch();
  return check_launch("absmax_f32_kernel");
}

int run_quantize_i8(const float *x, int64_t n, const float *absmax_dev, float scale, int8_t *q, cudaStream_t stream) {
  if (n <= 0) return PGB_OK;
  int64_t grid = (n + 4095) / 4096;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (grid > cap) grid = cap;
  quantize_i8_kernel<<<(unsigned)grid, 256, 0, stream>>>(x, n, absmax_dev, scale, q);
  count_launch();
  return check_launch("quantize_i8_kernel");
}

int read_gemm_error(int *out, bool reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return PGB_ERR_CUDA; }
  if (reset && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  }
  *out = v;
  return PGB_OK;
}

}  // namespace pgb
