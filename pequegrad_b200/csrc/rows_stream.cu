// LayerNorm over many fp32 rows as a persistent, pipelined streaming kernel.
//
// The warp-per-row kernel in rows.cu is a chain load -> two reductions -> store per CTA; on a tensor of a few
// tens of MB (LayerNorm over [16384, 768] is 50 MB in, 50 MB out: 15 us at the HBM peak) the grid is only two
// or three waves of such chains and the memory system idles between them. Here two CTAs per SM stay resident
// and walk the tensor: a producer warp keeps a ring of row blocks (8 rows each) filling through the TMA unit
// (1-D bulk copies, completion on an mbarrier, no multicast), eight consumer warps take one row each out of
// shared memory, normalise it in registers and store it with coalesced 128-bit stores. Loads of the blocks to
// come are in flight while the current one is computed and stored, so the DRAM queue never drains.
// The arithmetic is that of layernorm_warp_kernel (and of the composite, pequegrad/ops.py:515-551): mean,
// biased variance of the deviations, eps before the square root.
#include <cstdlib>

#include "gemm_ptx.cuh"
#include "reduce_common.cuh"

namespace pgb {

namespace {

constexpr int kRowsPerBlock = 8;  // one per consumer warp
constexpr int kConsumers = kRowsPerBlock * 32;
constexpr int kStreamThreads = kConsumers + 32;  // + the producer warp

struct StreamParams {
  const float *x;
  float *y;
  const float *gamma, *beta;
  int64_t rows;
  int C;
  int stages;
  float eps;
  int *err;  // device error word shared with the GEMM kernels: a wait that ran out is recorded there
};

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

// 1-D bulk copy global -> shared through the TMA unit; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)), "l"(gsrc),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int NV>
__global__ void __launch_bounds__(kStreamThreads, 2) layernorm_stream_kernel(const __grid_constant__ StreamParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int C = p.C, S = p.stages;
  const uint32_t row_bytes = (uint32_t)C * 4u, blk_bytes = row_bytes * kRowsPerBlock;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);  // [S] producer -> consumers (transaction bytes)
  uint64_t *empty = full + S;                            // [S] consumers -> producer (one arrival per warp)
  volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + S);
  float *ring = reinterpret_cast<float *>(smem + 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (*(volatile int *)p.err != 0) return;  // an earlier kernel gave up on a wait: do nothing until the host has cleared the word
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kRowsPerBlock); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int64_t nblk = (p.rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (warp == kRowsPerBlock) {
    if (lane == 0) {
      uint32_t phase = 0;
      int s = 0;
      for (int64_t b = blockIdx.x; b < nblk; b += gridDim.x) {
        if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) {  // the stage's previous block has been read by all eight warps
          *abort_flag = 1;
          atomicCAS(p.err, 0, (8 << 16) | (int)(blockIdx.x & 0xffff));
          break;
        }
        const int64_t r0 = b * kRowsPerBlock;
        const uint32_t bytes = (uint32_t)((p.rows - r0 < kRowsPerBlock ? p.rows - r0 : kRowsPerBlock)) * row_bytes;
        mbar_expect_tx(&full[s], bytes);
        bulk_load(reinterpret_cast<uint8_t *>(ring) + (size_t)s * blk_bytes, p.x + r0 * C, bytes, &full[s]);
        if (++s == S) { s = 0; phase ^= 1; }
      }
    }
    return;
  }
  // consumers: per-lane column operands stay in registers for the whole kernel
  float g[NV][4], be[NV][4];
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int c = (u * 32 + lane) * 4;
    float4 gv = make_float4(1.f, 1.f, 1.f, 1.f), bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < C) {
      if (p.gamma) gv = __ldg(reinterpret_cast<const float4 *>(p.gamma + c));
      if (p.beta) bv = __ldg(reinterpret_cast<const float4 *>(p.beta + c));
    }
    g[u][0] = gv.x; g[u][1] = gv.y; g[u][2] = gv.z; g[u][3] = gv.w;
    be[u][0] = bv.x; be[u][1] = bv.y; be[u][2] = bv.z; be[u][3] = bv.w;
  }
  const bool has_g = p.gamma != nullptr, has_b = p.beta != nullptr;
  const float n = (float)C;
  uint32_t phase = 0;
  int s = 0;
  for (int64_t b = blockIdx.x; b < nblk; b += gridDim.x) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait(&full[s], phase, abort_flag);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) {
      if (lane == 0) {
        *abort_flag = 1;
        atomicCAS(p.err, 0, (9 << 16) | (int)(blockIdx.x & 0xffff));
      }
      return;
    }
    const int64_t row = b * kRowsPerBlock + warp;
    const float *xr = ring + (size_t)s * (blk_bytes / 4) + (size_t)warp * C;
    float v[NV][4];
    float sum = 0.f;
    if (row < p.rows) {
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        const int c = (u * 32 + lane) * 4;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < C) t = *reinterpret_cast<const float4 *>(xr + c);
        v[u][0] = t.x; v[u][1] = t.y; v[u][2] = t.z; v[u][3] = t.w;
        sum += (t.x + t.y) + (t.z + t.w);
      }
    }
    // the row is in registers: hand the stage back before the arithmetic
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    if (++s == S) { s = 0; phase ^= 1; }
    if (row >= p.rows) continue;
    const float mean = wsum(sum) / n;
    float q = 0.f;
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const int c = (u * 32 + lane) * 4;
      if (c < C) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[u][e] = v[u][e] - mean;
          q += v[u][e] * v[u][e];
        }
      }
    }
    const float var = wsum(q) / n;
    const float rsd = 1.0f / sqrtf(var + p.eps);
    float *yr = p.y + row * C;
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const int c = (u * 32 + lane) * 4;
      if (c < C) {
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[e] = v[u][e] * rsd;
          if (has_g) o[e] = o[e] * g[u][e];
          if (has_b) o[e] = o[e] + be[u][e];
        }
        __stcs(reinterpret_cast<float4 *>(yr + c), make_float4(o[0], o[1], o[2], o[3]));
      }
    }
  }
}

template <int NV>
int launch_stream(const StreamParams &p, int grid, size_t smem, cudaStream_t stream) {
  static cudaError_t attr_err = [] {
    cudaError_t e = cudaFuncSetAttribute(layernorm_stream_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    // two CTAs of ~100 KB per SM only fit when the L1 / shared split leans fully to shared memory
    if (e == cudaSuccess) e = cudaFuncSetAttribute(layernorm_stream_kernel<NV>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return e;
  }();
  if (attr_err != cudaSuccess) return 0;
  layernorm_stream_kernel<NV><<<grid, kStreamThreads, smem, stream>>>(p);
  count_launch();
  return check_launch("layernorm_stream_kernel") == PGB_OK ? 1 : PGB_ERR_CUDA;
}

}  // namespace

// Returns 1 when the streaming kernel took the call, 0 when the shape is not its case (the caller falls back to
// the warp-per-row kernel), a negative status on a launch error.
int launch_layernorm_stream_f32(const float *x, float *y, const float *gamma, const float *beta, int64_t rows, int64_t C, float eps,
                                cudaStream_t stream) {
  const auto a16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (C % 4 != 0 || C < 128 || C > 1024 || rows < 2048) return 0;
  if (!a16(x) || !a16(y) || (gamma && !a16(gamma)) || (beta && !a16(beta))) return 0;
  const size_t blk = (size_t)C * 4 * kRowsPerBlock;
  const char *var = getenv("PGB_LN_VARIANT");
  const int variant = var ? atoi(var) : 1;
  if (variant == 0 || variant >= 3) return 0;
  const int per_sm = variant == 2 ? 1 : 2;
  int stages = (int)(((variant == 2 ? 200 : 100) * 1024) / blk);  // two CTAs per SM: about 100 KB of ring each
  if (stages > 6) stages = 6;
  if (stages < 2) return 0;
  StreamParams p{x, y, gamma, beta, rows, (int)C, stages, eps, gemm_error_word()};
  if (!p.err) return 0;
  const int64_t nblk = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  int64_t grid = (int64_t)sm_count() * per_sm;
  if (grid > nblk) grid = nblk;
  const size_t smem = 128 + (size_t)stages * blk;
  const int nv = (int)((C + 127) / 128);
  if (nv <= 2) return launch_stream<2>(p, (int)grid, smem, stream);
  if (nv <= 4) return launch_stream<4>(p, (int)grid, smem, stream);
  if (nv <= 6) return launch_stream<6>(p, (int)grid, smem, stream);
  return launch_stream<8>(p, (int)grid, smem, stream);
}

}  // namespace pgb
