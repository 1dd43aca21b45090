// Dynamic per-tensor int8 quantisation of activations (absmax, then quantise).
// The reference has no int8 type; its example scales by max|.| floored at 1e-6
// (examples/quantized_mlp.py:28-34), which these kernels keep.
#include "gemm_ptx.cuh"
#include "reduce_common.cuh"

namespace pgb {

// absmax: one pass, atomicMax on the bit pattern. quantize: q = clip(rint(x / s), -127, 127),
// s = max(absmax, 1e-6) / 127, the rounding of the true fp32 quotient, round half to even.
// Both stream the tensor in tiles of 256 threads x U 128-bit vectors, one tile per CTA: every load of a thread is
// issued before the first is used, a CTA touches one contiguous 16 / 32 KB span, and the hardware scheduler balances
// the tail. (A grid-stride loop over far-apart vectors left a fifth of the tensor to a remainder loop with a single
// load in flight: 3.7 TB/s from DRAM.)
constexpr int kAbsmaxU = 8, kQuantU = 4;

__global__ void __launch_bounds__(256) absmax_f32_kernel(const float *__restrict__ x, int64_t n, float *out) {
  const int64_t nvec = n >> 2;
  const float4 *x4 = reinterpret_cast<const float4 *>(x);
  const int64_t base = (int64_t)blockIdx.x * (256 * kAbsmaxU) + threadIdx.x;
  float4 v[kAbsmaxU];
#pragma unroll
  for (int u = 0; u < kAbsmaxU; ++u) {
    const int64_t i = base + u * 256;
    v[u] = i < nvec ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);  // default caching: the tail of the tensor stays in L2 for the quantise pass
  }
  float m = 0.f;
#pragma unroll
  for (int u = 0; u < kAbsmaxU; ++u) m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) m = fmaxf(m, fabsf(x[(nvec << 2) + threadIdx.x]));
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, k));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, wm[w]);
    // one atomic per CTA, and none once the running maximum is at least this CTA's (non-negative floats order like their bits)
    if (m > 0.f && m > __ldcg(out)) atomicMax(reinterpret_cast<unsigned int *>(out), __float_as_uint(m));
  }
}

// One float4 in, one packed word out per thread and vector: a warp reads 512 and writes 128 contiguous bytes.
// Tiles are taken from the END of the tensor backwards: after the absmax pass the last part of a tensor larger than
// the L2 is what the L2 still holds.
__global__ void __launch_bounds__(256) quantize_i8_kernel(const float *__restrict__ x, int64_t n, const float *__restrict__ absmax,
                                                          float scale_host, int8_t *__restrict__ q) {
  const float s = absmax ? fmaxf(__ldg(absmax), 1e-6f) / 127.0f : scale_host;
  const float r = 1.0f / s, thr = 0.49999f * s;
  const int64_t nvec = n >> 2;
  const float4 *x4 = reinterpret_cast<const float4 *>(x);
  uint32_t *q4 = reinterpret_cast<uint32_t *>(q);
  const int64_t base = (int64_t)(gridDim.x - 1 - blockIdx.x) * (256 * kQuantU) + threadIdx.x;
  float4 v[kQuantU];
#pragma unroll
  for (int u = 0; u < kQuantU; ++u) {
    const int64_t i = base + u * 256;
    v[u] = i < nvec ? __ldcs(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int u = 0; u < kQuantU; ++u) {
    const int64_t i = base + u * 256;
    if (i >= nvec) break;
    bool recheck = false;
    uint32_t w = quant_i8_fast4<false>(v[u].x, v[u].y, v[u].z, v[u].w, s, r, thr, recheck);
    if (recheck) w = quant_i8_pack4(v[u].x, v[u].y, v[u].z, v[u].w, s, r);
    q4[i] = w;
  }
  // the last n % 4 elements
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const int64_t j = (nvec << 2) + threadIdx.x;
    q[j] = (int8_t)(int)quant_i8_exact(x[j], s, r);
  }
}

int run_absmax_f32(const float *x, int64_t n, float *out, cudaStream_t stream) {
  if (cudaMemsetAsync(out, 0, sizeof(float), stream) != cudaSuccess) { set_error("absmax: memset failed"); return PGB_ERR_CUDA; }
  if (n <= 0) return PGB_OK;
  const int64_t per = 256 * kAbsmaxU * 4;
  const int64_t grid = (n + per - 1) / per;
  if (grid > 2147483647LL) { set_error("absmax: tensor too large"); return PGB_ERR_UNSUPPORTED; }
  absmax_f32_kernel<<<(unsigned)grid, 256, 0, stream>>>(x, n, out);
  count_launch();
  return check_launch("absmax_f32_kernel");
}

int run_quantize_i8(const float *x, int64_t n, const float *absmax_dev, float scale, int8_t *q, cudaStream_t stream) {
  if (n <= 0) return PGB_OK;
  const int64_t per = 256 * kQuantU * 4;
  const int64_t grid = (n + per - 1) / per;
  if (grid > 2147483647LL) { set_error("quantize: tensor too large"); return PGB_ERR_UNSUPPORTED; }
  quantize_i8_kernel<<<(unsigned)grid, 256, 0, stream>>>(x, n, absmax_dev, scale, q);
  count_launch();
  return check_launch("quantize_i8_kernel");
}

}  // namespace pgb
