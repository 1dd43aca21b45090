// Dynamic per-tensor int8 quantisation of activations (absmax, then quantise).
// The reference has no int8 type; its example scales by max|.| floored at 1e-6
// (examples/quantized_mlp.py:28-34), which these kernels keep.
#include "gemm_ptx.cuh"
#include "reduce_common.cuh"

namespace pgb {

// absmax: one pass, atomicMax on the bit pattern. quantize: q = clip(rint(x / s), -127, 127),
// s = max(absmax, 1e-6) / 127, the rounding of the true fp32 quotient, round half to even.
__global__ void __launch_bounds__(256) absmax_f32_kernel(const float *__restrict__ x, int64_t n, float *out) {
  float m = 0.f;
  const int64_t nvec = n >> 2, stride = (int64_t)gridDim.x * 256;
  const float4 *x4 = reinterpret_cast<const float4 *>(x);
  int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  for (; i + 7 * stride < nvec; i += 8 * stride) {  // eight independent 128-bit loads in flight per thread
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcs(x4 + i + u * stride);
#pragma unroll
    for (int u = 0; u < 8; ++u) m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
  }
  for (; i < nvec; i += stride) {
    const float4 v = __ldcs(x4 + i);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) m = fmaxf(m, fabsf(x[(nvec << 2) + threadIdx.x]));
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, k));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int *>(out), __float_as_uint(m));
}

// One float4 in, one packed word out per thread and step: a warp reads 512 and writes 128 contiguous
// bytes. Four independent steps are in flight per thread.
__global__ void __launch_bounds__(256) quantize_i8_kernel(const float *__restrict__ x, int64_t n, const float *__restrict__ absmax,
                                                          float scale_host, int8_t *__restrict__ q) {
  const float s = absmax ? fmaxf(__ldg(absmax), 1e-6f) / 127.0f : scale_host;
  const float r = 1.0f / s, thr = 0.49999f * s;
  const int64_t nvec = n >> 2;
  const int64_t stride = (int64_t)gridDim.x * 256;
  const float4 *x4 = reinterpret_cast<const float4 *>(x);
  uint32_t *q4 = reinterpret_cast<uint32_t *>(q);
  int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcs(x4 + i + u * stride);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      bool recheck = false;
      uint32_t w = quant_i8_fast4<false>(v[u].x, v[u].y, v[u].z, v[u].w, s, r, thr, recheck);
      if (recheck) w = quant_i8_pack4(v[u].x, v[u].y, v[u].z, v[u].w, s, r);
      q4[i + u * stride] = w;
    }
  }
  for (; i < nvec; i += stride) {
    const float4 v = __ldcs(x4 + i);
    q4[i] = quant_i8_pack4(v.x, v.y, v.z, v.w, s, r);
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
  int64_t grid = (n + 8191) / 8192;  // 8 vectors of 4 elements per thread
  const int64_t cap = (int64_t)sm_count() * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  absmax_f32_kernel<<<(unsigned)grid, 256, 0, stream>>>(x, n, out);
  count_launch();
  return check_launch("absmax_f32_kernel");
}

int run_quantize_i8(const float *x, int64_t n, const float *absmax_dev, float scale, int8_t *q, cudaStream_t stream) {
  if (n <= 0) return PGB_OK;
  int64_t grid = (n + 4095) / 4096;  // 4 vectors of 4 elements per thread
  const int64_t cap = (int64_t)sm_count() * 32;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  quantize_i8_kernel<<<(unsigned)grid, 256, 0, stream>>>(x, n, absmax_dev, scale, q);
  count_launch();
  return check_launch("quantize_i8_kernel");
}

}  // namespace pgb
