// Single-kernel row softmax and LayerNorm.
//
// The reference computes both as chains of separate kernels with full-size
// intermediates: softmax = max_reduce, sub, exp, (again sub, exp), sum, div
// (pequegrad/ops.py:259-267); layer_norm = mean, var (mean, sub, pow, sum,
// div), add eps, pow 0.5, sub, div, mul, add (pequegrad/ops.py:515-551,
// 480-501). Here a warp keeps its row in registers: one read and one write of
// the tensor. The arithmetic follows the composites step by step (true
// division, biased variance, eps added before the square root).
#include <type_traits>

#include "reduce_common.cuh"
#include "vec.cuh"

namespace pgb {

struct RowsParams {
  const void *x;
  void *y;
  const void *gamma, *beta;
  int64_t rows, C;
  int64_t causal_rows;  // > 0: causal mask with this many rows per matrix
  float eps;
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

// 2^t on the special-function unit (2 ulp); 2^(-inf) = 0, so masked elements need no special case.
__device__ __forceinline__ float ex2_approx(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
// e^d for d <= 0 as 2^(d * log2 e). The rounding of the product adds |d| * 1e-7 relative error,
// below 2e-6 for |d| < 20.
__device__ __forceinline__ float exp_nonpos(float d) { return ex2_approx(d * 1.4426950408889634f); }

// One warp per row, the row held in NV vectors of V elements per lane. With a causal mask the
// vectors that lie wholly above the diagonal are neither loaded nor exponentiated (the test is
// warp-uniform); they are stored as zeros.
template <typename IoT, int V, int NV>
__global__ void __launch_bounds__(256, 5) softmax_warp_kernel(const __grid_constant__ RowsParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const IoT *xr = (const IoT *)p.x + row * p.C;
  IoT *yr = (IoT *)p.y + row * p.C;
  const int C = (int)p.C;  // at most 16 * 32 * V here
  // number of columns that take part (the rest are masked out)
  int L = C;
  if (p.causal_rows > 0) {
    const int64_t r = p.rows <= 0xffffffffLL ? (int64_t)((uint32_t)row % (uint32_t)p.causal_rows) : row % p.causal_rows;
    L = (int)min((int64_t)C, r + 1);
  }
  float v[NV][V];
  float m = -INFINITY;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int c = (u * 32 + lane) * V;
    if (c < L) {
      load_vec<float, IoT, V>(xr + c, v[u]);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        if (c + e >= L) v[u][e] = -INFINITY;
        m = fmaxf(m, v[u][e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) v[u][e] = -INFINITY;
    }
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    if (u * 32 * V < L) {  // warp-uniform
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float ex = exp_nonpos(v[u][e] - m);
        v[u][e] = ex;
        s += ex;
      }
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) v[u][e] = 0.f;
    }
  }
  s = warp_sum(s);
  const float inv = 1.0f / s;  // v * (1/s) is within 1 ulp of the composite's v / s
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int c = (u * 32 + lane) * V;
    if (c < C) {
      float o[V];
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = v[u][e] * inv;
      store_vec<IoT, float, V>(yr + c, o);
    }
  }
}

// 16-bit rows of up to 16 * 256 columns: the row stays in its packed form, 4 registers per 8 elements, so that
// six CTAs fit on an SM (the fp32-register kernel above ran at 62 % occupancy and was bound by instruction issue
// and load latency, not by DRAM). Max on packed pairs (exact), exp in fp32 as one fused multiply-add and one
// ex2.approx per element, the sum in fp32; the unnormalised p in (0, 1] is packed back to 16 bits and scaled by
// 1 / sum with a packed multiply: three 16-bit roundings, ~1.5e-3 relative, inside the 2e-2 of 16-bit outputs.
template <typename IoT, int NV>
__global__ void __launch_bounds__(256, (NV <= 4 ? 6 : (NV <= 8 ? 4 : 2))) softmax_warp16_kernel(const __grid_constant__ RowsParams p) {
  constexpr bool IS_H = std::is_same<IoT, __half>::value;
  using T2 = typename std::conditional<IS_H, __half2, __nv_bfloat162>::type;
  constexpr uint32_t NINF = IS_H ? 0xFC00u : 0xFF80u, NINF2 = NINF | (NINF << 16);
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const IoT *xr = (const IoT *)p.x + row * p.C;
  IoT *yr = (IoT *)p.y + row * p.C;
  const int C = (int)p.C;
  int L = C;
  if (p.causal_rows > 0) {
    const int64_t r = p.rows <= 0xffffffffLL ? (int64_t)((uint32_t)row % (uint32_t)p.causal_rows) : row % p.causal_rows;
    L = (int)min((int64_t)C, r + 1);
  }
  uint32_t w[NV][4];
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int c = (u * 32 + lane) * 8;
    uint4 r = make_uint4(NINF2, NINF2, NINF2, NINF2);
    if (c < L) r = __ldcs(reinterpret_cast<const uint4 *>(xr + c));
    w[u][0] = r.x; w[u][1] = r.y; w[u][2] = r.z; w[u][3] = r.w;
    if (c < L && c + 8 > L) {  // the one lane whose vector straddles the mask
      const int n = L - c;     // 1..7 elements take part
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int vj = n - 2 * j;
        if (vj <= 0) w[u][j] = NINF2;
        else if (vj == 1) w[u][j] = (w[u][j] & 0xffffu) | (NINF << 16);
      }
    }
  }
  T2 m2;
  {
    const uint32_t init = NINF2;
    m2 = *reinterpret_cast<const T2 *>(&init);
  }
#pragma unroll
  for (int u = 0; u < NV; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, *reinterpret_cast<const T2 *>(&w[u][j]));
  float2 mf;
  if constexpr (IS_H) mf = __half22float2(m2);
  else mf = __bfloat1622float2(m2);
  const float m = warp_max(fmaxf(mf.x, mf.y));
  const float ml = m * 1.4426950408889634f;
  float s = 0.f;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    if (u * 256 < L) {  // warp-uniform: vectors wholly above the diagonal are not exponentiated
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f;
        if constexpr (IS_H) f = __half22float2(*reinterpret_cast<const T2 *>(&w[u][j]));
        else f = __bfloat1622float2(*reinterpret_cast<const T2 *>(&w[u][j]));
        const float p0 = ex2_approx(fmaf(f.x, 1.4426950408889634f, -ml)), p1 = ex2_approx(fmaf(f.y, 1.4426950408889634f, -ml));
        s += p0 + p1;
        T2 pk;
        if constexpr (IS_H) pk = __floats2half2_rn(p0, p1);
        else pk = __floats2bfloat162_rn(p0, p1);
        w[u][j] = *reinterpret_cast<const uint32_t *>(&pk);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) w[u][j] = 0u;
    }
  }
  s = warp_sum(s);
  const float inv = 1.0f / s;
  T2 inv2;
  if constexpr (IS_H) inv2 = __floats2half2_rn(inv, inv);
  else inv2 = __floats2bfloat162_rn(inv, inv);
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int c = (u * 32 + lane) * 8;
    if (c < C) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const T2 q = __hmul2(*reinterpret_cast<const T2 *>(&w[u][j]), inv2);
        o[j] = *reinterpret_cast<const uint32_t *>(&q);
      }
      *reinterpret_cast<uint4 *>(yr + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Any row length / alignment: one CTA per row, three passes over the row
// (the repeats are served by L1/L2).
template <typename IoT>
__global__ void __launch_bounds__(256) softmax_cta_kernel(const __grid_constant__ RowsParams p) {
  __shared__ float red[8];
  __shared__ float bc;
  const int64_t row = blockIdx.x;
  const IoT *xr = (const IoT *)p.x + row * p.C;
  IoT *yr = (IoT *)p.y + row * p.C;
  int64_t L = p.C;
  if (p.causal_rows > 0) L = min(p.C, (row % p.causal_rows) + 1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -INFINITY;
  for (int64_t c = threadIdx.x; c < L; c += 256) m = fmaxf(m, to_compute<float, IoT>(xr[c]));
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  if (threadIdx.x == 0) { float t = red[0]; for (int i = 1; i < 8; ++i) t = fmaxf(t, red[i]); bc = t; }
  __syncthreads();
  m = bc;
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < L; c += 256) {
    const float xv = to_compute<float, IoT>(xr[c]);
    s += exp_nonpos(xv - m);
  }
  s = warp_sum(s);
  __syncthreads();
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.f; for (int i = 0; i < 8; ++i) t += red[i]; bc = t; }
  __syncthreads();
  s = 1.0f / bc;
  for (int64_t c = threadIdx.x; c < p.C; c += 256) {
    float o = 0.f;
    if (c < L) o = exp_nonpos(to_compute<float, IoT>(xr[c]) - m) * s;
    yr[c] = from_compute<IoT, float>(o);
  }
}

template <typename IoT, int V, int NV>
__global__ void __launch_bounds__(256) layernorm_warp_kernel(const __grid_constant__ RowsParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const int C = (int)p.C;  // at most 16 * 32 * V here: 32-bit column arithmetic
  const IoT *xr = (const IoT *)p.x + row * C + lane * V;
  IoT *yr = (IoT *)p.y + row * C + lane * V;
  // vector u of this lane covers columns (u * 32 + lane) * V ..: inside the row for u < nu (C is a multiple of V)
  const int nu = max(0, (C / V - lane + 31) >> 5);
  float v[NV][V];
  float s = 0.f;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    if (u < nu) {
      load_vec<float, IoT, V>(xr + u * 32 * V, v[u]);
#pragma unroll
      for (int e = 0; e < V; ++e) s += v[u][e];
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) v[u][e] = 0.f;
    }
  }
  const float n = (float)C;
  const float mean = warp_sum(s) / n;
  float q = 0.f;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    if (u < nu) {
#pragma unroll
      for (int e = 0; e < V; ++e) {
        v[u][e] = v[u][e] - mean;
        q += v[u][e] * v[u][e];
      }
    }
  }
  const float var = warp_sum(q) / n;
  const float rsd = 1.0f / sqrtf(var + p.eps);  // d * (1/sd) is within 1 ulp of the composite's d / sd
  const IoT *gp = p.gamma ? (const IoT *)p.gamma + lane * V : nullptr;
  const IoT *bp = p.beta ? (const IoT *)p.beta + lane * V : nullptr;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    if (u < nu) {
      float o[V];
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = v[u][e] * rsd;
      if (gp) {
        float g[V];
        load_vec_cached<float, IoT, V>(gp + u * 32 * V, g);
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] = o[e] * g[e];
      }
      if (bp) {
        float b[V];
        load_vec_cached<float, IoT, V>(bp + u * 32 * V, b);
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] = o[e] + b[e];
      }
      store_vec<IoT, float, V>(yr + u * 32 * V, o);
    }
  }
}

// LayerNorm for 16-bit rows of up to 16 * 256 columns, same idea as softmax_warp16_kernel: the row stays packed
// (4 registers per 8 elements) and is widened on the fly in each of the three passes, which leaves room for six CTAs
// per SM; squared deviations and the affine output use fused multiply-adds (fp32 statistics, 16-bit tolerance).
template <typename IoT, int NV>
__global__ void __launch_bounds__(256, (NV <= 4 ? 6 : (NV <= 8 ? 4 : 2))) layernorm_warp16_kernel(const __grid_constant__ RowsParams p) {
  constexpr bool IS_H = std::is_same<IoT, __half>::value;
  using T2 = typename std::conditional<IS_H, __half2, __nv_bfloat162>::type;
  auto widen = [](uint32_t w) -> float2 {
    if constexpr (IS_H) return __half22float2(*reinterpret_cast<const T2 *>(&w));
    else return __bfloat1622float2(*reinterpret_cast<const T2 *>(&w));
  };
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const int C = (int)p.C;
  const IoT *xr = (const IoT *)p.x + row * C;
  IoT *yr = (IoT *)p.y + row * C;
  uint32_t w[NV][4];
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int c = (u * 32 + lane) * 8;
    uint4 r = make_uint4(0, 0, 0, 0);
    if (c < C) r = __ldcs(reinterpret_cast<const uint4 *>(xr + c));
    w[u][0] = r.x; w[u][1] = r.y; w[u][2] = r.z; w[u][3] = r.w;
  }
  float s = 0.f;
#pragma unroll
  for (int u = 0; u < NV; ++u)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = widen(w[u][j]);  // columns beyond C are zeros
      s += f.x + f.y;
    }
  const float n = (float)C;
  const float mean = warp_sum(s) / n;
  float q = 0.f;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    if ((u * 32 + lane) * 8 < C) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = widen(w[u][j]);
        const float d0 = f.x - mean, d1 = f.y - mean;
        q = fmaf(d0, d0, q);
        q = fmaf(d1, d1, q);
      }
    }
  }
  const float var = warp_sum(q) / n;
  const float rsd = 1.0f / sqrtf(var + p.eps);
  const float nmr = -mean * rsd;  // (x - mean) * rsd = x * rsd + nmr
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int c = (u * 32 + lane) * 8;
    if (c < C) {
      uint4 g4 = make_uint4(0, 0, 0, 0), b4 = g4;
      if (p.gamma) g4 = __ldg(reinterpret_cast<const uint4 *>((const IoT *)p.gamma + c));
      if (p.beta) b4 = __ldg(reinterpret_cast<const uint4 *>((const IoT *)p.beta + c));
      const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, bw[4] = {b4.x, b4.y, b4.z, b4.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = widen(w[u][j]);
        float y0 = fmaf(f.x, rsd, nmr), y1 = fmaf(f.y, rsd, nmr);
        if (p.gamma) { const float2 g = widen(gw[j]); y0 *= g.x; y1 *= g.y; }
        if (p.beta) { const float2 b = widen(bw[j]); y0 += b.x; y1 += b.y; }
        T2 pk;
        if constexpr (IS_H) pk = __floats2half2_rn(y0, y1);
        else pk = __floats2bfloat162_rn(y0, y1);
        o[j] = *reinterpret_cast<const uint32_t *>(&pk);
      }
      *reinterpret_cast<uint4 *>(yr + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

template <typename IoT>
__global__ void __launch_bounds__(256) layernorm_cta_kernel(const __grid_constant__ RowsParams p) {
  __shared__ float red[8];
  __shared__ float bc;
  const int64_t row = blockIdx.x;
  const IoT *xr = (const IoT *)p.x + row * p.C;
  IoT *yr = (IoT *)p.y + row * p.C;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float n = (float)p.C;
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < p.C; c += 256) s += to_compute<float, IoT>(xr[c]);
  s = warp_sum(s);
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.f; for (int i = 0; i < 8; ++i) t += red[i]; bc = t / n; }
  __syncthreads();
  const float mean = bc;
  float q = 0.f;
  for (int64_t c = threadIdx.x; c < p.C; c += 256) { const float d = to_compute<float, IoT>(xr[c]) - mean; q += d * d; }
  q = warp_sum(q);
  __syncthreads();
  if (lane == 0) red[warp] = q;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.f; for (int i = 0; i < 8; ++i) t += red[i]; bc = sqrtf(t / n + p.eps); }
  __syncthreads();
  const float sd = bc;
  for (int64_t c = threadIdx.x; c < p.C; c += 256) {
    float o = (to_compute<float, IoT>(xr[c]) - mean) / sd;
    if (p.gamma) o = o * to_compute<float, IoT>(((const IoT *)p.gamma)[c]);
    if (p.beta) o = o + to_compute<float, IoT>(((const IoT *)p.beta)[c]);
    yr[c] = from_compute<IoT, float>(o);
  }
}

// ---------------------------------------------------------------------------
static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename IoT, bool SOFTMAX>
static int rows_launch(const RowsParams &p, cudaStream_t stream) {
  constexpr int V = 16 / (int)sizeof(IoT);
  const bool vec = (p.C % V) == 0 && aligned16(p.x) && aligned16(p.y) && (!p.gamma || aligned16(p.gamma)) && (!p.beta || aligned16(p.beta));
  const int64_t per_lane_vecs = (p.C + 32 * V - 1) / (32 * V);
  const unsigned wgrid = (unsigned)((p.rows + 7) / 8);
  if (p.rows > 2147483647LL * 8) return PGB_ERR_UNSUPPORTED;
  const char *name = SOFTMAX ? "softmax_warp_kernel" : "layernorm_warp_kernel";
#define PGB_ROWS_CASE(NV)                                                                   \
  if constexpr (SOFTMAX && sizeof(IoT) == 2) softmax_warp16_kernel<IoT, NV><<<wgrid, 256, 0, stream>>>(p); \
  else if constexpr (SOFTMAX) softmax_warp_kernel<IoT, V, NV><<<wgrid, 256, 0, stream>>>(p); \
  else if constexpr (sizeof(IoT) == 2) layernorm_warp16_kernel<IoT, NV><<<wgrid, 256, 0, stream>>>(p); \
  else layernorm_warp_kernel<IoT, V, NV><<<wgrid, 256, 0, stream>>>(p)
  if (vec && per_lane_vecs <= 16) {
    if (per_lane_vecs <= 1) { PGB_ROWS_CASE(1); }
    else if (per_lane_vecs <= 2) { PGB_ROWS_CASE(2); }
    else if (per_lane_vecs <= 3) { PGB_ROWS_CASE(3); }
    else if (per_lane_vecs <= 4) { PGB_ROWS_CASE(4); }
    else if (per_lane_vecs <= 6) { PGB_ROWS_CASE(6); }
    else if (per_lane_vecs <= 8) { PGB_ROWS_CASE(8); }
    else { PGB_ROWS_CASE(16); }
  } else {
    name = SOFTMAX ? "softmax_cta_kernel" : "layernorm_cta_kernel";
    if (SOFTMAX) softmax_cta_kernel<IoT><<<(unsigned)p.rows, 256, 0, stream>>>(p);
    else layernorm_cta_kernel<IoT><<<(unsigned)p.rows, 256, 0, stream>>>(p);
  }
#undef PGB_ROWS_CASE
  count_launch();
  return check_launch(name);
}

static int rows_common(const pgb_tensor *x, const pgb_tensor *y, const char *what, RowsParams &p) {
  if (!x || !y) { set_error(std::string(what) + ": null tensor"); return PGB_ERR_INVALID_ARG; }
  if (x->ndim < 1 || x->ndim > PGB_MAX_DIMS || y->ndim != x->ndim) { set_error(std::string(what) + ": bad rank"); return PGB_ERR_INVALID_ARG; }
  for (int d = 0; d < x->ndim; ++d)
    if (x->shape[d] != y->shape[d]) { set_error(std::string(what) + ": input and output shapes differ"); return PGB_ERR_INVALID_ARG; }
  if (x->dtype != y->dtype) { set_error(std::string(what) + ": input and output dtypes differ"); return PGB_ERR_INVALID_ARG; }
  if (x->dtype != PGB_F32 && x->dtype != PGB_F16 && x->dtype != PGB_BF16) {
    set_error(std::string(what) + " not implemented for " + dtype_name(x->dtype));
    return PGB_ERR_UNSUPPORTED;
  }
  if (!is_contiguous(*x) || !is_contiguous(*y)) { set_error(std::string(what) + ": tensors must be contiguous"); return PGB_ERR_UNSUPPORTED; }
  p = RowsParams{};
  p.x = x->data;
  p.y = y->data;
  p.C = x->shape[x->ndim - 1];
  p.rows = p.C ? numel_of(*x) / p.C : 0;
  return PGB_OK;
}

int run_softmax_rows(const pgb_tensor *x, const pgb_tensor *y, int causal, cudaStream_t stream) {
  RowsParams p;
  int st = rows_common(x, y, "softmax", p);
  if (st != PGB_OK) return st;
  if (causal) {
    if (x->ndim < 2) { set_error("softmax: a causal mask needs at least 2 dims"); return PGB_ERR_INVALID_ARG; }
    p.causal_rows = x->shape[x->ndim - 2];
  }
  if (p.rows == 0 || p.C == 0) return PGB_OK;
  if (x->dtype == PGB_F32) return rows_launch<float, true>(p, stream);
  if (x->dtype == PGB_F16) return rows_launch<__half, true>(p, stream);
  return rows_launch<__nv_bfloat16, true>(p, stream);
}

int run_layernorm_rows(const pgb_tensor *x, const pgb_tensor *gamma, const pgb_tensor *beta, float eps, const pgb_tensor *y,
                       cudaStream_t stream) {
  RowsParams p;
  int st = rows_common(x, y, "layer_norm", p);
  if (st != PGB_OK) return st;
  for (const pgb_tensor *t : {gamma, beta}) {
    if (!t) continue;
    if (t->dtype != x->dtype || numel_of(*t) != p.C || !is_contiguous(*t)) {
      set_error("layer_norm: weight and bias must be contiguous, of the input dtype and of the normalised length");
      return PGB_ERR_INVALID_ARG;
    }
  }
  p.gamma = gamma ? gamma->data : nullptr;
  p.beta = beta ? beta->data : nullptr;
  p.eps = eps;
  if (p.rows == 0 || p.C == 0) return PGB_OK;
  if (x->dtype == PGB_F32) return rows_launch<float, false>(p, stream);
  if (x->dtype == PGB_F16) return rows_launch<__half, false>(p, stream);
  return rows_launch<__nv_bfloat16, false>(p, stream);
}

// ---------------------------------------------------------------------------
// Token + position embedding: out[r, :] = wte[ids[r], :] + wpe[r % T, :].
// Replaces the Select-with-index-tensor gather plus the add of
// pequegrad/modules.py:329-337 and examples/gpt2.py:365-372. One warp per row,
// 128-bit loads; an id outside [0, V) yields a zero row instead of a wild read.
template <typename IoT>
__global__ void __launch_bounds__(256) embedding_rows_kernel(const int *__restrict__ ids, const IoT *__restrict__ wte,
                                                             const IoT *__restrict__ wpe, IoT *__restrict__ out, int64_t rows, int64_t C,
                                                             int64_t V, int64_t T) {
  constexpr int VEC = 16 / (int)sizeof(IoT);
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int id = __ldg(ids + row);
  const bool ok = id >= 0 && id < V;
  const IoT *te = wte + (int64_t)(ok ? id : 0) * C;
  const IoT *pe = wpe ? wpe + (row % T) * C : nullptr;
  IoT *o = out + row * C;
  for (int64_t c = (int64_t)lane * VEC; c < C; c += 32 * VEC) {
    float a[VEC], b[VEC];
    load_vec_cached<float, IoT, VEC>(te + c, a);
    if (pe) load_vec_cached<float, IoT, VEC>(pe + c, b);
#pragma unroll
    for (int e = 0; e < VEC; ++e) a[e] = ok ? (pe ? a[e] + b[e] : a[e]) : 0.f;
    store_vec<IoT, float, VEC>(o + c, a);
  }
}

int run_embedding_rows(const pgb_tensor *ids, const pgb_tensor *wte, const pgb_tensor *wpe, int64_t T, const pgb_tensor *out,
                       cudaStream_t stream) {
  if (!ids || !wte || !out) { set_error("embedding: null tensor"); return PGB_ERR_INVALID_ARG; }
  if (ids->dtype != PGB_I32 || !is_contiguous(*ids)) { set_error("embedding: ids must be contiguous int32"); return PGB_ERR_INVALID_ARG; }
  if (wte->ndim != 2 || !is_contiguous(*wte) || !is_contiguous(*out) || out->dtype != wte->dtype) {
    set_error("embedding: the table must be a contiguous [V, C] matrix and the output of its dtype");
    return PGB_ERR_INVALID_ARG;
  }
  if (wte->dtype != PGB_F16 && wte->dtype != PGB_F32 && wte->dtype != PGB_BF16) {
    set_error(std::string("embedding not implemented for ") + dtype_name(wte->dtype));
    return PGB_ERR_UNSUPPORTED;
  }
  const int64_t rows = numel_of(*ids), V = wte->shape[0], C = wte->shape[1];
  if (numel_of(*out) != rows * C) { set_error("embedding: output shape does not match"); return PGB_ERR_INVALID_ARG; }
  if (wpe && (wpe->ndim != 2 || wpe->shape[1] != C || wpe->shape[0] < T || wpe->dtype != wte->dtype || !is_contiguous(*wpe) || T <= 0)) {
    set_error("embedding: the position table must be [>= T, C] of the same dtype");
    return PGB_ERR_INVALID_ARG;
  }
  const int es = dtype_size(wte->dtype);
  if ((C * es) % 16 || (reinterpret_cast<uintptr_t>(wte->data) & 15) || (reinterpret_cast<uintptr_t>(out->data) & 15) ||
      (wpe && (reinterpret_cast<uintptr_t>(wpe->data) & 15))) {
    set_error("embedding: rows must be 16-byte aligned");
    return PGB_ERR_UNSUPPORTED;
  }
  if (rows == 0) return PGB_OK;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  const int *idp = (const int *)ids->data;
  if (wte->dtype == PGB_F32)
    embedding_rows_kernel<float><<<grid, 256, 0, stream>>>(idp, (const float *)wte->data, wpe ? (const float *)wpe->data : nullptr, (float *)out->data, rows, C, V, T > 0 ? T : 1);
  else if (wte->dtype == PGB_F16)
    embedding_rows_kernel<__half><<<grid, 256, 0, stream>>>(idp, (const __half *)wte->data, wpe ? (const __half *)wpe->data : nullptr, (__half *)out->data, rows, C, V, T > 0 ? T : 1);
  else
    embedding_rows_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(idp, (const __nv_bfloat16 *)wte->data, wpe ? (const __nv_bfloat16 *)wpe->data : nullptr, (__nv_bfloat16 *)out->data, rows, C, V, T > 0 ? T : 1);
  count_launch();
  return check_launch("embedding_rows_kernel");
}

}  // namespace pgb
