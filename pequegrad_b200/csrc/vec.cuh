// 128-bit streaming loads / stores of V consecutive elements, widened to the
// compute type. The reference loads one element per thread per access
// (csrc/cuda/reduce.cuh:69, csrc/cuda/binary.cuh:34-37).
#pragma once
#include "common.cuh"

namespace pgb {

template <typename T, typename InT>
__device__ __forceinline__ T to_compute(InT x) { return (T)x; }
template <> __device__ __forceinline__ float to_compute<float, __half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_compute<float, __nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename OutT, typename T>
__device__ __forceinline__ OutT from_compute(T x) { return (OutT)x; }
template <> __device__ __forceinline__ __half from_compute<__half, float>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_compute<__nv_bfloat16, float>(float x) { return __float2bfloat16_rn(x); }

template <bool STREAM, typename P>
__device__ __forceinline__ P ld_sel(const P *p) {
  if constexpr (STREAM) return __ldcs(p);
  else return __ldg(p);
}

// p must be aligned to V * sizeof(InT) bytes (V = 4 halves is a 64-bit access).
template <typename T, typename InT, int V, bool STREAM>
__device__ __forceinline__ void load_vec_impl(const InT *p, T (&d)[V]) {
  if constexpr (V == 1) {
    d[0] = to_compute<T, InT>(ld_sel<STREAM>(p));
  } else if constexpr (sizeof(InT) == 4) {
    static_assert(V == 4, "128-bit load of 4-byte elements");
    const uint4 r = ld_sel<STREAM>(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      InT x;
      memcpy(&x, &w[e], 4);
      d[e] = to_compute<T, InT>(x);
    }
  } else if constexpr (sizeof(InT) == 2 && V == 4) {
    const uint2 r = ld_sel<STREAM>(reinterpret_cast<const uint2 *>(p));
    const uint32_t w[2] = {r.x, r.y};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      InT lo, hi;
      const uint16_t l16 = (uint16_t)(w[e] & 0xffffu), h16 = (uint16_t)(w[e] >> 16);
      memcpy(&lo, &l16, 2);
      memcpy(&hi, &h16, 2);
      d[2 * e] = to_compute<T, InT>(lo);
      d[2 * e + 1] = to_compute<T, InT>(hi);
    }
  } else if constexpr (sizeof(InT) == 2) {
    static_assert(V == 8, "128-bit load of 2-byte elements");
    const uint4 r = ld_sel<STREAM>(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      InT lo, hi;
      const uint16_t l16 = (uint16_t)(w[e] & 0xffffu), h16 = (uint16_t)(w[e] >> 16);
      memcpy(&lo, &l16, 2);
      memcpy(&hi, &h16, 2);
      d[2 * e] = to_compute<T, InT>(lo);
      d[2 * e + 1] = to_compute<T, InT>(hi);
    }
  } else {
    static_assert(sizeof(InT) == 8 && V == 2, "128-bit load of 8-byte elements");
    const double2 r = ld_sel<STREAM>(reinterpret_cast<const double2 *>(p));
    d[0] = (T)r.x;
    d[1] = (T)r.y;
  }
}

// read-once data: evict-first
template <typename T, typename InT, int V>
__device__ __forceinline__ void load_vec(const InT *p, T (&d)[V]) { load_vec_impl<T, InT, V, true>(p, d); }
// data every row re-reads (weights): keep it cached
template <typename T, typename InT, int V>
__device__ __forceinline__ void load_vec_cached(const InT *p, T (&d)[V]) { load_vec_impl<T, InT, V, false>(p, d); }

template <typename OutT, typename T, int V>
__device__ __forceinline__ void store_vec(OutT *p, const T (&s)[V]) {
  if constexpr (V == 1) {
    *p = from_compute<OutT, T>(s[0]);
  } else if constexpr (sizeof(OutT) == 4) {
    static_assert(V == 4, "128-bit store of 4-byte elements");
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const OutT x = from_compute<OutT, T>(s[e]);
      memcpy(&w[e], &x, 4);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  } else if constexpr (sizeof(OutT) == 2 && V == 4) {
    uint32_t w[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const OutT lo = from_compute<OutT, T>(s[2 * e]), hi = from_compute<OutT, T>(s[2 * e + 1]);
      uint16_t l16, h16;
      memcpy(&l16, &lo, 2);
      memcpy(&h16, &hi, 2);
      w[e] = (uint32_t)l16 | ((uint32_t)h16 << 16);
    }
    *reinterpret_cast<uint2 *>(p) = make_uint2(w[0], w[1]);
  } else if constexpr (sizeof(OutT) == 2) {
    static_assert(V == 8, "128-bit store of 2-byte elements");
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const OutT lo = from_compute<OutT, T>(s[2 * e]), hi = from_compute<OutT, T>(s[2 * e + 1]);
      uint16_t l16, h16;
      memcpy(&l16, &lo, 2);
      memcpy(&h16, &hi, 2);
      w[e] = (uint32_t)l16 | ((uint32_t)h16 << 16);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    static_assert(sizeof(OutT) == 8 && V == 2, "128-bit store of 8-byte elements");
    *reinterpret_cast<double2 *>(p) = make_double2((double)s[0], (double)s[1]);
  }
}

}  // namespace pgb
