/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * CPU restatement, in plain C, of the reference's CPU backend for the hot
 * path. Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs
 * may load this; the product (libpgb200.so) never does.
 *
 * Parity pin: every function here is checked bit-for-bit against the
 * reference's own header-only CPU templates compiled from their sources
 * (oracle/_ref/libpgref.so, built by oracle/build.py) and against the
 * torch-CPU comparisons the reference's tests make (tests/test_ops.py:20-80,
 * seed 1337); the vectors are committed under tests/golden/.
 * Functions with no reference counterpart (argmax as an index, the int8 path,
 * single-pass softmax / LayerNorm in fp16) say "parity unpinned" below.
 *
 * Strides are in BYTES, as in the reference's View (csrc/tensor.hpp:263-273).
 * dtype codes: 0 int32, 2 float32, 3 float64 (csrc/dtype.hpp:9-14).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

enum { ORC_SUM = 0, ORC_MAX = 1, ORC_MEAN = 2 };
enum { B_ADD, B_SUB, B_MUL, B_DIV, B_GT, B_LT, B_EQ, B_NEQ, B_GE, B_LE, B_POW, B_MAX };

/* ---------------------------------------------------------------------------
 * Single-axis reduce: csrc/cpu/reduce.hpp:11-55 (reduce_base_fn) with the
 * functors of csrc/cpu/reduce.hpp:57-86. The output is contiguous with the
 * reduced axis of extent 1. Accumulation is serial in axis order; max starts
 * from the LOWEST finite value, not -inf (reduce.hpp:68-78); mean divides the
 * sum by the extent at the end (reduce.hpp:82-86).
 * ------------------------------------------------------------------------- */
#define DEF_REDUCE(NAME, T, LOWEST)                                                          \
  static void NAME(const T *in, T *out, const int64_t *strides, const int64_t *shape,        \
                   int ndim, int axis, int op) {                                             \
    int64_t total_out = 1;                                                                   \
    for (int i = 0; i < ndim; i++)                                                           \
      if (i != axis) total_out *= shape[i];                                                  \
    const int64_t red = shape[axis];                                                         \
    _Pragma("omp parallel for") for (int64_t o = 0; o < total_out; o++) {                    \
      T accum = (op == ORC_MAX) ? (T)(LOWEST) : (T)0;                                        \
      for (int64_t i = 0; i < red; i++) {                                                    \
        int64_t rem = o, in_idx = 0;                                                         \
        for (int j = ndim - 1; j >= 0; j--) {                                                \
          if (j == axis) {                                                                   \
            in_idx += i * strides[j] / (int64_t)sizeof(T);                                   \
          } else {                                                                           \
            in_idx += (rem % shape[j]) * strides[j] / (int64_t)sizeof(T);                    \
            rem /= shape[j];                                                                 \
          }                                                                                  \
        }                                                                                    \
        const T el = in[in_idx];                                                             \
        if (op == ORC_MAX) accum = (accum < el) ? el : accum; /* std::max(a, b) */           \
        else accum = accum + el;                                                             \
      }                                                                                      \
      out[o] = (op == ORC_MEAN) ? (T)(accum / (int)red) : accum;                             \
    }                                                                                        \
  }

#include <float.h>
#include <limits.h>
DEF_REDUCE(reduce_f32, float, -FLT_MAX)
DEF_REDUCE(reduce_f64, double, -DBL_MAX)
DEF_REDUCE(reduce_i32, int32_t, INT_MIN)

ORC_API int orc_reduce_axis(const void *in, void *out, const int64_t *strides, const int64_t *shape, int ndim, int axis,
                            int op, int dtype) {
  switch (dtype) {
    case 2: reduce_f32((const float *)in, (float *)out, strides, shape, ndim, axis, op); return 0;
    case 3: reduce_f64((const double *)in, (double *)out, strides, shape, ndim, axis, op); return 0;
    case 0: reduce_i32((const int32_t *)in, (int32_t *)out, strides, shape, ndim, axis, op); return 0;
    default: return -2; /* "reduce_cpu not implemented for <dtype>", csrc/dispatch.hpp:38-44 */
  }
}

/* ---------------------------------------------------------------------------
 * Strided binary op: csrc/cpu/binary.hpp:29-56 (binary_op_ker) with the
 * lambdas of binary.hpp:70-83. Comparisons return 0/1 in the operand type.
 * ------------------------------------------------------------------------- */
#define DEF_BINARY(NAME, T, POWF)                                                            \
  static void NAME(const T *lhs, const T *rhs, T *res, const int64_t *ls, const int64_t *rs, \
                   const int64_t *os, const int64_t *shape, int ndim, int op) {              \
    int64_t total = 1;                                                                       \
    for (int i = 0; i < ndim; i++) total *= shape[i];                                        \
    _Pragma("omp parallel for") for (int64_t index = 0; index < total; index++) {            \
      int64_t ol = 0, or_ = 0, oo = 0, rem = index;                                          \
      for (int d = ndim - 1; d >= 0; d--) {                                                  \
        const int64_t c = rem % shape[d];                                                    \
        ol += c * ls[d] / (int64_t)sizeof(T);                                                \
        or_ += c * rs[d] / (int64_t)sizeof(T);                                               \
        oo += c * os[d] / (int64_t)sizeof(T);                                                \
        rem /= shape[d];                                                                     \
      }                                                                                      \
      const T a = lhs[ol], b = rhs[or_];                                                     \
      T r;                                                                                   \
      switch (op) {                                                                          \
        case B_ADD: r = a + b; break;                                                        \
        case B_SUB: r = a - b; break;                                                        \
        case B_MUL: r = a * b; break;                                                        \
        case B_DIV: r = a / b; break;                                                        \
        case B_GT: r = (T)(a > b); break;                                                    \
        case B_LT: r = (T)(a < b); break;                                                    \
        case B_EQ: r = (T)(a == b); break;                                                   \
        case B_NEQ: r = (T)(a != b); break;                                                  \
        case B_GE: r = (T)(a >= b); break;                                                   \
        case B_LE: r = (T)(a <= b); break;                                                   \
        case B_POW: r = (T)POWF(a, b); break;                                                \
        default: r = (a < b) ? b : a; break; /* std::max */                                  \
      }                                                                                      \
      res[oo] = r;                                                                           \
    }                                                                                        \
  }

DEF_BINARY(binary_f32, float, powf)
DEF_BINARY(binary_f64, double, pow)
DEF_BINARY(binary_i32, int32_t, pow)

ORC_API int orc_binary(const void *lhs, const void *rhs, void *res, const int64_t *ls, const int64_t *rs, const int64_t *os,
                       const int64_t *shape, int ndim, int op, int dtype) {
  switch (dtype) {
    case 2: binary_f32((const float *)lhs, (const float *)rhs, (float *)res, ls, rs, os, shape, ndim, op); return 0;
    case 3: binary_f64((const double *)lhs, (const double *)rhs, (double *)res, ls, rs, os, shape, ndim, op); return 0;
    case 0: binary_i32((const int32_t *)lhs, (const int32_t *)rhs, (int32_t *)res, ls, rs, os, shape, ndim, op); return 0;
    default: return -2;
  }
}

/* ---------------------------------------------------------------------------
 * where: csrc/cpu/ternary.hpp:11-43 with `a ? b : c` (csrc/cpu/ternary.cpp).
 * ------------------------------------------------------------------------- */
#define DEF_WHERE(NAME, T)                                                                   \
  static void NAME(const T *a, const T *b, const T *c, T *res, const int64_t *as,            \
                   const int64_t *bs, const int64_t *cs, const int64_t *os,                  \
                   const int64_t *shape, int ndim) {                                         \
    int64_t total = 1;                                                                       \
    for (int i = 0; i < ndim; i++) total *= shape[i];                                        \
    _Pragma("omp parallel for") for (int64_t index = 0; index < total; index++) {            \
      int64_t oa = 0, ob = 0, oc = 0, oo = 0, rem = index;                                   \
      for (int d = ndim - 1; d >= 0; d--) {                                                  \
        const int64_t k = rem % shape[d];                                                    \
        oa += k * as[d] / (int64_t)sizeof(T);                                                \
        ob += k * bs[d] / (int64_t)sizeof(T);                                                \
        oc += k * cs[d] / (int64_t)sizeof(T);                                                \
        oo += k * os[d] / (int64_t)sizeof(T);                                                \
        rem /= shape[d];                                                                     \
      }                                                                                      \
      res[oo] = a[oa] ? b[ob] : c[oc];                                                       \
    }                                                                                        \
  }
DEF_WHERE(where_f32, float)
DEF_WHERE(where_f64, double)
DEF_WHERE(where_i32, int32_t)

ORC_API int orc_where(const void *a, const void *b, const void *c, void *res, const int64_t *as, const int64_t *bs,
                      const int64_t *cs, const int64_t *os, const int64_t *shape, int ndim, int dtype) {
  switch (dtype) {
    case 2: where_f32(a, b, c, res, as, bs, cs, os, shape, ndim); return 0;
    case 3: where_f64(a, b, c, res, as, bs, cs, os, shape, ndim); return 0;
    case 0: where_i32(a, b, c, res, as, bs, cs, os, shape, ndim); return 0;
    default: return -2;
  }
}

/* ---------------------------------------------------------------------------
 * Dense unary exp / log: csrc/cpu/unary.cpp:14-18 walks nbytes/size elements
 * with csrc/cpu/unary.hpp:39-51 (scalar std::exp / std::log without AVX).
 * ------------------------------------------------------------------------- */
ORC_API int orc_unary(const void *in, void *out, int64_t n, int op /*0 exp 1 log*/, int dtype) {
  if (dtype == 2) {
    const float *x = in;
    float *y = out;
#pragma omp parallel for
    for (int64_t i = 0; i < n; i++) y[i] = op == 0 ? expf(x[i]) : logf(x[i]);
    return 0;
  }
  if (dtype == 3) {
    const double *x = in;
    double *y = out;
#pragma omp parallel for
    for (int64_t i = 0; i < n; i++) y[i] = op == 0 ? exp(x[i]) : log(x[i]);
    return 0;
  }
  return -2;
}

/* ---------------------------------------------------------------------------
 * Generic contiguous matmul: csrc/cpu/matmul.hpp:6-21 (matmul_ker<T>), serial
 * k loop per output. The reference's float/double specialisations call cblas
 * (matmul.hpp:23-43, OpenBLAS, version unpinned, absent here); this loop is
 * what the template computes for every other type and is the int32 oracle.
 * ------------------------------------------------------------------------- */
ORC_API void orc_matmul_f32(const float *lhs, const float *rhs, float *res, int64_t M, int64_t N, int64_t K, int64_t B) {
#pragma omp parallel for collapse(2)
  for (int64_t b = 0; b < B; b++)
    for (int64_t i = 0; i < M; i++)
      for (int64_t j = 0; j < N; j++) {
        float sum = 0;
        for (int64_t k = 0; k < K; k++) sum += lhs[b * M * K + i * K + k] * rhs[b * K * N + k * N + j];
        res[b * M * N + i * N + j] = sum;
      }
}

ORC_API void orc_matmul_i32(const int32_t *lhs, const int32_t *rhs, int32_t *res, int64_t M, int64_t N, int64_t K, int64_t B) {
#pragma omp parallel for collapse(2)
  for (int64_t b = 0; b < B; b++)
    for (int64_t i = 0; i < M; i++)
      for (int64_t j = 0; j < N; j++) {
        int32_t sum = 0;
        for (int64_t k = 0; k < K; k++) sum += lhs[b * M * K + i * K + k] * rhs[b * K * N + k * N + j];
        res[b * M * N + i * N + j] = sum;
      }
}

/* ---------------------------------------------------------------------------
 * argmax as an index — parity unpinned: the reference has only the Python
 * composite pequegrad/ops.py:968-978 (2-D, float result, ties summed). This
 * returns the FIRST position of the maximum along `axis`, int32, any rank.
 * ------------------------------------------------------------------------- */
ORC_API int orc_argmax_f32(const float *in, int32_t *out, const int64_t *strides, const int64_t *shape, int ndim, int axis) {
  int64_t total_out = 1;
  for (int i = 0; i < ndim; i++)
    if (i != axis) total_out *= shape[i];
  const int64_t red = shape[axis];
#pragma omp parallel for
  for (int64_t o = 0; o < total_out; o++) {
    int64_t rem = o, base = 0;
    for (int j = ndim - 1; j >= 0; j--) {
      if (j == axis) continue;
      base += (rem % shape[j]) * strides[j] / 4;
      rem /= shape[j];
    }
    float best = in[base];
    int32_t bi = 0;
    for (int64_t i = 1; i < red; i++) {
      const float v = in[base + i * strides[axis] / 4];
      if (v > best) { best = v; bi = (int32_t)i; }
    }
    out[o] = bi;
  }
  return 0;
}

/* ---------------------------------------------------------------------------
 * int8 quantised linear — parity unpinned: the reference has no int8 dtype
 * (csrc/dtype.hpp:9-14); its "quantized" MLP fake-quantises weights in fp32
 * (examples/quantized_mlp.py:28-34). The scheme below keeps that example's
 * symmetric scaling (max|.| floored at 1e-6, scaled to 127) but with real
 * int8 storage, round-half-to-even and int32 accumulation.
 * ------------------------------------------------------------------------- */
ORC_API float orc_absmax_f32(const float *x, int64_t n) {
  float m = 0.f;
#pragma omp parallel for reduction(max : m)
  for (int64_t i = 0; i < n; i++) {
    const float a = fabsf(x[i]);
    if (a > m) m = a;
  }
  return m;
}

/* q = clip(rint(x / scale), -127, 127), scale = max(absmax, 1e-6) / 127 */
ORC_API void orc_quantize_i8(const float *x, int8_t *q, int64_t n, float scale) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; i++) {
    float r = rintf(x[i] / scale);
    if (r > 127.f) r = 127.f;
    if (r < -127.f) r = -127.f;
    q[i] = (int8_t)r;
  }
}

/* acc[m,n] = sum_k a[m,k] * w[n,k]  (both K-major), int32 exact */
ORC_API void orc_gemm_i8(const int8_t *a, const int8_t *w, int32_t *acc, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for
  for (int64_t m = 0; m < M; m++)
    for (int64_t n = 0; n < N; n++) {
      int32_t s = 0;
      for (int64_t k = 0; k < K; k++) s += (int32_t)a[m * K + k] * (int32_t)w[n * K + k];
      acc[m * N + n] = s;
    }
}

/* out[m,n] = act(acc * (a_scale * w_scale[n]) + bias[n]) in fp32, that association */
ORC_API void orc_dequant_bias_act(const int32_t *acc, const float *w_scale, float a_scale, const float *bias, int relu,
                                  float *out, int64_t M, int64_t N) {
#pragma omp parallel for
  for (int64_t m = 0; m < M; m++)
    for (int64_t n = 0; n < N; n++) {
      const float s = a_scale * w_scale[n];
      float v = (float)acc[m * N + n] * s;
      if (bias) v = v + bias[n];
      if (relu) v = (v > 0.f) ? v : 0.f; /* max(x, 0), pequegrad/tensor.py:162-163 */
      out[m * N + n] = v;
    }
}

/* ---------------------------------------------------------------------------
 * Row softmax and LayerNorm, following the composites op by op in fp32
 * (pequegrad/ops.py:259-267; pequegrad/ops.py:515-551 with the biased
 * variance of ops.py:480-501). Contiguous rows. causal_rows > 0 masks column
 * j > (row % causal_rows). For the fp16 cases the caller rounds the inputs to
 * half first and the outputs afterwards — parity unpinned for fp16 (the
 * reference cannot run a 1024-wide fp16 softmax at all).
 * ------------------------------------------------------------------------- */
ORC_API void orc_softmax_rows_f32(const float *x, float *y, int64_t rows, int64_t C, int64_t causal_rows) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; r++) {
    const float *xr = x + r * C;
    float *yr = y + r * C;
    int64_t L = C;
    if (causal_rows > 0) { L = (r % causal_rows) + 1; if (L > C) L = C; }
    float m = -FLT_MAX;
    for (int64_t c = 0; c < L; c++) m = (m < xr[c]) ? xr[c] : m;
    float s = 0.f;
    for (int64_t c = 0; c < L; c++) { yr[c] = expf(xr[c] - m); s += yr[c]; }
    for (int64_t c = 0; c < L; c++) yr[c] = yr[c] / s;
    for (int64_t c = L; c < C; c++) yr[c] = 0.f;
  }
}

ORC_API void orc_layernorm_rows_f32(const float *x, const float *gamma, const float *beta, float eps, float *y, int64_t rows,
                                    int64_t C) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; r++) {
    const float *xr = x + r * C;
    float *yr = y + r * C;
    float s = 0.f;
    for (int64_t c = 0; c < C; c++) s += xr[c];
    const float mean = s / (int)C;
    float q = 0.f;
    for (int64_t c = 0; c < C; c++) { const float d = xr[c] - mean; q += powf(d, 2.0f); }
    const float var = q / (float)C;
    const float sd = powf(var + eps, 0.5f);
    for (int64_t c = 0; c < C; c++) {
      float v = (xr[c] - mean) / sd;
      if (gamma) v = v * gamma[c];
      if (beta) v = v + beta[c];
      yr[c] = v;
    }
  }
}
