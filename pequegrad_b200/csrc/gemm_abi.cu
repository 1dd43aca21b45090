// extern "C" entry points of the tensor-core GEMMs and of the dynamic int8
// activation quantisation. Validation and view handling only; the kernels are
// in gemm_sm100.cu.
#include <string>

#include "gemm.hpp"
#include "reduce_common.cuh"

namespace pgb {

static bool device_present() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    set_error("no CUDA device: this library has no CPU fallback");
    return false;
  }
  return true;
}

// Views the dims [lo, hi) of t as one dim: count and element stride. False if they do not merge.
static bool merge_dims(const pgb_tensor &t, int lo, int hi, int64_t *count, int64_t *stride) {
  const int es = dtype_size(t.dtype);
  int64_t cnt = 1, str = 0;
  bool have = false;
  for (int d = hi - 1; d >= lo; --d) {
    if (t.shape[d] == 1) continue;
    const int64_t s = t.stride_bytes[d] / es;
    if (!have) { str = s; cnt = t.shape[d]; have = true; }
    else {
      if (s != str * cnt) return false;
      cnt *= t.shape[d];
    }
  }
  *count = cnt;
  *stride = have ? str : 0;
  return true;
}
static bool merge_leading(const pgb_tensor &t, int nlead, int64_t *count, int64_t *stride) { return merge_dims(t, 0, nlead, count, stride); }

// A row-major-like 2-D (+ batch) operand: rows x cols with cols contiguous.
struct Mat {
  const void *ptr;
  int64_t rows, cols, ld, batch, batch_stride;
};

// Interprets t as [batch..., rows, cols] with the LAST dim contiguous.
static std::string as_mat(const pgb_tensor &t, const char *what, Mat &m, bool need_one_batch = true) {
  const int es = dtype_size(t.dtype);
  if (es == 0) return std::string("matmul: unknown dtype of ") + what;
  if (t.ndim < 2) return std::string("matmul: ") + what + " must have at least 2 dims";
  for (int d = 0; d < t.ndim; ++d)
    if (t.stride_bytes[d] % es || t.stride_bytes[d] < 0) return std::string("matmul: bad stride in ") + what;
  const int nd = t.ndim;
  m.ptr = t.data;
  m.rows = t.shape[nd - 2];
  m.cols = t.shape[nd - 1];
  if (m.cols > 1 && t.stride_bytes[nd - 1] != es) return std::string("matmul: ") + what + " must be contiguous along its contraction dim";
  m.ld = t.stride_bytes[nd - 2] / es;
  if (m.rows <= 1 && m.ld == 0) m.ld = m.cols;
  m.batch = 1;
  m.batch_stride = 0;
  if (need_one_batch && !merge_leading(t, nd - 2, &m.batch, &m.batch_stride))
    return std::string("matmul: batch dims of ") + what + " do not form one stride";
  return "";
}

// True if the [.., rows, K] view can feed the TMA loads as it is: K contiguous, base and every pitch 16-byte aligned.
static bool tma_ready(const pgb_tensor &t) {
  const int es = dtype_size(t.dtype), nd = t.ndim;
  if (reinterpret_cast<uintptr_t>(t.data) & 15) return false;
  if (t.shape[nd - 1] > 1 && t.stride_bytes[nd - 1] != es) return false;
  for (int d = 0; d < nd - 1; ++d)
    if (t.shape[d] > 1 && (t.stride_bytes[d] % 16 || t.stride_bytes[d] <= 0)) return false;
  return true;
}

// Describes a packed copy [lead..., rows, K] with row pitch Kp at `ptr` (contiguous over the leading dims).
static pgb_tensor packed_view(const pgb_tensor &t, void *ptr, int64_t Kp) {
  pgb_tensor v = t;
  const int es = dtype_size(t.dtype), nd = t.ndim;
  v.data = ptr;
  int64_t pitch = es;
  v.stride_bytes[nd - 1] = pitch;
  pitch *= Kp;
  for (int d = nd - 2; d >= 0; --d) {
    v.stride_bytes[d] = pitch;
    pitch *= t.shape[d];
  }
  return v;
}

// fp32 matmul: both operands are re-laid-out as K-major [big | big | small] / [big | small | big] splits
// (gemm_pack.cu) in a stream-ordered scratch buffer, then one tf32 GEMM of contraction length 3 * Kp runs.
// Any strides are accepted for a and b, since they are packed anyway.
static int matmul_f32(const pgb_tensor *a, const pgb_tensor *b, const pgb_tensor *bias, int act, float alpha, const pgb_tensor *residual,
                      const pgb_tensor *out, cudaStream_t stream) {
  if (a->ndim < 2 || b->ndim < 2 || out->ndim != a->ndim) { set_error("matmul: operands need at least 2 dims and the output the rank of a"); return PGB_ERR_INVALID_ARG; }
  const int nla = a->ndim - 2;
  if (nla > 6) { set_error("matmul: at most 6 batch dims"); return PGB_ERR_UNSUPPORTED; }
  const int64_t M = a->shape[nla], K = a->shape[nla + 1], N = b->shape[b->ndim - 1];
  if (b->shape[b->ndim - 2] != K) { set_error("matmul: contraction dims differ"); return PGB_ERR_INVALID_ARG; }
  const bool shared_b = b->ndim == 2;
  if (!shared_b && b->ndim != a->ndim) { set_error("matmul: batch dims differ"); return PGB_ERR_INVALID_ARG; }
  int64_t nbatch = 1;
  for (int d = 0; d < nla; ++d) {
    if (out->shape[d] != a->shape[d] || (!shared_b && b->shape[d] != a->shape[d]) || (residual && residual->shape[d] != a->shape[d])) {
      set_error("matmul: batch dims differ");
      return PGB_ERR_INVALID_ARG;
    }
    nbatch *= a->shape[d];
  }
  for (const pgb_tensor *t : {a, b})
    for (int d = 0; d < t->ndim; ++d)
      if (t->stride_bytes[d] % 4 || t->stride_bytes[d] < 0) { set_error("matmul: bad stride"); return PGB_ERR_INVALID_ARG; }
  if (out->dtype != PGB_F32 && out->dtype != PGB_F16 && out->dtype != PGB_BF16) {
    set_error(std::string("matmul output not implemented for ") + dtype_name(out->dtype));
    return PGB_ERR_UNSUPPORTED;
  }
  Mat O, R{};
  std::string err = as_mat(*out, "the output", O, false);
  if (err.empty() && residual) err = as_mat(*residual, "the residual", R, false);
  if (!err.empty()) { set_error(err); return PGB_ERR_UNSUPPORTED; }
  if (O.rows != M || O.cols != N || (residual && (residual->ndim != out->ndim || R.rows != M || R.cols != N))) {
    set_error("matmul: output shape does not match");
    return PGB_ERR_INVALID_ARG;
  }
  if (M == 0 || N == 0 || nbatch == 0) return PGB_OK;
  if (K == 0) { set_error("matmul: empty contraction dim"); return PGB_ERR_INVALID_ARG; }
  // batch layout of the output: folded into M (shared b, contiguous batches) or at most two strided dims
  int64_t gM = M, nb0 = 1, nb1 = 1, obs0 = 0, obs1 = 0, rbs0 = 0, rbs1 = 0;
  bool fold = false;
  if (nla > 0) {
    int64_t cnt = 1, st = 0;
    auto folds = [&](const pgb_tensor &t, const Mat &m) { return merge_leading(t, nla, &cnt, &st) && (cnt == 1 || st == m.rows * m.ld); };
    fold = shared_b && folds(*out, O) && (!residual || folds(*residual, R));
    if (fold) {
      gM = M * nbatch;
    } else {
      bool found = false;
      for (int sp = 0; sp <= nla && !found; ++sp) {
        int64_t c0, c1, d0, d1;
        bool ok = merge_dims(*out, 0, sp, &c0, &obs0) && merge_dims(*out, sp, nla, &c1, &obs1);
        if (ok && residual) ok = merge_dims(*residual, 0, sp, &d0, &rbs0) && merge_dims(*residual, sp, nla, &d1, &rbs1);
        // the packed operands are contiguous over the leading dims in order, so the split must cover them in order too
        int64_t e0 = 1, e1 = 1;
        for (int d = 0; d < sp; ++d) e0 *= a->shape[d];
        for (int d = sp; d < nla; ++d) e1 *= a->shape[d];
        if (ok && c0 == e0 && c1 == e1) { nb0 = c0; nb1 = c1; found = true; }
      }
      if (!found) { set_error("matmul: the batch dims of the output do not reduce to two strided dims"); return PGB_ERR_UNSUPPORTED; }
    }
  }
  GemmEpilogue e{};
  e.act = act;
  e.alpha = alpha;
  e.out = out->data;
  e.out_dtype = out->dtype;
  e.ldc = O.ld;
  e.out_batch = obs1;
  e.out_batch0 = obs0;
  if (bias) {
    if (numel_of(*bias) != N || !is_contiguous(*bias) || dtype_size(bias->dtype) == 0) {
      set_error("matmul: the bias must be a contiguous vector of the output width");
      return PGB_ERR_INVALID_ARG;
    }
    e.bias = bias->data;
    e.bias_dtype = bias->dtype;
  }
  if (residual) {
    e.residual = residual->data;
    e.res_dtype = residual->dtype;
    e.res_ld = R.ld;
    e.res_batch = rbs1;
    e.res_batch0 = rbs0;
  }
  if (!device_present()) return PGB_ERR_CUDA;
  const int64_t Kp = (K + 31) / 32 * 32;  // whole 128-byte slabs per segment
  const int64_t nbB = (shared_b && fold) || nla == 0 ? 1 : nbatch;
  const int64_t a_elems = nbatch * M * 3 * Kp, b_elems = nbB * N * 3 * Kp;
  float *scratch = nullptr;
  if (cudaMallocAsync(&scratch, (size_t)(a_elems + b_elems) * sizeof(float), stream) != cudaSuccess) {
    cudaGetLastError();
    set_error("matmul: cannot allocate the scratch buffer for the split fp32 operands");
    return PGB_ERR_CUDA;
  }
  int64_t lsz[6], lst[6], bst[6];
  for (int d = 0; d < nla; ++d) {
    lsz[d] = a->shape[d];
    lst[d] = a->stride_bytes[d] / 4;
    bst[d] = shared_b ? 0 : b->stride_bytes[d] / 4;  // a shared b that cannot be folded is replicated per batch
  }
  int st = run_pack_tf32x3((const float *)a->data, scratch, nla, lsz, lst, M, K, Kp, a->stride_bytes[nla] / 4, a->stride_bytes[nla + 1] / 4, false,
                           stream);
  if (st == PGB_OK)
    st = run_pack_tf32x3((const float *)b->data, scratch + a_elems, nbB == 1 ? 0 : nla, lsz, bst, N, K, Kp, b->stride_bytes[b->ndim - 1] / 4,
                         b->stride_bytes[b->ndim - 2] / 4, true, stream);
  if (st == PGB_OK)
    st = run_gemm_tc(GEMM_TF32, scratch, 3 * Kp, nb1 * M * 3 * Kp, M * 3 * Kp, scratch + a_elems, 3 * Kp, nbB == 1 ? 0 : nb1 * N * 3 * Kp,
                     nbB == 1 ? 0 : N * 3 * Kp, gM, N, 3 * Kp, nb0, nb1, e, stream);
  cudaFreeAsync(scratch, stream);
  return st;
}

// fp64 matmul: shape checks, then the fp64-unit kernel (matmul_f64.cu) reads every operand through its strides.
static int matmul_f64(const pgb_tensor *a, const pgb_tensor *b, const pgb_tensor *bias, int act, float alpha, const pgb_tensor *residual,
                      const pgb_tensor *out, cudaStream_t stream) {
  if (a->ndim < 2 || b->ndim < 2 || out->ndim != a->ndim) { set_error("matmul: operands need at least 2 dims and the output the rank of a"); return PGB_ERR_INVALID_ARG; }
  const int nla = a->ndim - 2;
  if (nla > 6) { set_error("matmul: at most 6 batch dims"); return PGB_ERR_UNSUPPORTED; }
  const int64_t M = a->shape[nla], K = a->shape[nla + 1], N = b->shape[b->ndim - 1];
  if (b->shape[b->ndim - 2] != K) { set_error("matmul: contraction dims differ"); return PGB_ERR_INVALID_ARG; }
  const bool shared_b = b->ndim == 2;
  if (!shared_b && b->ndim != a->ndim) { set_error("matmul: batch dims differ"); return PGB_ERR_INVALID_ARG; }
  if (out->dtype != PGB_F64 || (residual && residual->dtype != PGB_F64) || (bias && bias->dtype != PGB_F64)) {
    set_error("matmul: a float64 matmul takes and gives float64 tensors");
    return PGB_ERR_INVALID_ARG;
  }
  if (out->shape[nla] != M || out->shape[nla + 1] != N || (N > 1 && out->stride_bytes[nla + 1] != 8) ||
      (residual && (residual->ndim != out->ndim || residual->shape[nla] != M || residual->shape[nla + 1] != N || (N > 1 && residual->stride_bytes[nla + 1] != 8)))) {
    set_error("matmul: output shape does not match");
    return PGB_ERR_INVALID_ARG;
  }
  if (bias && (numel_of(*bias) != N || !is_contiguous(*bias))) { set_error("matmul: the bias must be a contiguous vector of the output width"); return PGB_ERR_INVALID_ARG; }
  int64_t lead[6], als[6], bls[6], cls[6], rls[6];
  for (int d = 0; d < nla; ++d) {
    if (out->shape[d] != a->shape[d] || (!shared_b && b->shape[d] != a->shape[d]) || (residual && residual->shape[d] != a->shape[d])) {
      set_error("matmul: batch dims differ");
      return PGB_ERR_INVALID_ARG;
    }
    lead[d] = a->shape[d];
    als[d] = a->stride_bytes[d] / 8;
    bls[d] = shared_b ? 0 : b->stride_bytes[d] / 8;
    cls[d] = out->stride_bytes[d] / 8;
    rls[d] = residual ? residual->stride_bytes[d] / 8 : 0;
  }
  if (K == 0 && M > 0 && N > 0) { set_error("matmul: empty contraction dim"); return PGB_ERR_INVALID_ARG; }
  if (!device_present()) return PGB_ERR_CUDA;
  const int64_t strides[6] = {a->stride_bytes[nla] / 8, a->stride_bytes[nla + 1] / 8, b->stride_bytes[b->ndim - 2] / 8, b->stride_bytes[b->ndim - 1] / 8,
                              out->stride_bytes[nla] / 8, residual ? residual->stride_bytes[nla] / 8 : 0};
  return run_matmul_f64((const double *)a->data, (const double *)b->data, (double *)out->data, bias ? (const double *)bias->data : nullptr,
                        residual ? (const double *)residual->data : nullptr, M, N, K, strides, nla, lead, als, bls, cls, rls, (double)alpha, act, stream);
}

}  // namespace pgb

using namespace pgb;

extern "C" {

PGB_API int pgb_device_error(int *code, int reset) {
  if (!code) return PGB_ERR_INVALID_ARG;
  const int st = read_gemm_error(code, reset != 0);
  if (st != PGB_OK) return st;
  if (*code != 0) {
    set_error("a bounded device-side wait ran out: role " + std::to_string(*code >> 16) + ", block " + std::to_string(*code & 0xffff));
    return PGB_ERR_TIMEOUT;
  }
  return PGB_OK;
}

PGB_API int pgb_gemm_pair_mode(int mode) { return set_gemm_pair_mode(mode); }

PGB_API int pgb_gemm_wait_drill(unsigned int polls, int skip_loads) {
  if (polls == 0) { set_error("gemm_wait_drill: the poll limit must be positive"); return PGB_ERR_INVALID_ARG; }
  set_next_gemm_wait_test(polls, skip_loads != 0);
  return PGB_OK;
}

PGB_API int pgb_absmax_f32(const pgb_tensor *x, float *absmax_dev, void *stream) {
  if (!x || !absmax_dev) { set_error("absmax: null argument"); return PGB_ERR_INVALID_ARG; }
  if (x->dtype != PGB_F32) { set_error(std::string("absmax not implemented for ") + dtype_name(x->dtype)); return PGB_ERR_UNSUPPORTED; }
  if (!is_contiguous(*x)) { set_error("absmax: the tensor must be contiguous"); return PGB_ERR_UNSUPPORTED; }
  if (reinterpret_cast<uintptr_t>(x->data) & 15) { set_error("absmax: the tensor must be 16-byte aligned"); return PGB_ERR_UNSUPPORTED; }
  if (!device_present()) return PGB_ERR_CUDA;
  return run_absmax_f32((const float *)x->data, numel_of(*x), absmax_dev, (cudaStream_t)stream);
}

PGB_API int pgb_quantize_i8(const pgb_tensor *x, const float *absmax_dev, float scale, const pgb_tensor *q, void *stream) {
  if (!x || !q) { set_error("quantize: null argument"); return PGB_ERR_INVALID_ARG; }
  if (x->dtype != PGB_F32 || q->dtype != PGB_I8) { set_error("quantize: expects a float32 input and an int8 output"); return PGB_ERR_UNSUPPORTED; }
  if (!is_contiguous(*x) || !is_contiguous(*q) || numel_of(*x) != numel_of(*q)) {
    set_error("quantize: input and output must be contiguous and of one size");
    return PGB_ERR_INVALID_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(x->data) & 15) || (reinterpret_cast<uintptr_t>(q->data) & 3)) {
    set_error("quantize: the input must be 16-byte and the output 4-byte aligned");
    return PGB_ERR_UNSUPPORTED;
  }
  if (!absmax_dev && !(scale > 0.f)) { set_error("quantize: a positive scale or a device absmax is required"); return PGB_ERR_INVALID_ARG; }
  if (!device_present()) return PGB_ERR_CUDA;
  return run_quantize_i8((const float *)x->data, numel_of(*x), absmax_dev, scale, (int8_t *)q->data, (cudaStream_t)stream);
}

// [.., T, 64] view -> batch / head / row strides in elements; leading dims are padded to [B, H, T, 64]
static std::string as_heads(const pgb_tensor &t, const char *what, int64_t dims[3], int64_t str[3]) {
  if (t.ndim < 2 || t.ndim > 4) return std::string("attention: ") + what + " must have 2 to 4 dims";
  const int es = dtype_size(t.dtype);
  if (t.shape[t.ndim - 1] != 64) return std::string("attention: only a head dim of 64 is implemented (") + what + ")";
  if (t.stride_bytes[t.ndim - 1] != es) return std::string("attention: the head dim of ") + what + " must be contiguous";
  for (int i = 0; i < 3; ++i) { dims[i] = 1; str[i] = 0; }
  for (int d = 0; d < t.ndim - 1; ++d) {
    const int slot = 3 - (t.ndim - 1) + d;
    dims[slot] = t.shape[d];
    if (t.stride_bytes[d] % es || t.stride_bytes[d] < 0) return std::string("attention: bad stride in ") + what;
    str[slot] = t.stride_bytes[d] / es;
  }
  // dims of extent 1 take the stride a contiguous layout would give them
  if (dims[2] == 1) str[2] = 64;
  if (dims[1] == 1) str[1] = str[2] * dims[2];
  if (dims[0] == 1) str[0] = str[1] * dims[1];
  return "";
}

PGB_API int pgb_attention(const pgb_tensor *q, const pgb_tensor *k, const pgb_tensor *v, float scale, int causal, const pgb_tensor *out,
                          void *stream) {
  if (!q || !k || !v || !out) { set_error("attention: null tensor"); return PGB_ERR_INVALID_ARG; }
  if (q->dtype != PGB_F16 && q->dtype != PGB_BF16) {
    set_error(std::string("attention not implemented for ") + dtype_name(q->dtype));
    return PGB_ERR_UNSUPPORTED;
  }
  if (k->dtype != q->dtype || v->dtype != q->dtype || out->dtype != q->dtype) { set_error("attention: q, k, v and out must share one dtype"); return PGB_ERR_INVALID_ARG; }
  int64_t qd[3], kd[3], vd[3], od[3], qs[3], ks[3], vs[3], os[3];
  std::string err = as_heads(*q, "q", qd, qs);
  if (err.empty()) err = as_heads(*k, "k", kd, ks);
  if (err.empty()) err = as_heads(*v, "v", vd, vs);
  if (err.empty()) err = as_heads(*out, "out", od, os);
  if (!err.empty()) { set_error(err); return err.find("only a head dim") != std::string::npos ? PGB_ERR_UNSUPPORTED : PGB_ERR_INVALID_ARG; }
  if (kd[0] != qd[0] || kd[1] != qd[1] || vd[0] != qd[0] || vd[1] != qd[1] || vd[2] != kd[2] || od[0] != qd[0] || od[1] != qd[1] || od[2] != qd[2]) {
    set_error("attention: q, k, v and out disagree on batch, heads or sequence length");
    return PGB_ERR_INVALID_ARG;
  }
  if (qd[2] > 0 && kd[2] == 0) { set_error("attention: no keys"); return PGB_ERR_INVALID_ARG; }
  if (!device_present()) return PGB_ERR_CUDA;
  return run_attention(q->data, k->data, v->data, out->data, q->dtype == PGB_F16, qd[0], qd[1], qd[2], kd[2], qs, ks, vs, os, scale, causal,
                       (cudaStream_t)stream);
}

PGB_API int pgb_qlinear_i8(const pgb_tensor *a, const pgb_tensor *w, const float *w_scale, float a_scale, const float *a_absmax_dev,
                           const pgb_tensor *bias, int relu, const pgb_tensor *out, const pgb_tensor *acc_i32, float *out_absmax_dev,
                           void *stream) {
  if (!a || !w) { set_error("qlinear: null operand"); return PGB_ERR_INVALID_ARG; }
  if (a->dtype != PGB_I8 || w->dtype != PGB_I8) { set_error("qlinear: activations and weights must be int8"); return PGB_ERR_UNSUPPORTED; }
  Mat A, W;
  std::string err = as_mat(*a, "the activations", A);
  if (err.empty()) err = as_mat(*w, "the weights", W);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  if (A.batch != 1 || W.batch != 1) { set_error("qlinear: activations [M,K] and weights [N,K] must be 2-D"); return PGB_ERR_INVALID_ARG; }
  if (A.cols != W.cols) { set_error("qlinear: contraction dims differ"); return PGB_ERR_INVALID_ARG; }
  const int64_t M = A.rows, N = W.rows, K = A.cols;
  GemmEpilogue e{};
  e.col_scale = w_scale;
  e.a_scale = a_scale;
  e.a_scale_dev = a_absmax_dev;
  e.act = relu ? 1 : 0;
  e.absmax = out_absmax_dev;
  if (bias) {
    if (numel_of(*bias) != N || !is_contiguous(*bias) || (bias->dtype != PGB_F32 && bias->dtype != PGB_F16)) {
      set_error("qlinear: the bias must be a contiguous float32 / float16 vector of the output width");
      return PGB_ERR_INVALID_ARG;
    }
    e.bias = bias->data;
    e.bias_dtype = bias->dtype;
  }
  if (out) {
    Mat O;
    err = as_mat(*out, "the output", O);
    if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
    if (O.rows != M || O.cols != N || O.batch != 1) { set_error("qlinear: the output must be [M,N]"); return PGB_ERR_INVALID_ARG; }
    if (out->dtype != PGB_F32 && out->dtype != PGB_F16 && out->dtype != PGB_BF16 && out->dtype != PGB_I8) {
      set_error(std::string("qlinear output not implemented for ") + dtype_name(out->dtype));
      return PGB_ERR_UNSUPPORTED;
    }
    if (out->dtype == PGB_I8) {
      // requantising mode: the absmax of this layer's output is an INPUT (from an earlier output-less pass)
      if (!out_absmax_dev) { set_error("qlinear: an int8 output is quantised with the device absmax, which is missing"); return PGB_ERR_INVALID_ARG; }
      e.requant_absmax = out_absmax_dev;
      e.absmax = nullptr;
    }
    e.out = out->data;
    e.out_dtype = out->dtype;
    e.ldc = O.ld;
  }
  if (acc_i32) {
    Mat C;
    err = as_mat(*acc_i32, "the accumulator output", C);
    if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
    if (acc_i32->dtype != PGB_I32 || C.rows != M || C.cols != N || C.batch != 1) { set_error("qlinear: the accumulator output must be int32 [M,N]"); return PGB_ERR_INVALID_ARG; }
    e.acc_out = (int32_t *)acc_i32->data;
    e.ld_acc = C.ld;
  }
  if (!out && !acc_i32 && !out_absmax_dev) { set_error("qlinear: nothing to write"); return PGB_ERR_INVALID_ARG; }
  if (!device_present()) return PGB_ERR_CUDA;
  e.alpha = 1.f;
  return run_gemm_tc(GEMM_I8, A.ptr, A.ld, 0, 0, W.ptr, W.ld, 0, 0, M, N, K, 1, 1, e, (cudaStream_t)stream);
}

PGB_API int pgb_matmul(const pgb_tensor *a, const pgb_tensor *b, const pgb_tensor *bias, int act, float alpha, const pgb_tensor *residual,
                       const pgb_tensor *out, void *stream) {
  if (!a || !b || !out) { set_error("matmul: null operand"); return PGB_ERR_INVALID_ARG; }
  if (a->dtype != b->dtype) { set_error("matmul: operand dtypes differ"); return PGB_ERR_INVALID_ARG; }
  if (act < 0 || act > 2) { set_error("matmul: unknown activation"); return PGB_ERR_INVALID_ARG; }
  if (a->dtype == PGB_F32) return matmul_f32(a, b, bias, act, alpha, residual, out, (cudaStream_t)stream);
  if (a->dtype == PGB_F64) return matmul_f64(a, b, bias, act, alpha, residual, out, (cudaStream_t)stream);
  if (a->dtype != PGB_F16 && a->dtype != PGB_BF16) {
    // reference wording, csrc/cuda/matmul.cu:157-160
    set_error(std::string("matmul_cuda not implemented for ") + dtype_name(a->dtype));
    return PGB_ERR_UNSUPPORTED;
  }
  if (act < 0 || act > 2) { set_error("matmul: unknown activation"); return PGB_ERR_INVALID_ARG; }
  if (b->ndim < 2) { set_error("matmul: b must have at least 2 dims"); return PGB_ERR_INVALID_ARG; }
  // b is the [.., K, N] operand of `a @ b`; the kernel wants it K-major, i.e. as a view whose K dim is the contiguous one
  pgb_tensor bt = *b;
  const int nb = b->ndim;
  bt.shape[nb - 2] = b->shape[nb - 1];
  bt.shape[nb - 1] = b->shape[nb - 2];
  bt.stride_bytes[nb - 2] = b->stride_bytes[nb - 1];
  bt.stride_bytes[nb - 1] = b->stride_bytes[nb - 2];
  // Operands that TMA cannot read as they are (K not the contiguous dim, e.g. a plain row-major [K, N] b, or pitches that
  // are not multiples of 16 bytes) are copied K-major into a stream-ordered scratch buffer first, as the reference
  // contiguises its inputs (csrc/cuda/matmul.cu:80-93). Weights laid out [N, K] once and packed qkv views skip this.
  pgb_tensor a_use = *a;
  void *scratch = nullptr;
  {
    const bool pack_a = !tma_ready(*a), pack_b = !tma_ready(bt);
    if ((pack_a || pack_b) && a->shape[a->ndim - 1] == bt.shape[nb - 1] && a->ndim - 2 <= 6 && nb - 2 <= 6 && device_present()) {
      const int64_t K = a->shape[a->ndim - 1], Kp = (K + 7) / 8 * 8;
      auto elems = [&](const pgb_tensor &t) { int64_t n = Kp; for (int d = 0; d < t.ndim - 1; ++d) n *= t.shape[d]; return (n + 7) / 8 * 8; };
      const int64_t na = pack_a ? elems(*a) : 0, nbe = pack_b ? elems(bt) : 0;
      if (na + nbe > 0) {
        if (cudaMallocAsync(&scratch, (size_t)(na + nbe) * 2, (cudaStream_t)stream) != cudaSuccess) {
          cudaGetLastError();
          set_error("matmul: cannot allocate the scratch buffer for the operand re-layout");
          return PGB_ERR_CUDA;
        }
        auto pack = [&](const pgb_tensor &t, void *dst) {
          int64_t lsz[6], lst[6];
          const int nl = t.ndim - 2;
          for (int d = 0; d < nl; ++d) { lsz[d] = t.shape[d]; lst[d] = t.stride_bytes[d] / 2; }
          return run_pack_copy16(t.data, dst, nl, lsz, lst, t.shape[nl], K, Kp, t.stride_bytes[nl] / 2, t.stride_bytes[nl + 1] / 2, (cudaStream_t)stream);
        };
        int st = PGB_OK;
        if (pack_a) { st = pack(*a, scratch); a_use = packed_view(*a, scratch, Kp); }
        if (st == PGB_OK && pack_b) {
          void *dst = (uint16_t *)scratch + na;
          st = pack(bt, dst);
          bt = packed_view(bt, dst, Kp);
        }
        if (st != PGB_OK) { cudaFreeAsync(scratch, (cudaStream_t)stream); return st; }
      }
    }
  }
  struct ScratchGuard {
    void *p; cudaStream_t s;
    ~ScratchGuard() { if (p) cudaFreeAsync(p, s); }
  } guard{scratch, (cudaStream_t)stream};
  a = &a_use;
  Mat A, B, O;
  std::string err = as_mat(*a, "a", A, false);
  if (err.empty()) err = as_mat(bt, "b", B, false);
  if (err.empty()) err = as_mat(*out, "the output", O, false);
  Mat R{};
  if (err.empty() && residual) err = as_mat(*residual, "the residual", R, false);
  if (!err.empty()) { set_error(err); return PGB_ERR_UNSUPPORTED; }
  if (A.cols != B.cols) { set_error("matmul: contraction dims differ"); return PGB_ERR_INVALID_ARG; }
  const int64_t N = B.rows, K = A.cols;
  int64_t M = A.rows, nb0 = 1, nb1 = 1;
  int64_t abs0 = 0, abs1 = 0, bbs0 = 0, bbs1 = 0, obs0 = 0, obs1 = 0, rbs0 = 0, rbs1 = 0;
  const int nla = a->ndim - 2;
  if (O.cols != N || O.rows != A.rows || out->ndim != a->ndim) { set_error("matmul: output shape does not match"); return PGB_ERR_INVALID_ARG; }
  for (int d = 0; d < nla; ++d)
    if (out->shape[d] != a->shape[d] || (residual && residual->shape[d] != a->shape[d])) { set_error("matmul: batch dims differ"); return PGB_ERR_INVALID_ARG; }
  if (residual && (residual->ndim != out->ndim || R.rows != O.rows || R.cols != N)) { set_error("matmul: the residual must have the output's shape"); return PGB_ERR_INVALID_ARG; }
  if (b->ndim == 2 && nla > 0) {
    // shared weight: fold a's batch into M when its rows (and the output's) form one pitch
    int64_t cnt = 1, st = 0;
    auto folds = [&](const pgb_tensor &t, const Mat &m) { return merge_leading(t, nla, &cnt, &st) && (cnt == 1 || st == m.rows * m.ld); };
    if (!folds(*a, A) || !folds(*out, O) || (residual && !folds(*residual, R))) {
      set_error("matmul: a batched `a` with a 2-D `b` needs batches that are contiguous in memory");
      return PGB_ERR_UNSUPPORTED;
    }
    merge_leading(*a, nla, &cnt, &st);
    M = A.rows * cnt;
  } else if (nla > 0) {
    if (b->ndim != a->ndim) { set_error("matmul: batch dims differ"); return PGB_ERR_INVALID_ARG; }
    for (int d = 0; d < nla; ++d)
      if (b->shape[d] != a->shape[d]) { set_error("matmul: batch dims differ"); return PGB_ERR_INVALID_ARG; }
    // the leading dims become at most two batch dims with one stride each, the same split for every operand
    bool found = false;
    for (int sp = 0; sp <= nla && !found; ++sp) {
      int64_t c0, c1, d0, d1;
      bool ok = merge_dims(*a, 0, sp, &c0, &abs0) && merge_dims(*a, sp, nla, &c1, &abs1);
      ok = ok && merge_dims(bt, 0, sp, &d0, &bbs0) && merge_dims(bt, sp, nla, &d1, &bbs1);
      ok = ok && merge_dims(*out, 0, sp, &d0, &obs0) && merge_dims(*out, sp, nla, &d1, &obs1);
      if (ok && residual) ok = merge_dims(*residual, 0, sp, &d0, &rbs0) && merge_dims(*residual, sp, nla, &d1, &rbs1);
      if (ok) { nb0 = c0; nb1 = c1; found = true; }
    }
    if (!found) { set_error("matmul: the batch dims do not reduce to two strided dims"); return PGB_ERR_UNSUPPORTED; }
  }
  if (out->dtype != PGB_F32 && out->dtype != PGB_F16 && out->dtype != PGB_BF16) {
    set_error(std::string("matmul output not implemented for ") + dtype_name(out->dtype));
    return PGB_ERR_UNSUPPORTED;
  }
  GemmEpilogue e{};
  e.act = act;
  e.alpha = alpha;
  e.out = out->data;
  e.out_dtype = out->dtype;
  e.ldc = O.ld;
  e.out_batch = obs1;
  e.out_batch0 = obs0;
  if (bias) {
    if (numel_of(*bias) != N || !is_contiguous(*bias) || dtype_size(bias->dtype) == 0) {
      set_error("matmul: the bias must be a contiguous vector of the output width");
      return PGB_ERR_INVALID_ARG;
    }
    e.bias = bias->data;
    e.bias_dtype = bias->dtype;
  }
  if (residual) {
    e.residual = residual->data;
    e.res_dtype = residual->dtype;
    e.res_ld = R.ld;
    e.res_batch = rbs1;
    e.res_batch0 = rbs0;
  }
  if (!device_present()) return PGB_ERR_CUDA;
  return run_gemm_tc(a->dtype == PGB_F16 ? GEMM_F16 : GEMM_BF16, A.ptr, A.ld, abs0, abs1, B.ptr, B.ld, bbs0, bbs1, M, N, K, nb0, nb1, e,
                     (cudaStream_t)stream);
}

}  // extern "C"
