// Host-side canonicalisation of strided views into the few loop nests the
// kernels implement. Pure C++ (no CUDA) so the same code runs in the CPU tests.
//
// The reference never canonicalises: every kernel walks all n dims with a
// div/mod chain per element (csrc/cuda/reduce.cuh:56-67,
// csrc/cuda/cuda_utils.cuh:40-52). Here permuted / broadcast / sliced views are
// first reduced to "kept dims" and "reduced dims" with element strides, size-1
// dims dropped and mergeable neighbours merged, so that most permutes vanish.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/pgb200.h"

namespace pgb {

inline int dtype_size(int dt) {
  switch (dt) {
    case PGB_I32: return 4;
    case PGB_F16: return 2;
    case PGB_F32: return 4;
    case PGB_F64: return 8;
    case PGB_I8: return 1;
    case PGB_BF16: return 2;
    default: return 0;
  }
}

inline const char *dtype_name(int dt) {
  // names as the reference prints them (csrc/dtype.cpp dtype_to_string)
  switch (dt) {
    case PGB_I32: return "int32";
    case PGB_F16: return "float16";
    case PGB_F32: return "float32";
    case PGB_F64: return "float64";
    case PGB_I8: return "int8";
    case PGB_BF16: return "bfloat16";
    default: return "unknown";
  }
}

struct CanonReduce {
  int n_in = 0;
  int nk = 0, nr = 0;                 // kept / reduced dims after merging
  int64_t ksize[PGB_MAX_DIMS] = {0};  // outer -> inner (output order)
  int64_t rsize[PGB_MAX_DIMS] = {0};  // outer -> inner (largest stride first)
  int64_t kin[PGB_MAX_INPUTS][PGB_MAX_DIMS] = {{0}};  // element strides of each input
  int64_t rin[PGB_MAX_INPUTS][PGB_MAX_DIMS] = {{0}};
  int64_t n_out = 1, n_red = 1;
  // the output index space before merging (keepdims shape without the reduced
  // dims), for epilogue operands
  int out_ndim = 0;
  int64_t out_size[PGB_MAX_DIMS] = {0};
  int out_axis[PGB_MAX_DIMS] = {0};  // original axis of each entry of out_size
};

struct Dim {
  int64_t size;
  int64_t out_stride;  // kept dims only
  int64_t in[PGB_MAX_INPUTS];
  int axis;
};

// Returns "" on success, otherwise an error message.
inline std::string canonicalise_reduce(const pgb_tensor *in, int n_in, const int32_t *axes, int n_axes,
                                       CanonReduce &c) {
  if (n_in < 1 || n_in > PGB_MAX_INPUTS) return "fused_reduce: between 1 and 6 inputs are supported";
  const int nd = in[0].ndim;
  if (nd < 0 || nd > PGB_MAX_DIMS) return "fused_reduce: at most 8 dims are supported";
  bool red[PGB_MAX_DIMS] = {false};
  for (int i = 0; i < n_axes; ++i) {
    int a = axes[i] < 0 ? axes[i] + nd : axes[i];
    if (a < 0 || a >= nd) return "fused_reduce: axis out of range";
    if (red[a]) return "fused_reduce: duplicate axis";
    red[a] = true;
  }
  for (int k = 0; k < n_in; ++k) {
    if (in[k].ndim != nd) return "fused_reduce: all inputs must have the same number of dims";
    const int sz = dtype_size(in[k].dtype);
    if (sz == 0) return "fused_reduce: unknown dtype";
    for (int d = 0; d < nd; ++d) {
      if (in[k].shape[d] != in[0].shape[d]) return "fused_reduce: all inputs must have the same shape";
      if (in[k].stride_bytes[d] < 0) return "fused_reduce: negative strides are not supported";
      if (in[k].stride_bytes[d] % sz != 0) return "fused_reduce: stride is not a multiple of the element size";
    }
  }
  c = CanonReduce();
  c.n_in = n_in;
  std::vector<Dim> kept, reduced;
  for (int d = 0; d < nd; ++d) {
    const int64_t s = in[0].shape[d];
    if (s < 0) return "fused_reduce: negative extent";
    if (red[d]) c.n_red *= s; else {
      c.n_out *= s;
      c.out_size[c.out_ndim] = s;
      c.out_axis[c.out_ndim] = d;
      c.out_ndim++;
    }
    if (s == 1) continue;
    Dim dm;
    dm.size = s;
    dm.axis = d;
    dm.out_stride = 0;
    for (int k = 0; k < n_in; ++k) dm.in[k] = in[k].stride_bytes[d] / dtype_size(in[k].dtype);
    (red[d] ? reduced : kept).push_back(dm);
  }
  // reduced dims: order is free; put the largest stride outermost so the
  // innermost loop walks the most contiguous memory
  auto key = [&](const Dim &a) {
    int64_t m = 0;
    for (int k = 0; k < n_in; ++k) m = std::max(m, a.in[k]);
    return m;
  };
  std::stable_sort(reduced.begin(), reduced.end(), [&](const Dim &a, const Dim &b) { return key(a) > key(b); });
  auto merge = [&](std::vector<Dim> &v) {
    std::vector<Dim> o;
    for (const Dim &d : v) {
      if (!o.empty()) {
        Dim &p = o.back();
        bool ok = true;
        for (int k = 0; k < n_in; ++k) ok = ok && (p.in[k] == d.in[k] * d.size);
        if (ok) {
          p.size *= d.size;
          for (int k = 0; k < n_in; ++k) p.in[k] = d.in[k];
          continue;
        }
      }
      o.push_back(d);
    }
    v.swap(o);
  };
  merge(kept);
  merge(reduced);
  c.nk = (int)kept.size();
  c.nr = (int)reduced.size();
  for (int i = 0; i < c.nk; ++i) {
    c.ksize[i] = kept[i].size;
    for (int k = 0; k < n_in; ++k) c.kin[k][i] = kept[i].in[k];
  }
  for (int i = 0; i < c.nr; ++i) {
    c.rsize[i] = reduced[i].size;
    for (int k = 0; k < n_in; ++k) c.rin[k][i] = reduced[i].in[k];
  }
  return "";
}

// Elementwise canonical form: dims outer -> inner in output order, merged.
struct CanonEw {
  int n_in = 0;
  int nd = 0;
  int64_t size[PGB_MAX_DIMS] = {0};
  int64_t in[PGB_MAX_INPUTS][PGB_MAX_DIMS] = {{0}};
  int64_t numel = 1;
};

inline std::string canonicalise_elementwise(const pgb_tensor *in, int n_in, const pgb_tensor *out, CanonEw &c) {
  if (n_in < 0 || n_in > PGB_MAX_INPUTS) return "fused_elementwise: at most 6 inputs are supported";
  const int nd = out->ndim;
  if (nd < 0 || nd > PGB_MAX_DIMS) return "fused_elementwise: at most 8 dims are supported";
  c = CanonEw();
  c.n_in = n_in;
  for (int k = 0; k < n_in; ++k) {
    if (in[k].ndim != nd) return "fused_elementwise: inputs must have the shape of the output";
    const int sz = dtype_size(in[k].dtype);
    if (sz == 0) return "fused_elementwise: unknown dtype";
    for (int d = 0; d < nd; ++d) {
      if (in[k].shape[d] != out->shape[d]) return "fused_elementwise: inputs must have the shape of the output";
      if (in[k].stride_bytes[d] < 0) return "fused_elementwise: negative strides are not supported";
      if (in[k].stride_bytes[d] % sz != 0) return "fused_elementwise: stride is not a multiple of the element size";
    }
  }
  std::vector<Dim> dims;
  for (int d = 0; d < nd; ++d) {
    const int64_t s = out->shape[d];
    if (s < 0) return "fused_elementwise: negative extent";
    c.numel *= s;
    if (s == 1) continue;
    Dim dm;
    dm.size = s;
    dm.axis = d;
    dm.out_stride = 0;
    for (int k = 0; k < n_in; ++k) dm.in[k] = in[k].stride_bytes[d] / dtype_size(in[k].dtype);
    if (!dims.empty()) {
      Dim &p = dims.back();
      bool ok = true;
      for (int k = 0; k < n_in; ++k) ok = ok && (p.in[k] == dm.in[k] * dm.size);
      if (ok) {
        p.size *= dm.size;
        for (int k = 0; k < n_in; ++k) p.in[k] = dm.in[k];
        continue;
      }
    }
    dims.push_back(dm);
  }
  c.nd = (int)dims.size();
  for (int i = 0; i < c.nd; ++i) {
    c.size[i] = dims[i].size;
    for (int k = 0; k < n_in; ++k) c.in[k][i] = dims[i].in[k];
  }
  return "";
}

// True if `t` is contiguous in the logical order of its shape (size-1 dims ignored).
inline bool is_contiguous(const pgb_tensor &t) {
  int64_t expect = dtype_size(t.dtype);
  for (int d = t.ndim - 1; d >= 0; --d) {
    if (t.shape[d] == 1) continue;
    if (t.stride_bytes[d] != expect) return false;
    expect *= t.shape[d];
  }
  return true;
}

inline int64_t numel_of(const pgb_tensor &t) {
  int64_t n = 1;
  for (int d = 0; d < t.ndim; ++d) n *= t.shape[d];
  return n;
}

}  // namespace pgb
