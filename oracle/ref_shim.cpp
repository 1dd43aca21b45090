// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points around the reference's OWN header-only CPU templates,
// compiled from where they lie (the include path points into the reference
// checkout; nothing is copied). Built by oracle/build.py into
// oracle/_ref/libpgref.so and used to pin the C restatement in pgoracle.c.
//   cpu::reduce_base_fn + SumOp/MaxOp/MeanOp   csrc/cpu/reduce.hpp:11-86
//   cpu::_dispatch_binary_op_helper            csrc/cpu/binary.hpp:58-85
//   cpu::ternar_op_ker                         csrc/cpu/ternary.hpp:11-43
//   matmul_ker<T> (generic)                    csrc/cpu/matmul.hpp:6-21
#include <cstdint>
#include <stdexcept>
#include <vector>

#include "cpu/binary.hpp"
#include "cpu/matmul.hpp"
#include "cpu/reduce.hpp"
#include "cpu/ternary.hpp"

#define REF_API extern "C" __attribute__((visibility("default")))

using namespace pg;

template <typename T>
static void reduce_t(const void *in, void *out, const strides_t &st, const shape_t &sh, int axis, int op) {
  if (op == 0) cpu::reduce_base_fn<cpu::SumOp<T>, T>((const T *)in, (T *)out, st, sh, axis);
  else if (op == 1) cpu::reduce_base_fn<cpu::MaxOp<T>, T>((const T *)in, (T *)out, st, sh, axis);
  else cpu::reduce_base_fn<cpu::MeanOp<T>, T>((const T *)in, (T *)out, st, sh, axis);
}

REF_API int orc_reduce_axis(const void *in, void *out, const int64_t *strides, const int64_t *shape, int ndim, int axis, int op,
                            int dtype) {
  strides_t st(strides, strides + ndim);
  shape_t sh(shape, shape + ndim);
  switch (dtype) {
    case 2: reduce_t<float>(in, out, st, sh, axis, op); return 0;
    case 3: reduce_t<double>(in, out, st, sh, axis, op); return 0;
    case 0: reduce_t<int>(in, out, st, sh, axis, op); return 0;
    default: return -2;
  }
}

REF_API int orc_binary(const void *lhs, const void *rhs, void *res, const int64_t *ls, const int64_t *rs, const int64_t *os,
                       const int64_t *shape, int ndim, int op, int dtype) {
  strides_t l(ls, ls + ndim), r(rs, rs + ndim), o(os, os + ndim);
  shape_t sh(shape, shape + ndim);
  const cpu::BinaryOpType t = (cpu::BinaryOpType)op;  // same order as the enum, csrc/cpu/binary.hpp:10-23
  switch (dtype) {
    case 2: cpu::_dispatch_binary_op_helper<float>(sh, l, r, o, lhs, rhs, res, t); return 0;
    case 3: cpu::_dispatch_binary_op_helper<double>(sh, l, r, o, lhs, rhs, res, t); return 0;
    case 0: cpu::_dispatch_binary_op_helper<int>(sh, l, r, o, lhs, rhs, res, t); return 0;
    default: return -2;
  }
}

template <typename T>
static void where_t(const void *a, const void *b, const void *c, void *res, const strides_t &as, const strides_t &bs,
                    const strides_t &cs, const strides_t &os, const shape_t &sh) {
  cpu::ternar_op_ker<T>((const T *)a, (const T *)b, (const T *)c, (T *)res, as, bs, cs, os, sh,
                        [](T x, T y, T z) { return x ? y : z; });  // csrc/cpu/ternary.cpp where lambda
}

REF_API int orc_where(const void *a, const void *b, const void *c, void *res, const int64_t *as, const int64_t *bs, const int64_t *cs,
                      const int64_t *os, const int64_t *shape, int ndim, int dtype) {
  strides_t A(as, as + ndim), B(bs, bs + ndim), Cc(cs, cs + ndim), O(os, os + ndim);
  shape_t sh(shape, shape + ndim);
  switch (dtype) {
    case 2: where_t<float>(a, b, c, res, A, B, Cc, O, sh); return 0;
    case 3: where_t<double>(a, b, c, res, A, B, Cc, O, sh); return 0;
    case 0: where_t<int>(a, b, c, res, A, B, Cc, O, sh); return 0;
    default: return -2;
  }
}

REF_API void orc_matmul_i32(const int32_t *lhs, const int32_t *rhs, int32_t *res, int64_t M, int64_t N, int64_t K, int64_t B) {
  matmul_ker<int32_t>(lhs, rhs, res, M, N, K, B);
}
