// Host-side handling of expression programs: validation, choice of the
// compute type, and lowering to the two device forms (general SSA, chain).
// The reference lowers the same op set to CUDA source text
// (csrc/compiler/ir.cpp:599-742, 1384-1557); here the program is data that
// pre-compiled kernels interpret.
#pragma once
#include <string>

#include "common.cuh"
#include "plan.hpp"

namespace pgb {

inline bool op_is_unary(int op) { return op >= PGB_OP_LOG && op <= PGB_OP_CAST_BF16; }
inline bool op_is_binary(int op) { return op >= PGB_OP_ADD && op <= PGB_OP_GTE; }

// allow_acc: epilogue programs may read the reduction result.
inline std::string validate_program(const pgb_instr *p, int n, int n_loads, bool allow_acc, const char *what) {
  if (n < 0 || n > PGB_MAX_INSTRS) return std::string(what) + ": program longer than 32 instructions";
  if (n > 0 && p == nullptr) return std::string(what) + ": null program";
  for (int i = 0; i < n; ++i) {
    const int op = p[i].op;
    auto ref = [&](int v) { return v >= 0 && v < i; };
    if (op == PGB_OP_LOAD) {
      if (p[i].a < 0 || p[i].a >= n_loads) return std::string(what) + ": LOAD of a tensor that was not passed";
    } else if (op == PGB_OP_IMM) {
    } else if (op == PGB_OP_ACC) {
      if (!allow_acc) return std::string(what) + ": ACC is only valid in an epilogue";
    } else if (op_is_unary(op)) {
      if (!ref(p[i].a)) return std::string(what) + ": operand refers to a later value";
    } else if (op_is_binary(op)) {
      if (!ref(p[i].a) || !ref(p[i].b)) return std::string(what) + ": operand refers to a later value";
    } else if (op == PGB_OP_WHERE) {
      if (!ref(p[i].a) || !ref(p[i].b) || !ref(p[i].c)) return std::string(what) + ": operand refers to a later value";
    } else {
      return std::string(what) + ": unknown opcode";
    }
  }
  return "";
}

// f64 if any tensor is f64, i32 if all are integer, f32 otherwise.
inline int compute_dtype(const pgb_tensor *in, int n_in, int fallback) {
  if (n_in == 0) return (fallback == PGB_F64) ? PGB_F64 : ((fallback == PGB_I32 || fallback == PGB_I8) ? PGB_I32 : PGB_F32);
  bool any64 = false, all_int = true;
  for (int k = 0; k < n_in; ++k) {
    if (in[k].dtype == PGB_F64) any64 = true;
    if (in[k].dtype != PGB_I32 && in[k].dtype != PGB_I8) all_int = false;
  }
  return any64 ? PGB_F64 : (all_int ? PGB_I32 : PGB_F32);
}

template <typename T>
inline void to_vm(const pgb_instr *p, int n, VmProg<T> &o) {
  o.n = n;
  for (int i = 0; i < n; ++i) {
    o.op[i] = p[i].op;
    o.a[i] = (int8_t)p[i].a;
    o.b[i] = (int8_t)p[i].b;
    o.c[i] = (int8_t)p[i].c;
    o.imm[i] = (T)p[i].imm;
  }
  for (int i = n; i < kMaxInstr; ++i) {
    o.op[i] = 0; o.a[i] = o.b[i] = o.c[i] = 0; o.imm[i] = (T)0;
  }
}

// Lowers to chain form when the expression tree is a caterpillar (at every
// binary / ternary node at most one operand is not a leaf). Returns false
// otherwise.
template <typename T>
inline bool to_chain(const pgb_instr *p, int n, ChainProg<T> &o) {
  if (n <= 0) return false;
  auto is_leaf = [&](int v) { return p[v].op == PGB_OP_LOAD || p[v].op == PGB_OP_IMM; };
  struct Step { uint8_t op; uint8_t kind[3]; uint8_t idx[3]; T imm[3]; };
  Step steps[kChainSteps];
  int ns = 0;
  auto leaf = [&](Step &s, int slot, int v) {
    if (p[v].op == PGB_OP_LOAD) { s.kind[slot] = LEAF_LOAD; s.idx[slot] = (uint8_t)p[v].a; s.imm[slot] = (T)0; }
    else { s.kind[slot] = LEAF_IMM; s.idx[slot] = 0; s.imm[slot] = (T)p[v].imm; }
  };
  int cur = n - 1;
  while (!is_leaf(cur)) {
    if (ns >= kChainSteps) return false;
    const int op = p[cur].op;
    Step s{};
    s.op = (uint8_t)op;
    if (op == PGB_OP_ACC) return false;
    if (op_is_unary(op)) {
      s.kind[0] = LEAF_RUN;
      steps[ns++] = s;
      cur = p[cur].a;
    } else if (op_is_binary(op)) {
      const int a = p[cur].a, b = p[cur].b;
      if (is_leaf(b)) { s.kind[0] = LEAF_RUN; leaf(s, 1, b); steps[ns++] = s; cur = a; }
      else if (is_leaf(a)) {
        // the running value becomes the first operand: swap, mirror or use the reversed opcode
        int rop = op;
        switch (op) {
          case PGB_OP_SUB: rop = IOP_RSUB; break;
          case PGB_OP_DIV: rop = IOP_RDIV; break;
          case PGB_OP_POW: rop = IOP_RPOW; break;
          case PGB_OP_MOD: rop = IOP_RMOD; break;
          case PGB_OP_GT: rop = PGB_OP_LT; break;
          case PGB_OP_LT: rop = PGB_OP_GT; break;
          case PGB_OP_LTE: rop = PGB_OP_GTE; break;
          case PGB_OP_GTE: rop = PGB_OP_LTE; break;
          default: break;  // add, mul, max, eq, neq commute
        }
        s.op = (uint8_t)rop;
        s.kind[0] = LEAF_RUN; leaf(s, 1, a); steps[ns++] = s; cur = b;
      }
      else return false;
    } else {  // where
      const int v[3] = {p[cur].a, p[cur].b, p[cur].c};
      int spine = -1;
      for (int q = 0; q < 3; ++q)
        if (!is_leaf(v[q])) { if (spine >= 0) return false; spine = q; }
      if (spine < 0) spine = 0;
      for (int q = 0; q < 3; ++q) { if (q == spine) s.kind[q] = LEAF_RUN; else leaf(s, q, v[q]); }
      steps[ns++] = s;
      cur = v[spine];
    }
  }
  o = ChainProg<T>();
  o.n_steps = ns;
  o.first_kind = (p[cur].op == PGB_OP_LOAD) ? LEAF_LOAD : LEAF_IMM;
  o.first_idx = (p[cur].op == PGB_OP_LOAD) ? (uint8_t)p[cur].a : 0;
  o.first_imm = (T)p[cur].imm;
  o.identity = (ns == 0 && o.first_kind == LEAF_LOAD && o.first_idx == 0) ? 1 : 0;
  o.lite = 1;
  for (int s = 0; s < ns; ++s) {
    const int op = steps[s].op;
    const bool cheap = (op_is_binary(op) && op != PGB_OP_POW && op != PGB_OP_MOD) || op == IOP_RSUB || op == IOP_RDIV;
    if (!cheap) o.lite = 0;
  }
  if (ns > kFastSteps) o.lite = 0;
  // x * a + b on input 0 (steps are still in reverse order here: steps[0] is the last op)
  o.affine = (ns == 2 && o.first_kind == LEAF_LOAD && o.first_idx == 0 && steps[1].op == PGB_OP_MUL && steps[1].kind[1] == LEAF_IMM &&
              steps[0].op == PGB_OP_ADD && steps[0].kind[1] == LEAF_IMM) ? 1 : 0;
  for (int s = 0; s < ns; ++s) {
    const Step &st = steps[ns - 1 - s];
    o.op[s] = st.op;
    for (int q = 0; q < 3; ++q) { o.kind[s][q] = st.kind[q]; o.idx[s][q] = st.idx[q]; o.imm[s][q] = st.imm[q]; }
  }
  return true;
}

}  // namespace pgb
