// Device-side building blocks shared by the reduce and elementwise kernels:
// typed loads/stores, the expression evaluators (chain form and general SSA
// form), and the reduction combiners.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pgb200.h"

namespace pgb {

constexpr int kMaxDims = PGB_MAX_DIMS;
constexpr int kMaxIn = PGB_MAX_INPUTS;
constexpr int kMaxInstr = PGB_MAX_INSTRS;
constexpr int kChainSteps = 12;
constexpr int kBatch = 16;  // elements a thread evaluates per program dispatch

// ---------------------------------------------------------------------------
// Programs as the kernels see them (passed by value in kernel parameters).
// ---------------------------------------------------------------------------

// General SSA program; evaluated one element at a time with the values in a
// per-thread array. Used by the generic kernels and by every epilogue.
template <typename T>
struct VmProg {
  int n;
  uint8_t op[kMaxInstr];
  int8_t a[kMaxInstr], b[kMaxInstr], c[kMaxInstr];
  T imm[kMaxInstr];
};

// Chain ("caterpillar") form of a program: one running value, each step
// combines it with leaves (an immediate or a freshly loaded input element).
// The running value stays in named registers, so a thread can run one step
// over a whole batch of elements per dispatch.
enum LeafKind : uint8_t { LEAF_NONE = 0, LEAF_IMM = 1, LEAF_LOAD = 2, LEAF_RUN = 3 };

template <typename T>
struct ChainProg {
  int n_steps;
  int identity;  // 1: the program is exactly LOAD 0
  int lite;      // 1: at most kFastSteps steps, all cheap binary ops (see chain_eval_fast)
  int affine;    // 1: exactly (LOAD 0) * imm[0][1] + imm[1][1]
  uint8_t first_kind, first_idx;
  T first_imm;
  // step s: run = op(x, y[, z]) where exactly one of x/y/z is LEAF_RUN
  uint8_t op[kChainSteps];
  uint8_t kind[kChainSteps][3];
  uint8_t idx[kChainSteps][3];
  T imm[kChainSteps][3];
};

// ---------------------------------------------------------------------------
// Arithmetic in the compute type. Compiled with -fmad=false so that + - * /
// round exactly as the reference's separate eager kernels do.
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ T t_exp(T x);
template <> __device__ __forceinline__ float t_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double t_exp<double>(double x) { return exp(x); }
template <> __device__ __forceinline__ int t_exp<int>(int x) { return (int)expf((float)x); }
template <typename T> __device__ __forceinline__ T t_log(T x);
template <> __device__ __forceinline__ float t_log<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double t_log<double>(double x) { return log(x); }
template <> __device__ __forceinline__ int t_log<int>(int x) { return (int)logf((float)x); }
template <typename T> __device__ __forceinline__ T t_sin(T x) { return (T)sin((double)x); }
template <> __device__ __forceinline__ float t_sin<float>(float x) { return sinf(x); }
template <typename T> __device__ __forceinline__ T t_cos(T x) { return (T)cos((double)x); }
template <> __device__ __forceinline__ float t_cos<float>(float x) { return cosf(x); }
template <typename T> __device__ __forceinline__ T t_pow(T x, T y);
template <> __device__ __forceinline__ float t_pow<float>(float x, float y) { return powf(x, y); }
template <> __device__ __forceinline__ double t_pow<double>(double x, double y) { return pow(x, y); }
template <> __device__ __forceinline__ int t_pow<int>(int x, int y) { return (int)pow((double)x, (double)y); }
template <typename T> __device__ __forceinline__ T t_mod(T x, T y);
template <> __device__ __forceinline__ float t_mod<float>(float x, float y) { return fmodf(x, y); }
template <> __device__ __forceinline__ double t_mod<double>(double x, double y) { return fmod(x, y); }
template <> __device__ __forceinline__ int t_mod<int>(int x, int y) { return y == 0 ? 0 : x % y; }
template <typename T> __device__ __forceinline__ T t_div(T x, T y) { return x / y; }
template <> __device__ __forceinline__ int t_div<int>(int x, int y) {
  // the reference divides by zero here (undefined); return 0 rather than trap
  if (y == 0) return 0;
  if (x == INT32_MIN && y == -1) return INT32_MIN;
  return x / y;
}
template <typename T> __device__ __forceinline__ T t_trunc_i32(T x) { return (T)(int)x; }
template <> __device__ __forceinline__ int t_trunc_i32<int>(int x) { return x; }
template <typename T> __device__ __forceinline__ T t_round_f16(T x) { return (T)__half2float(__float2half_rn((float)x)); }
template <typename T> __device__ __forceinline__ T t_round_bf16(T x) { return (T)__bfloat162float(__float2bfloat16_rn((float)x)); }
template <typename T> __device__ __forceinline__ T t_round_f32(T x) { return (T)(float)x; }

template <typename T>
__device__ __forceinline__ T apply_unary(int op, T x) {
  switch (op) {
    case PGB_OP_LOG: return t_log<T>(x);
    case PGB_OP_EXP: return t_exp<T>(x);
    case PGB_OP_SIN: return t_sin<T>(x);
    case PGB_OP_COS: return t_cos<T>(x);
    case PGB_OP_CAST_F16: return t_round_f16<T>(x);
    case PGB_OP_CAST_F32: return t_round_f32<T>(x);
    case PGB_OP_CAST_I32: return t_trunc_i32<T>(x);
    case PGB_OP_CAST_BF16: return t_round_bf16<T>(x);
    default: return x;
  }
}

template <typename T>
__device__ __forceinline__ T apply_binary(int op, T x, T y) {
  switch (op) {
    case PGB_OP_ADD: return x + y;
    case PGB_OP_MUL: return x * y;
    case PGB_OP_MAX: return x > y ? x : y;
    case PGB_OP_SUB: return x - y;
    case PGB_OP_DIV: return t_div<T>(x, y);
    case PGB_OP_GT: return (T)(x > y);
    case PGB_OP_LT: return (T)(x < y);
    case PGB_OP_MOD: return t_mod<T>(x, y);
    case PGB_OP_EQ: return (T)(x == y);
    case PGB_OP_POW: return t_pow<T>(x, y);
    case PGB_OP_LTE: return (T)(x <= y);
    case PGB_OP_NEQ: return (T)(x != y);
    case PGB_OP_GTE: return (T)(x >= y);
    default: return x;
  }
}

// ---------------------------------------------------------------------------
// Typed scalar access by runtime dtype (generic kernels, epilogue operands).
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ T load_as(const void *p, int dtype, int64_t off) {
  switch (dtype) {
    case PGB_F32: return (T)__ldg((const float *)p + off);
    case PGB_F16: return (T)__half2float(__ldg((const __half *)p + off));
    case PGB_BF16: return (T)__bfloat162float(__ldg((const __nv_bfloat16 *)p + off));
    case PGB_F64: return (T)__ldg((const double *)p + off);
    case PGB_I32: return (T)__ldg((const int *)p + off);
    case PGB_I8: return (T)__ldg((const signed char *)p + off);
    default: return (T)0;
  }
}

template <typename T>
__device__ __forceinline__ void store_as(void *p, int dtype, int64_t off, T v) {
  switch (dtype) {
    case PGB_F32: ((float *)p)[off] = (float)v; break;
    case PGB_F16: ((__half *)p)[off] = __float2half_rn((float)v); break;
    case PGB_BF16: ((__nv_bfloat16 *)p)[off] = __float2bfloat16_rn((float)v); break;
    case PGB_F64: ((double *)p)[off] = (double)v; break;
    case PGB_I32: ((int *)p)[off] = (int)v; break;
    case PGB_I8: ((signed char *)p)[off] = (signed char)(int)v; break;
    default: break;
  }
}

// ---------------------------------------------------------------------------
// General SSA evaluation of one element. `loader(k)` yields input k at this
// position; `acc` is what PGB_OP_ACC reads.
// ---------------------------------------------------------------------------
template <typename T, typename Loader>
__device__ __forceinline__ void vm_eval(const VmProg<T> &pr, T *v, T acc, Loader loader) {
  for (int i = 0; i < pr.n; ++i) {
    const int op = pr.op[i];
    T r;
    if (op == PGB_OP_LOAD) r = loader(pr.a[i]);
    else if (op == PGB_OP_IMM) r = pr.imm[i];
    else if (op == PGB_OP_ACC) r = acc;
    else if (op < PGB_OP_ADD) r = apply_unary<T>(op, v[pr.a[i]]);
    else if (op < PGB_OP_WHERE) r = apply_binary<T>(op, v[pr.a[i]], v[pr.b[i]]);
    else r = (v[pr.a[i]] != (T)0) ? v[pr.b[i]] : v[pr.c[i]];
    v[i] = r;
  }
}

// ---------------------------------------------------------------------------
// Chain evaluation over a batch of N elements held in registers.
// w[k][e] = element e of input k (already widened to T).
//
// In a chain the running value is always the FIRST operand of a binary step;
// where the program had it second, the host swaps the operands of commutative
// ops, mirrors comparisons, and uses the reversed opcodes below for the rest.
// ---------------------------------------------------------------------------
enum { IOP_RSUB = 40, IOP_RDIV = 41, IOP_RPOW = 42, IOP_RMOD = 43 };

template <typename T, int NIN, int N>
__device__ __forceinline__ void chain_first(int is_imm, int idx, T imm, const T (&w)[NIN][N], T (&run)[N]) {
  if (is_imm) {
#pragma unroll
    for (int e = 0; e < N; ++e) run[e] = imm;
  } else {
#pragma unroll
    for (int k = 0; k < NIN; ++k)
      if (k == idx || k == NIN - 1) {
#pragma unroll
        for (int e = 0; e < N; ++e) run[e] = w[k][e];
        break;
      }
  }
}

// One binary step over the batch. The op is chosen by ONE uniform branch with
// the element loop inside each case (a per-element switch gets if-converted
// into "compute every op, then select", which multiplies the instruction count).
// `y(e)` yields the leaf operand of element e without materialising an array.
template <typename T, int N, bool FULL, typename Y>
__device__ __forceinline__ void chain_binary(int op, T (&run)[N], Y y) {
#define PGB_STEP(EXPR)                         \
  {                                            \
    _Pragma("unroll") for (int e = 0; e < N; ++e) { \
      const T a = run[e];                      \
      const T b = y(e);                        \
      run[e] = (EXPR);                         \
    }                                          \
  }                                            \
  break;
  switch (op) {
    case PGB_OP_ADD: PGB_STEP(a + b)
    case PGB_OP_MUL: PGB_STEP(a * b)
    case PGB_OP_SUB: PGB_STEP(a - b)
    case IOP_RSUB: PGB_STEP(b - a)
    case PGB_OP_MAX: PGB_STEP(a > b ? a : b)
    case PGB_OP_DIV: PGB_STEP(t_div<T>(a, b))
    case IOP_RDIV: PGB_STEP(t_div<T>(b, a))
    case PGB_OP_GT: PGB_STEP((T)(a > b))
    case PGB_OP_LT: PGB_STEP((T)(a < b))
    case PGB_OP_EQ: PGB_STEP((T)(a == b))
    case PGB_OP_NEQ: PGB_STEP((T)(a != b))
    case PGB_OP_LTE: PGB_STEP((T)(a <= b))
    case PGB_OP_GTE: PGB_STEP((T)(a >= b))
    default:
      if (FULL) {
        switch (op) {
          case PGB_OP_POW: PGB_STEP(t_pow<T>(a, b))
          case IOP_RPOW: PGB_STEP(t_pow<T>(b, a))
          case PGB_OP_MOD: PGB_STEP(t_mod<T>(a, b))
          case IOP_RMOD: PGB_STEP(t_mod<T>(b, a))
          default: break;
        }
      }
      break;
  }
#undef PGB_STEP
}

template <typename T, int NIN, int N, bool FULL>
__device__ __forceinline__ void chain_step_binary(int op, int leaf_is_imm, int idx, T imm, const T (&w)[NIN][N], T (&run)[N]) {
  if (leaf_is_imm) {
    chain_binary<T, N, FULL>(op, run, [&](int) { return imm; });
  } else {
#pragma unroll
    for (int k = 0; k < NIN; ++k)
      if (k == idx) chain_binary<T, N, FULL>(op, run, [&](int e) { return w[k][e]; });
  }
}

// Value of a leaf for element e, by selects (used by `where`, whose three
// operands would otherwise need three arrays).
template <typename T, int NIN, int N>
__device__ __forceinline__ T leaf_val(int kind, int idx, T imm, const T (&w)[NIN][N], const T (&run)[N], int e) {
  T v = w[NIN - 1][e];
#pragma unroll
  for (int k = 0; k < NIN - 1; ++k) v = (idx == k) ? w[k][e] : v;
  v = (kind == LEAF_IMM) ? imm : v;
  return (kind == LEAF_RUN) ? run[e] : v;
}

// General chain: any op, any length up to kChainSteps; the program is read
// from the kernel parameters step by step. Callers use a small batch.
template <typename T, int NIN, int N>
__device__ __forceinline__ void chain_eval(const ChainProg<T> &pr, const T (&w)[NIN][N], T (&run)[N]) {
  chain_first<T, NIN, N>(pr.first_kind == LEAF_IMM, pr.first_idx, pr.first_imm, w, run);
  for (int s = 0; s < pr.n_steps; ++s) {
    const int op = pr.op[s];
    if (op < PGB_OP_ADD) {
      switch (op) {
#define PGB_UN(OPC, EXPR)                                              \
  case OPC: {                                                          \
    _Pragma("unroll") for (int e = 0; e < N; ++e) run[e] = (EXPR);   \
  } break;
        PGB_UN(PGB_OP_LOG, t_log<T>(run[e]))
        PGB_UN(PGB_OP_EXP, t_exp<T>(run[e]))
        PGB_UN(PGB_OP_SIN, t_sin<T>(run[e]))
        PGB_UN(PGB_OP_COS, t_cos<T>(run[e]))
        PGB_UN(PGB_OP_CAST_F16, t_round_f16<T>(run[e]))
        PGB_UN(PGB_OP_CAST_F32, t_round_f32<T>(run[e]))
        PGB_UN(PGB_OP_CAST_I32, t_trunc_i32<T>(run[e]))
        PGB_UN(PGB_OP_CAST_BF16, t_round_bf16<T>(run[e]))
#undef PGB_UN
        default: break;
      }
    } else if (op != PGB_OP_WHERE) {
      chain_step_binary<T, NIN, N, true>(op, pr.kind[s][1] == LEAF_IMM, pr.idx[s][1], pr.imm[s][1], w, run);
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const T x = leaf_val<T, NIN, N>(pr.kind[s][0], pr.idx[s][0], pr.imm[s][0], w, run, e);
        const T y = leaf_val<T, NIN, N>(pr.kind[s][1], pr.idx[s][1], pr.imm[s][1], w, run, e);
        const T z = leaf_val<T, NIN, N>(pr.kind[s][2], pr.idx[s][2], pr.imm[s][2], w, run, e);
        run[e] = (x != (T)0) ? y : z;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Fast chains: at most kFastSteps cheap binary steps (no where, no unary, no
// pow / mod). The program is decoded ONCE per thread into registers and the
// step loop is fully unrolled and predicated on the step count.
// ---------------------------------------------------------------------------
constexpr int kFastSteps = 6;

template <typename T>
struct ChainRegs {
  int n;
  int first;  // bit 0: 1 = immediate, 0 = load; bits 4..: input index
  T first_imm;
  int op[kFastSteps];
  int leaf[kFastSteps];  // bit 0: leaf is an immediate; bits 4..: input index
  T imm[kFastSteps];
};

template <typename T>
__device__ __forceinline__ void chain_decode(const ChainProg<T> &pr, ChainRegs<T> &r) {
  r.n = pr.n_steps;
  r.first = (pr.first_kind == LEAF_IMM ? 1 : 0) | ((int)pr.first_idx << 4);
  r.first_imm = pr.first_imm;
#pragma unroll
  for (int s = 0; s < kFastSteps; ++s) {
    r.op[s] = pr.op[s];
    r.leaf[s] = (pr.kind[s][1] == LEAF_IMM ? 1 : 0) | ((int)pr.idx[s][1] << 4);
    r.imm[s] = pr.imm[s][1];
  }
}

template <typename T, int NIN, int N>
__device__ __forceinline__ void chain_eval_fast(const ChainRegs<T> &r, const T (&w)[NIN][N], T (&run)[N]) {
  chain_first<T, NIN, N>(r.first & 1, r.first >> 4, r.first_imm, w, run);
#pragma unroll
  for (int s = 0; s < kFastSteps; ++s) {
    if (s < r.n) chain_step_binary<T, NIN, N, false>(r.op[s], r.leaf[s] & 1, r.leaf[s] >> 4, r.imm[s], w, run);
  }
}

// ---------------------------------------------------------------------------
// Reduction state: value plus (for argmax) the position along the reduced axis.
// ---------------------------------------------------------------------------
enum { ROP_SUM = 0, ROP_MAX = 1, ROP_ARGMAX = 2 };


template <typename T> __device__ __forceinline__ T lowest_of();
template <> __device__ __forceinline__ float lowest_of<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double lowest_of<double>() { return -INFINITY; }
template <> __device__ __forceinline__ int lowest_of<int>() { return INT32_MIN; }

template <typename T, int ROP>
struct Acc {
  T v;
  int i;
  __device__ __forceinline__ void init() {
    v = (ROP == ROP_SUM) ? (T)0 : lowest_of<T>();
    i = 0x7fffffff;
  }
  __device__ __forceinline__ void add(T x, int idx) {
    if (ROP == ROP_SUM) v = v + x;
    else if (ROP == ROP_MAX) v = x > v ? x : v;
    else {
      if (x > v || (x == v && idx < i)) { v = x; i = idx; }
    }
  }
  // For a thread's own stream, which reaches each accumulator in increasing index order: a tie can never carry a
  // smaller index there, so argmax needs one comparison (ties across threads are settled by merge()).
  __device__ __forceinline__ void add_stream(T x, int idx) {
    if (ROP == ROP_ARGMAX) {
      if (x > v) { v = x; i = idx; }
    } else add(x, idx);
  }
  __device__ __forceinline__ void merge(T ov, int oi) { add(ov, oi); }
};

template <typename T>
__device__ __forceinline__ T shfl_xor_t(T v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }

template <typename T, int ROP>
__device__ __forceinline__ void warp_combine(Acc<T, ROP> &a) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    T ov = shfl_xor_t<T>(a.v, m);
    int oi = (ROP == ROP_ARGMAX) ? __shfl_xor_sync(0xffffffffu, a.i, m) : 0;
    a.merge(ov, oi);
  }
}

// ---------------------------------------------------------------------------
// What happens to a finished reduction value: mean divide, epilogue program,
// conversion to the output dtype, store. Shared by all reduce kernels.
// ---------------------------------------------------------------------------
template <typename T>
struct EpiParams {
  void *out;
  int out_dtype;
  int is_mean;
  int is_argmax;
  T count;  // reduced element count, in the compute type
  int n_epi_in;
  int out_ndim;  // dims of the (merged) output index space used by epilogue operands
  int64_t out_size[kMaxDims];
  const void *epi_ptr[kMaxIn];
  int epi_dtype[kMaxIn];
  int64_t epi_stride[kMaxIn][kMaxDims];
  VmProg<T> prog;  // n == 0: store the value unchanged
  // The two commonest epilogues skip the interpreter (which costs a few hundred
  // instructions per output): 1 = one unary op on the result (exp, log, cast),
  // 2 = one binary op with an immediate (scale, shift, clamp).
  int fast_kind;
  int fast_op;
  int fast_rev;  // kind 2: the immediate is the first operand
  T fast_imm;
};

template <typename T>
__device__ __forceinline__ void finish_output(const EpiParams<T> &ep, int64_t o, T acc, int idx) {
  if (ep.is_argmax) {
    ((int *)ep.out)[o] = (idx == 0x7fffffff) ? 0 : idx;
    return;
  }
  if (ep.is_mean) acc = acc / ep.count;
  if (ep.fast_kind == 1) {
    acc = apply_unary<T>(ep.fast_op, acc);
  } else if (ep.fast_kind == 2) {
    acc = ep.fast_rev ? apply_binary<T>(ep.fast_op, ep.fast_imm, acc) : apply_binary<T>(ep.fast_op, acc, ep.fast_imm);
  } else if (ep.prog.n > 0) {
    T v[kMaxInstr];
    int64_t offs[kMaxIn];
    if (ep.n_epi_in > 0) {
      for (int k = 0; k < ep.n_epi_in; ++k) offs[k] = 0;
      int64_t rem = o;
      for (int d = ep.out_ndim - 1; d >= 0; --d) {
        int64_t c = rem % ep.out_size[d];
        rem /= ep.out_size[d];
        for (int k = 0; k < ep.n_epi_in; ++k) offs[k] += c * ep.epi_stride[k][d];
      }
    }
    vm_eval<T>(ep.prog, v, acc, [&](int k) { return load_as<T>(ep.epi_ptr[k], ep.epi_dtype[k], offs[k]); });
    acc = v[ep.prog.n - 1];
  }
  store_as<T>(ep.out, ep.out_dtype, o, acc);
}

}  // namespace pgb
