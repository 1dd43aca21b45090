// Shared declarations of the reduce kernel families and their host launchers.
#pragma once
#include <string>

#include "common.cuh"
#include "plan.hpp"
#include "program.hpp"

namespace pgb {

// Everything a launcher needs, assembled once by the ABI entry point.
struct ReduceJob {
  CanonReduce c;
  const pgb_tensor *in;  // n_in original descriptors (pointers, dtypes)
  const pgb_tensor *out;
  int rop;       // ROP_SUM / ROP_MAX / ROP_ARGMAX
  int is_mean;
  int cdtype;    // compute dtype (PGB_F32 / PGB_F64 / PGB_I32)
  const pgb_instr *pro; int n_pro;
  const pgb_instr *epi; int n_epi;
  const pgb_tensor *epi_in; int n_epi_in;
  void *workspace; size_t workspace_bytes;
  cudaStream_t stream;
  bool dry_run;        // plan only: fill `desc` / `ws_needed`, launch nothing
  bool no_alloc = false;  // a split reduction without a caller workspace is refused instead of allocating one
  std::string desc;
  size_t ws_needed = 0;
};

// Kernel-side parameter blocks ------------------------------------------------
template <typename T, int NIN>
struct RowParams {
  const void *in[NIN];
  int64_t kstr[NIN][3];  // kept dims (outer -> inner), element strides, 0-padded
  int64_t r1str[NIN];    // outer reduced dim
  int64_t cstr[NIN];     // inner reduced dim: 1 or 0 (broadcast)
  int64_t ksize1, ksize2;
  int nk;  // number of kept dims in use (0..3)
  int64_t n_out, C, R1;
  int64_t chunk;    // inner-dim elements per segment
  int64_t nchunks;  // segments per (row, r1)
  int64_t S;        // work items per row
  T *part_v;
  int *part_i;
  ChainProg<T> pro;
  EpiParams<T> epi;
};

template <typename T, int NIN>
struct ColParams {
  const void *in[NIN];
  int64_t bstr[NIN][2];  // the other kept dims ("batch"), element strides
  int64_t jstr[NIN];     // memory-contiguous kept dim: 1 or 0
  int64_t rstr[NIN][2];  // reduced dims (outer, inner)
  int64_t bsize1;        // size of batch dim 1 (dim 0 implied)
  int64_t bout[2];       // output strides of the batch dims
  int64_t jout;          // output stride of the contiguous kept dim
  int64_t nbatch, J, R0, R1, R;
  int64_t ntiles;
  int64_t S, rows_per_split;
  int64_t n_out;
  T *part_v;
  int *part_i;
  unsigned int *tickets;  // one counter per (batch, column tile) of a split reduction, or null: a finish kernel combines
  ChainProg<T> pro;
  EpiParams<T> epi;
};

template <typename T>
struct GenParams {
  int n_in;
  const void *in[kMaxIn];
  int dt[kMaxIn];
  int nk, nr;
  int64_t ksize[kMaxDims], rsize[kMaxDims];
  int64_t kin[kMaxIn][kMaxDims], rin[kMaxIn][kMaxDims];
  int64_t n_out, n_red;
  int G;
  VmProg<T> pro;
  EpiParams<T> epi;
};

// Fills the epilogue block from the job. Returns "" or an error message.
template <typename T>
std::string make_epi(const ReduceJob &j, EpiParams<T> &e);

// Each returns: 1 launched (or planned), 0 not applicable, <0 pgb_status error.
// The body of pgb_fused_reduce; `no_alloc` makes a split reduction without a workspace fail instead of allocating.
int fused_reduce_run(const pgb_tensor *in, int n_in, const pgb_tensor *out, int reduce_op, const int32_t *axes, int n_axes,
                     const pgb_instr *prologue, int n_pro, const pgb_tensor *epi_in, int n_epi_in, const pgb_instr *epilogue, int n_epi,
                     void *workspace, size_t workspace_bytes, void *stream, bool no_alloc);
int launch_reduce_row(ReduceJob &j);
int launch_reduce_col(ReduceJob &j);
int launch_reduce_plane(ReduceJob &j);
int launch_reduce_generic(ReduceJob &j);
// Ticket counters for the single-launch split reduction: `count` zeroed counters that only launches on `stream`
// use (launches on one stream run one after another, and the last CTA of each tile leaves its counter at zero).
// Null when `count` is too large or too many streams are in use: the caller then runs the finish kernel.
unsigned int *split_tickets(cudaStream_t stream, int64_t count);
// Second stage of split reductions: combines S partials per output.
int launch_reduce_finish(ReduceJob &j, const void *part_v, const int *part_i, int64_t S);

void set_error(const std::string &msg);
int check_launch(const char *what);
void count_launch();
int sm_count();

// ---------------------------------------------------------------------------
template <typename T>
std::string make_epi(const ReduceJob &j, EpiParams<T> &e) {
  e = EpiParams<T>();
  e.out = j.out->data;
  e.out_dtype = j.out->dtype;
  e.is_mean = j.is_mean;
  e.is_argmax = (j.rop == ROP_ARGMAX);
  e.count = (T)j.c.n_red;
  e.n_epi_in = j.n_epi_in;
  e.out_ndim = j.c.out_ndim;
  for (int d = 0; d < j.c.out_ndim; ++d) e.out_size[d] = j.c.out_size[d];
  for (int k = 0; k < j.n_epi_in; ++k) {
    const pgb_tensor &t = j.epi_in[k];
    e.epi_ptr[k] = t.data;
    e.epi_dtype[k] = t.dtype;
    const int sz = dtype_size(t.dtype);
    if (sz == 0) return "fused_reduce: unknown dtype of an epilogue operand";
    if (t.ndim != j.in[0].ndim) return "fused_reduce: epilogue operands must have the rank of the inputs";
    for (int d = 0; d < j.c.out_ndim; ++d) {
      const int ax = j.c.out_axis[d];
      if (t.shape[ax] != j.c.out_size[d]) return "fused_reduce: epilogue operand does not match the output shape";
      if (t.stride_bytes[ax] % sz) return "fused_reduce: stride is not a multiple of the element size";
      e.epi_stride[k][d] = t.stride_bytes[ax] / sz;
    }
  }
  to_vm<T>(j.epi, j.n_epi, e.prog);
  // epilogues that need no interpreter
  const pgb_instr *p = j.epi;
  if (j.n_epi == 2 && p[0].op == PGB_OP_ACC && op_is_unary(p[1].op) && p[1].a == 0) {
    e.fast_kind = 1;
    e.fast_op = p[1].op;
  } else if (j.n_epi == 3 && op_is_binary(p[2].op)) {
    const int ia = p[2].a, ib = p[2].b;
    if (ia >= 0 && ia < 2 && ib >= 0 && ib < 2 && ia != ib && p[ia].op + p[ib].op == PGB_OP_ACC + PGB_OP_IMM &&
        (p[ia].op == PGB_OP_ACC || p[ia].op == PGB_OP_IMM)) {
      e.fast_kind = 2;
      e.fast_op = p[2].op;
      e.fast_rev = p[ia].op == PGB_OP_IMM;
      e.fast_imm = (T)p[e.fast_rev ? ia : ib].imm;
    }
  }
  return "";
}

}  // namespace pgb
