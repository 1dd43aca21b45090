// extern "C" entry points: argument validation, planning, launch. Nothing here
// throws across the boundary and nothing synchronises the device.
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

#include "program.hpp"
#include "reduce_common.cuh"

namespace pgb {

static thread_local std::string g_last_error;
static std::atomic<uint64_t> g_launches{0};

void set_error(const std::string &msg) { g_last_error = msg; }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_launch(const char *what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error(std::string(what) + ": " + cudaGetErrorString(e));
    return PGB_ERR_CUDA;
  }
  return PGB_OK;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static bool device_ok() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    set_error("no CUDA device: this library has no CPU fallback");
    return false;
  }
  return true;
}

int run_fused_elementwise(const pgb_tensor *in, int n_in, const pgb_tensor *out, int n_out, const pgb_instr *prog, int n,
                          const int16_t *out_vals, cudaStream_t stream);

int run_softmax_rows(const pgb_tensor *x, const pgb_tensor *y, int causal, cudaStream_t stream);
int run_layernorm_rows(const pgb_tensor *x, const pgb_tensor *gamma, const pgb_tensor *beta, float eps, const pgb_tensor *y,
                       cudaStream_t stream);

int run_embedding_rows(const pgb_tensor *ids, const pgb_tensor *wte, const pgb_tensor *wpe, int64_t T, const pgb_tensor *out,
                       cudaStream_t stream);

static int build_reduce_job(ReduceJob &j, const pgb_tensor *in, int n_in, const pgb_tensor *out, int reduce_op, const int32_t *axes,
                            int n_axes, const pgb_instr *prologue, int n_pro, const pgb_tensor *epi_in, int n_epi_in,
                            const pgb_instr *epilogue, int n_epi) {
  if (!in || !out) { set_error("fused_reduce: null tensor"); return PGB_ERR_INVALID_ARG; }
  if (n_axes < 0 || n_axes > PGB_MAX_DIMS || (n_axes > 0 && !axes)) { set_error("fused_reduce: bad axes"); return PGB_ERR_INVALID_ARG; }
  if (reduce_op < PGB_REDUCE_SUM || reduce_op > PGB_REDUCE_ARGMAX) { set_error("fused_reduce: unknown reduce op"); return PGB_ERR_INVALID_ARG; }
  std::string err = canonicalise_reduce(in, n_in, axes, n_axes, j.c);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  // a missing prologue means "LOAD 0"
  static const pgb_instr kLoad0 = {PGB_OP_LOAD, 0, 0, 0, 0, 0.0};
  if (n_pro == 0) { prologue = &kLoad0; n_pro = 1; }
  err = validate_program(prologue, n_pro, n_in, false, "fused_reduce prologue");
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  if (n_epi_in < 0 || n_epi_in > PGB_MAX_INPUTS) { set_error("fused_reduce: too many epilogue operands"); return PGB_ERR_INVALID_ARG; }
  err = validate_program(epilogue, n_epi, n_epi_in, true, "fused_reduce epilogue");
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  if (reduce_op == PGB_REDUCE_ARGMAX) {
    if (n_axes != 1) { set_error("argmax: exactly one axis is supported"); return PGB_ERR_INVALID_ARG; }
    if (out->dtype != PGB_I32) { set_error("argmax: the output must be int32"); return PGB_ERR_INVALID_ARG; }
    if (n_epi != 0) { set_error("argmax: no epilogue is applied to an index"); return PGB_ERR_INVALID_ARG; }
  }
  if (dtype_size(out->dtype) == 0) { set_error("fused_reduce: unknown output dtype"); return PGB_ERR_INVALID_ARG; }
  if (numel_of(*out) != j.c.n_out) { set_error("fused_reduce: output shape does not match the reduced shape"); return PGB_ERR_INVALID_ARG; }
  if (!is_contiguous(*out)) { set_error("fused_reduce: the output must be contiguous"); return PGB_ERR_INVALID_ARG; }
  if (j.c.n_red == 0 && j.c.n_out > 0) { set_error("fused_reduce: cannot reduce over an empty axis"); return PGB_ERR_INVALID_ARG; }
  if (j.c.n_red > 2147483647LL && reduce_op == PGB_REDUCE_ARGMAX) { set_error("argmax: axis too long for an int32 index"); return PGB_ERR_UNSUPPORTED; }
  j.in = in;
  j.out = out;
  j.rop = reduce_op == PGB_REDUCE_MAX ? ROP_MAX : (reduce_op == PGB_REDUCE_ARGMAX ? ROP_ARGMAX : ROP_SUM);
  j.is_mean = reduce_op == PGB_REDUCE_MEAN;
  j.cdtype = compute_dtype(in, n_in, out->dtype);
  j.pro = prologue;
  j.n_pro = n_pro;
  j.epi = epilogue;
  j.n_epi = n_epi;
  j.epi_in = epi_in;
  j.n_epi_in = n_epi_in;
  return PGB_OK;
}

static int plan_and_launch(ReduceJob &j) {
  if (j.c.n_out == 0) { j.desc = "empty"; return PGB_OK; }
  int r = launch_reduce_row(j);
  if (r == 0) r = launch_reduce_col(j);
  if (r == 0) r = launch_reduce_plane(j);
  if (r == 0) r = launch_reduce_generic(j);
  return r == 1 ? PGB_OK : (r == 0 ? PGB_ERR_UNSUPPORTED : r);
}

int fused_reduce_run(const pgb_tensor *in, int n_in, const pgb_tensor *out, int reduce_op, const int32_t *axes, int n_axes,
                     const pgb_instr *prologue, int n_pro, const pgb_tensor *epi_in, int n_epi_in, const pgb_instr *epilogue, int n_epi,
                     void *workspace, size_t workspace_bytes, void *stream, bool no_alloc) {
  g_last_error.clear();
  ReduceJob j;
  int st = build_reduce_job(j, in, n_in, out, reduce_op, axes, n_axes, prologue, n_pro, epi_in, n_epi_in, epilogue, n_epi);
  if (st != PGB_OK) return st;
  if (!device_ok()) return PGB_ERR_CUDA;
  j.workspace = workspace;
  j.workspace_bytes = workspace_bytes;
  j.stream = (cudaStream_t)stream;
  j.dry_run = false;
  j.no_alloc = no_alloc;
  return plan_and_launch(j);
}

}  // namespace pgb

using namespace pgb;

extern "C" {

const char *pgb_status_string(int status) {
  switch (status) {
    case PGB_OK: return "ok";
    case PGB_ERR_INVALID_ARG: return "invalid argument";
    case PGB_ERR_UNSUPPORTED: return "not implemented";
    case PGB_ERR_CUDA: return "CUDA error";
    case PGB_ERR_TIMEOUT: return "device-side wait timed out";
    case PGB_ERR_WORKSPACE: return "workspace too small";
    default: return "unknown status";
  }
}

const char *pgb_last_error(void) { return g_last_error.c_str(); }
const char *pgb_version(void) { return "pgb200 0.1 (sm_100a)"; }
uint64_t pgb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int pgb_fused_elementwise(const pgb_tensor *in, int n_in, const pgb_tensor *out, int n_out, const pgb_instr *prog, int n_instr,
                          const int16_t *out_vals, void *stream) {
  g_last_error.clear();
  if (!out || n_out < 1 || n_out > PGB_MAX_OUTPUTS || !out_vals || (n_in > 0 && !in)) {
    set_error("fused_elementwise: between 1 and 4 outputs are required");
    return PGB_ERR_INVALID_ARG;
  }
  std::string err = validate_program(prog, n_instr, n_in, false, "fused_elementwise");
  if (!err.empty() || n_instr == 0) { set_error(err.empty() ? "fused_elementwise: empty program" : err); return PGB_ERR_INVALID_ARG; }
  for (int o = 0; o < n_out; ++o) {
    if (out_vals[o] < 0 || out_vals[o] >= n_instr) { set_error("fused_elementwise: output refers to a value that does not exist"); return PGB_ERR_INVALID_ARG; }
    if (dtype_size(out[o].dtype) == 0) { set_error("fused_elementwise: unknown output dtype"); return PGB_ERR_INVALID_ARG; }
    if (out[o].ndim != out[0].ndim) { set_error("fused_elementwise: outputs must have one shape"); return PGB_ERR_INVALID_ARG; }
    for (int d = 0; d < out[0].ndim; ++d)
      if (out[o].shape[d] != out[0].shape[d]) { set_error("fused_elementwise: outputs must have one shape"); return PGB_ERR_INVALID_ARG; }
    if (!is_contiguous(out[o])) { set_error("fused_elementwise: outputs must be contiguous"); return PGB_ERR_INVALID_ARG; }
  }
  if (!device_ok()) return PGB_ERR_CUDA;
  return run_fused_elementwise(in, n_in, out, n_out, prog, n_instr, out_vals, (cudaStream_t)stream);
}

int pgb_fused_reduce(const pgb_tensor *in, int n_in, const pgb_tensor *out, int reduce_op, const int32_t *axes, int n_axes,
                     const pgb_instr *prologue, int n_pro, const pgb_tensor *epi_in, int n_epi_in, const pgb_instr *epilogue, int n_epi,
                     void *workspace, size_t workspace_bytes, void *stream) {
  return fused_reduce_run(in, n_in, out, reduce_op, axes, n_axes, prologue, n_pro, epi_in, n_epi_in, epilogue, n_epi, workspace,
                          workspace_bytes, stream, false);
}

int pgb_fused_reduce_workspace(const pgb_tensor *in, int n_in, const pgb_tensor *out, int reduce_op, const int32_t *axes, int n_axes,
                               size_t *bytes_out) {
  g_last_error.clear();
  if (!bytes_out) { set_error("fused_reduce_workspace: null result pointer"); return PGB_ERR_INVALID_ARG; }
  ReduceJob j;
  int st = build_reduce_job(j, in, n_in, out, reduce_op, axes, n_axes, nullptr, 0, nullptr, 0, nullptr, 0);
  if (st != PGB_OK) return st;
  j.workspace = nullptr;
  j.workspace_bytes = 0;
  j.stream = nullptr;
  j.dry_run = true;
  st = plan_and_launch(j);
  *bytes_out = j.ws_needed;
  return st;
}

int pgb_fused_reduce_describe(const pgb_tensor *in, int n_in, const pgb_tensor *out, int reduce_op, const int32_t *axes, int n_axes,
                              const pgb_instr *prologue, int n_pro, char *buf, size_t buf_len) {
  g_last_error.clear();
  if (!buf || buf_len == 0) { set_error("fused_reduce_describe: null buffer"); return PGB_ERR_INVALID_ARG; }
  ReduceJob j;
  int st = build_reduce_job(j, in, n_in, out, reduce_op, axes, n_axes, prologue, n_pro, nullptr, 0, nullptr, 0);
  if (st != PGB_OK) return st;
  j.workspace = nullptr;
  j.workspace_bytes = 0;
  j.stream = nullptr;
  j.dry_run = true;
  st = plan_and_launch(j);
  snprintf(buf, buf_len, "%s", j.desc.c_str());
  return st;
}

int pgb_softmax_rows(const pgb_tensor *x, const pgb_tensor *y, int causal, void *stream) {
  g_last_error.clear();
  if (!device_ok()) return PGB_ERR_CUDA;
  return run_softmax_rows(x, y, causal, (cudaStream_t)stream);
}

int pgb_layernorm_rows(const pgb_tensor *x, const pgb_tensor *gamma, const pgb_tensor *beta, float eps, const pgb_tensor *y,
                       void *stream) {
  g_last_error.clear();
  if (!device_ok()) return PGB_ERR_CUDA;
  return run_layernorm_rows(x, gamma, beta, eps, y, (cudaStream_t)stream);
}

int pgb_embedding_rows(const pgb_tensor *ids, const pgb_tensor *wte, const pgb_tensor *wpe, int64_t T, const pgb_tensor *out, void *stream) {
  g_last_error.clear();
  if (!device_ok()) return PGB_ERR_CUDA;
  return run_embedding_rows(ids, wte, wpe, T, out, (cudaStream_t)stream);
}

}  // extern "C"
