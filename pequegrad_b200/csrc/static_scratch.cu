// pgb_fused_reduce_noalloc: the fused reduce for callers that must not
// allocate device memory.
//
// Who that is: code that runs where an allocation is forbidden or would
// break an invariant of the caller — a host that has handed the whole device
// to its own arena (the reference's "custom" allocator takes 40 % of free
// memory up front, csrc/cuda/mem.cu:13-142, and other frameworks take nearly
// all of it), a latency-critical serving loop that forbids driver calls which
// may synchronise or fail under memory pressure, or a sandboxed plugin that is
// only given pointers. Split reductions (few outputs, long reduced axis) need
// a few hundred KB of partial results between their two kernels; the regular
// entry point takes that from the caller or from cudaMallocAsync. This one
// takes it from a fixed array that is part of the loaded library image.
#include <mutex>

#include "reduce_common.cuh"

// Lives in every device's copy of the module from load until exit.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PGB_NOALLOC_SCRATCH_BYTES];

namespace {

std::mutex g_mu;
void *g_scratch_ptr[64] = {nullptr};
bool g_scratch_known[64] = {false};

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a
// device address; the address on the CURRENT device has to be asked for.
// Done once per device, with that device current.
int scratch_on_current_device(void **out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    pgb::set_error("fused_reduce_noalloc: no current CUDA device");
    return PGB_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_known[dev]) {
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      pgb::set_error(std::string("fused_reduce_noalloc: cannot resolve the built-in scratch array: ") + cudaGetErrorString(e));
      return PGB_ERR_CUDA;
    }
    g_scratch_ptr[dev] = p;
    g_scratch_known[dev] = true;
  }
  *out = g_scratch_ptr[dev];
  return PGB_OK;
}

}  // namespace

extern "C" PGB_API int pgb_fused_reduce_noalloc(const pgb_tensor *in, int n_in, const pgb_tensor *out, int reduce_op,
                                                const int32_t *axes, int n_axes, const pgb_instr *prologue, int n_pro,
                                                const pgb_tensor *epi_in, int n_epi_in, const pgb_instr *epilogue, int n_epi,
                                                void *stream) {
  // how much scratch would the regular entry point use for this problem?
  size_t need = 0;
  int st = pgb_fused_reduce_workspace(in, n_in, out, reduce_op, axes, n_axes, &need);
  if (st != PGB_OK) return st;
  if (need > (size_t)PGB_NOALLOC_SCRATCH_BYTES) {
    pgb::set_error("fused_reduce_noalloc: this reduction needs " + std::to_string(need) + " bytes of scratch but the built-in array holds " +
                   std::to_string((size_t)PGB_NOALLOC_SCRATCH_BYTES) + "; use pgb_fused_reduce with a workspace of your own");
    return PGB_ERR_WORKSPACE;
  }
  void *scratch = nullptr;
  if (need > 0) {
    st = scratch_on_current_device(&scratch);
    if (st != PGB_OK) return st;
  }
  // Nothing in the scratch has to start at zero: the first kernel writes every
  // partial result before the second one reads it.
  // `need` was planned without the prologue. That is the size the launch uses: how a reduction is split depends on
  // shapes and strides alone, and a prologue the fast kernels cannot take moves the call to the generic kernel, which
  // needs no scratch. Should the two ever disagree, the launch below is told not to allocate and refuses instead.
  return pgb::fused_reduce_run(in, n_in, out, reduce_op, axes, n_axes, prologue, n_pro, epi_in, n_epi_in, epilogue, n_epi, scratch,
                               need > 0 ? (size_t)PGB_NOALLOC_SCRATCH_BYTES : 0, stream, /*no_alloc=*/true);
}
