// Collectives of the batch-sharded path over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The data-parallel workloads exchange almost nothing: the int8 MLP needs the maximum of one float per layer over
// all row shards (its per-tensor activation scale) and, at the end, every rank's [rows / P, 10] slab of logits. A
// library collective costs tens of microseconds of launch and synchronisation for each of these, which is as long
// as a layer of an 8192-row shard. Here each exchange is one small kernel that stores straight into the peers'
// memory (plain stores through peer mappings opened with CUDA IPC; no multicast, no TMA) and then polls its own
// memory until every peer's contribution has arrived. The reference has no counterpart: its "devices" are aliases of
// one GPU and its all_reduce is a Python loop (pequegrad/distrib/__init__.py:4-29).
//
// Every rank runs the same sequence of these calls. A contribution carries the number of the call it belongs to
// (the epoch), packed with the value into one 64-bit store, so a reader can never take a stale value for a fresh
// one; two banks alternate by epoch parity, and a rank cannot be two calls ahead of a peer (it needs the peer's
// contribution to finish a call), so a bank is never overwritten before it was read. Every wait is bounded (2^21
// polls with a 100 ns sleep, one to two seconds; pgb_peer_poll_limit changes it): a rank whose peer never arrives
// records the error word that pgb_device_error() reads and returns.
#include <atomic>
#include <cstring>

#include "reduce_common.cuh"
#include "gemm.hpp"

namespace pgb {

namespace {

constexpr int kMaxPeers = PGB_MAX_PEERS;
std::atomic<unsigned> g_peer_polls{1u << 21};  // x (~100 ns of sleep + one system-scope load) per poll

struct PeerCtrl {
  unsigned long long max_slot[2][kMaxPeers];     // [epoch parity][source rank]: (epoch << 32) | float bits
  unsigned long long gather_flag[2][kMaxPeers];  // [epoch parity][source rank]: epoch
  unsigned int epoch_max, epoch_gather;          // this rank's call counters (written by this rank's kernels only)
  unsigned int ticket;
  unsigned int pad;
};

struct PeerPtrs {
  PeerCtrl *ctrl[kMaxPeers];
  void *dst[kMaxPeers];
};

__device__ __forceinline__ unsigned long long ld_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Waits (bounded) until the local slot carries `epoch` in its upper half. Returns false on a timeout.
__device__ __forceinline__ bool wait_epoch(const unsigned long long *slot, unsigned epoch, unsigned long long &v, unsigned polls) {
  for (unsigned i = 0; i < polls; ++i) {
    v = ld_sys(slot);
    if ((unsigned)(v >> 32) == epoch) return true;
    __nanosleep(100);
  }
  return false;
}

__global__ void __launch_bounds__(32) peer_max_kernel(float *value, const __grid_constant__ PeerPtrs pp, int rank, int world, unsigned polls,
                                                      int *err) {
  if (*(volatile int *)err != 0) return;
  PeerCtrl *me = pp.ctrl[rank];
  const int t = threadIdx.x;
  unsigned epoch = 0;
  if (t == 0) epoch = ++me->epoch_max;
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  const int bank = epoch & 1;
  const float mine = *value;
  if (t < world) st_sys(&pp.ctrl[t]->max_slot[bank][rank], ((unsigned long long)epoch << 32) | __float_as_uint(mine));
  float m = 0.f;
  bool ok = true;
  if (t < world) {
    unsigned long long v = 0;
    ok = wait_epoch(&me->max_slot[bank][t], epoch, v, polls);
    m = __uint_as_float((unsigned)(v & 0xffffffffu));
  }
  if (!__all_sync(0xffffffffu, ok)) {
    if (t == 0) atomicCAS(err, 0, (10 << 16) | (rank & 0xffff));
    return;
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, k));
  if (t == 0) *value = m;
}

// grid = world x chunks CTAs: CTA (peer, chunk) copies a chunk of this rank's slab into the peer's buffer at
// rank * bytes; the last CTA to finish announces the slab to every peer and waits for theirs.
__global__ void __launch_bounds__(256) peer_gather_kernel(const uint4 *__restrict__ src, size_t bytes, const __grid_constant__ PeerPtrs pp,
                                                          int rank, int world, int chunks, unsigned polls, int *err) {
  if (*(volatile int *)err != 0) return;
  PeerCtrl *me = pp.ctrl[rank];
  const int peer = blockIdx.x / chunks, chunk = blockIdx.x - peer * chunks;
  const size_t nvec = bytes >> 4;
  uint4 *dst = reinterpret_cast<uint4 *>(static_cast<char *>(pp.dst[peer]) + (size_t)rank * bytes);
  for (size_t i = (size_t)chunk * 256 + threadIdx.x; i < nvec; i += (size_t)chunks * 256) dst[i] = __ldg(src + i);
  if (chunk == 0 && threadIdx.x < (bytes & 15)) {
    const size_t o = (nvec << 4) + threadIdx.x;
    reinterpret_cast<char *>(dst)[o] = reinterpret_cast<const char *>(src)[o];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = atomicInc(&me->ticket, gridDim.x - 1) == gridDim.x - 1;
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence_system();
  const int t = threadIdx.x;
  unsigned epoch = 0;
  if (t == 0) epoch = ++me->epoch_gather;
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  const int bank = epoch & 1;
  if (t < world) st_sys(&pp.ctrl[t]->gather_flag[bank][rank], (unsigned long long)epoch << 32);
  bool ok = true;
  if (t < world) {
    unsigned long long v = 0;
    ok = wait_epoch(&me->gather_flag[bank][t], epoch, v, polls);
  }
  if (!__all_sync(0xffffffffu, ok) && t == 0) atomicCAS(err, 0, (11 << 16) | (rank & 0xffff));
}

int fill_ptrs(PeerPtrs &pp, void *const *peer_ctrl, void *const *peer_dst, int rank, int world, const char *what) {
  if (!peer_ctrl || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) {
    set_error(std::string(what) + ": between 1 and 16 peers and a rank among them are required");
    return PGB_ERR_INVALID_ARG;
  }
  std::memset(&pp, 0, sizeof pp);
  for (int r = 0; r < world; ++r) {
    if (!peer_ctrl[r] || (peer_dst && !peer_dst[r])) { set_error(std::string(what) + ": null peer pointer"); return PGB_ERR_INVALID_ARG; }
    pp.ctrl[r] = static_cast<PeerCtrl *>(peer_ctrl[r]);
    pp.dst[r] = peer_dst ? peer_dst[r] : nullptr;
  }
  return PGB_OK;
}

}  // namespace

}  // namespace pgb

using namespace pgb;

extern "C" {

PGB_API size_t pgb_peer_ctrl_bytes(void) { return sizeof(PeerCtrl); }

PGB_API unsigned int pgb_peer_poll_limit(unsigned int polls) {
  return polls ? g_peer_polls.exchange(polls) : g_peer_polls.load();
}

PGB_API int pgb_peer_alloc(size_t bytes, void **ptr) {
  if (!ptr || bytes == 0) { set_error("peer_alloc: null result pointer or zero size"); return PGB_ERR_INVALID_ARG; }
  void *p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess) {
    cudaGetLastError();
    if (p) cudaFree(p);
    set_error("peer_alloc: device allocation failed");
    return PGB_ERR_CUDA;
  }
  *ptr = p;
  return PGB_OK;
}

PGB_API int pgb_peer_free(void *ptr) {
  if (ptr && cudaFree(ptr) != cudaSuccess) { cudaGetLastError(); set_error("peer_free: cudaFree failed"); return PGB_ERR_CUDA; }
  return PGB_OK;
}

PGB_API int pgb_peer_export(const void *ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  if (!ptr || !handle) { set_error("peer_export: null argument"); return PGB_ERR_INVALID_ARG; }
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(ptr));
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(std::string("peer_export: cudaIpcGetMemHandle failed: ") + cudaGetErrorString(e));
    return PGB_ERR_CUDA;
  }
  std::memcpy(handle, &h, 64);
  return PGB_OK;
}

PGB_API int pgb_peer_open(const unsigned char handle[64], void **ptr) {
  if (!handle || !ptr) { set_error("peer_open: null argument"); return PGB_ERR_INVALID_ARG; }
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  void *p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(std::string("peer_open: cudaIpcOpenMemHandle failed: ") + cudaGetErrorString(e));
    return PGB_ERR_CUDA;
  }
  *ptr = p;
  return PGB_OK;
}

PGB_API int pgb_peer_close(void *ptr) {
  if (ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) { cudaGetLastError(); set_error("peer_close: cudaIpcCloseMemHandle failed"); return PGB_ERR_CUDA; }
  return PGB_OK;
}

PGB_API int pgb_peer_allreduce_max_f32(float *value, void *const *peer_ctrl, int rank, int world, void *stream) {
  if (!value) { set_error("peer_allreduce_max: null value"); return PGB_ERR_INVALID_ARG; }
  PeerPtrs pp;
  int st = fill_ptrs(pp, peer_ctrl, nullptr, rank, world, "peer_allreduce_max");
  if (st != PGB_OK) return st;
  int *err = gemm_error_word();
  if (!err) { set_error("peer_allreduce_max: cannot resolve the device error word"); return PGB_ERR_CUDA; }
  peer_max_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(value, pp, rank, world, g_peer_polls.load(), err);
  count_launch();
  return check_launch("peer_max_kernel");
}

PGB_API int pgb_peer_allgather(const void *src, size_t bytes, void *const *peer_dst, void *const *peer_ctrl, int rank, int world, void *stream) {
  if (!src || !peer_dst) { set_error("peer_allgather: null buffer"); return PGB_ERR_INVALID_ARG; }
  if (reinterpret_cast<uintptr_t>(src) & 15 || bytes % 16) { set_error("peer_allgather: the slab must be 16-byte aligned and a multiple of 16 bytes"); return PGB_ERR_UNSUPPORTED; }
  PeerPtrs pp;
  int st = fill_ptrs(pp, peer_ctrl, peer_dst, rank, world, "peer_allgather");
  if (st != PGB_OK) return st;
  int *err = gemm_error_word();
  if (!err) { set_error("peer_allgather: cannot resolve the device error word"); return PGB_ERR_CUDA; }
  // stores to a peer are posted: what bounds a copy is how many a CTA keeps in flight, so 16 KB per CTA and up to 64
  // CTAs per peer (a 1.3 MB slab from 32 CTAs took 25 us)
  int chunks = (int)((bytes + (16 << 10) - 1) / (16 << 10));
  chunks = chunks < 1 ? 1 : (chunks > 64 ? 64 : chunks);
  peer_gather_kernel<<<world * chunks, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint4 *>(src), bytes, pp, rank, world, chunks,
                                                                             g_peer_polls.load(), err);
  count_launch();
  return check_launch("peer_gather_kernel");
}

}  // extern "C"
