// Dispatcher of the col reduce family; the kernels are instantiated in reduce_col_*.cu
// (one translation unit per input type and input count, so they compile in parallel).
#include <mutex>

#include "reduce_col.cuh"

namespace pgb {

// Ticket counters of the single-launch split reductions. They live in the library image (zero when the module is
// loaded, and every launch leaves them at zero), one bank per stream so that launches which may overlap never share
// a counter. A kernel that is killed mid-flight would leave a bank dirty, but by then the context is lost anyway.
constexpr int kTicketBanks = 16;
constexpr int kTicketsPerBank = 4096;
static __device__ unsigned int g_split_tickets[kTicketBanks][kTicketsPerBank];

unsigned int *split_tickets(cudaStream_t stream, int64_t count) {
  static std::mutex mu;
  static unsigned int *base[64] = {};
  static cudaStream_t owner[64][kTicketBanks] = {};
  static int used[64] = {};
  if (count > kTicketsPerBank) return nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return nullptr; }
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_split_tickets) != cudaSuccess || !p) { cudaGetLastError(); return nullptr; }
    base[dev] = static_cast<unsigned int *>(p);
  }
  for (int b = 0; b < used[dev]; ++b)
    if (owner[dev][b] == stream) return base[dev] + (size_t)b * kTicketsPerBank;
  if (used[dev] == kTicketBanks) return nullptr;
  owner[dev][used[dev]] = stream;
  return base[dev] + (size_t)(used[dev]++) * kTicketsPerBank;
}

extern template int launch_col_typed<float, 1>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
extern template int launch_col_typed<float, 2>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
extern template int launch_col_typed<__half, 1>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);
extern template int launch_col_typed<__half, 2>(ReduceJob &j, int jd, bool ident, const ChainProg<float> &chain);

int launch_reduce_col(ReduceJob &j) {
  const CanonReduce &c = j.c;
  if (j.cdtype != PGB_F32) return 0;
  if (c.n_in > 2 || c.nr > 2 || c.nk < 1 || c.nk > 3) return 0;
  if (j.rop == ROP_ARGMAX && c.nr > 1) return 0;
  const int dt = j.in[0].dtype;
  if (dt != PGB_F32 && dt != PGB_F16) return 0;
  for (int k = 0; k < c.n_in; ++k) if (j.in[k].dtype != dt) return 0;
  // the kept dim that is contiguous in memory for every non-broadcast input;
  // prefer the innermost output dim
  int jd = -1;
  for (int d = c.nk - 1; d >= 0 && jd < 0; --d) {
    bool ok = true, any1 = false;
    for (int k = 0; k < c.n_in; ++k) {
      const int64_t s = c.kin[k][d];
      if (s != 0 && s != 1) ok = false;
      if (s == 1) any1 = true;
    }
    if (ok && any1) jd = d;
  }
  if (jd < 0) return 0;
  if (c.ksize[jd] < 32) return 0;
  ChainProg<float> chain;
  if (!to_chain<float>(j.pro, j.n_pro, chain)) return 0;
  const bool ident = chain.identity && c.n_in == 1;
  if (dt == PGB_F32) return c.n_in == 1 ? launch_col_typed<float, 1>(j, jd, ident, chain) : launch_col_typed<float, 2>(j, jd, ident, chain);
  return c.n_in == 1 ? launch_col_typed<__half, 1>(j, jd, ident, chain) : launch_col_typed<__half, 2>(j, jd, ident, chain);
}

}  // namespace pgb
