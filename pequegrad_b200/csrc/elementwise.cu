// Fused elementwise kernels. One launch evaluates a whole expression program
// per output element; binary-broadcast, unary, where and astype are the
// one-instruction cases. Replaces the JIT `elementwise_kernel`
// (csrc/compiler/ir.cpp:1395-1403) and the eager strided kernels
// (csrc/cuda/binary.cuh:7-40, unary.cuh:23-60, ternary.cuh:18-38,
// unary.cuh:104-117), which recompute a div/mod index chain per operand per
// element and move one element per thread.
//
// Fast path: after merging dims, every operand is contiguous or broadcast
// along the innermost dim -> 128-bit loads/stores, kBatch elements per thread
// per program dispatch, at most 3 outer dims resolved once per vector.
// Generic path: any strides, any dtype mix, general SSA programs.
#include <type_traits>

#include "program.hpp"
#include "reduce_common.cuh"
#include "vec.cuh"

namespace pgb {

template <typename T, int NIN>
struct EwFastParams {
  const void *in[NIN];
  void *out;
  int nd;               // 1..4 canonical dims, right-aligned into 4 slots
  int64_t size[4];
  int64_t istr[NIN][4];
  int64_t nvec;         // numel / V
  ChainProg<T> pro;
};

template <typename T>
struct EwGenParams {
  int n_in, n_out;
  const void *in[kMaxIn];
  int in_dt[kMaxIn];
  void *out[PGB_MAX_OUTPUTS];
  int out_dt[PGB_MAX_OUTPUTS];
  int out_val[PGB_MAX_OUTPUTS];
  int nd;
  int64_t size[kMaxDims];
  int64_t istr[kMaxIn][kMaxDims];
  int64_t numel;
  VmProg<T> prog;
};

// IdxT: the type of the element index and its div / mod chain (uint32_t whenever the tensor has fewer than 2^31
// elements: a 64-bit division costs several times the rest of the thread's work)
template <typename T, typename InT, typename OutT, int NIN, int V, bool LITE, typename IdxT>
__global__ void __launch_bounds__(256) ew_fast_kernel(const __grid_constant__ EwFastParams<T, NIN> p) {
  constexpr int B = LITE ? kBatch : V;
  constexpr int U = B / V;
  const int64_t v0 = (int64_t)blockIdx.x * (256 * U) + threadIdx.x;
  T w[NIN][B];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t vid = v0 + (int64_t)u * 256;
    if (vid < p.nvec) {
      const IdxT e0 = (IdxT)(vid * V);
      int64_t c3 = (int64_t)e0, c2 = 0, c1 = 0, c0 = 0;
      if (p.nd > 1) {
        const IdxT s3 = (IdxT)p.size[3], s2 = (IdxT)p.size[2], s1 = (IdxT)p.size[1];
        IdxT r = e0 / s3;
        c3 = (int64_t)(e0 - r * s3);
        IdxT q = r / s2;
        c2 = (int64_t)(r - q * s2);
        r = q / s1;
        c1 = (int64_t)(q - r * s1);
        c0 = (int64_t)r;
      }
#pragma unroll
      for (int k = 0; k < NIN; ++k) {
        const InT *src = (const InT *)p.in[k] + c0 * p.istr[k][0] + c1 * p.istr[k][1] + c2 * p.istr[k][2];
        T tmpv[V];
        if (p.istr[k][3] != 0) load_vec<T, InT, V>(src + c3, tmpv);
        else {
          const T b = to_compute<T, InT>(__ldg(src));
#pragma unroll
          for (int e = 0; e < V; ++e) tmpv[e] = b;
        }
#pragma unroll
        for (int e = 0; e < V; ++e) w[k][u * V + e] = tmpv[e];
      }
    } else {
#pragma unroll
      for (int k = 0; k < NIN; ++k)
#pragma unroll
        for (int e = 0; e < V; ++e) w[k][u * V + e] = (T)1;
    }
  }
  T run[B];
  if (LITE) {
    ChainRegs<T> cr;
    chain_decode<T>(p.pro, cr);
    chain_eval_fast<T, NIN, B>(cr, w, run);
  } else {
    chain_eval<T, NIN, B>(p.pro, w, run);
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t vid = v0 + (int64_t)u * 256;
    if (vid < p.nvec) {
      T tmpv[V];
#pragma unroll
      for (int e = 0; e < V; ++e) tmpv[e] = run[u * V + e];
      store_vec<OutT, T, V>((OutT *)p.out + vid * V, tmpv);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ew_generic_kernel(const __grid_constant__ EwGenParams<T> p) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  T v[kMaxInstr];
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < p.numel; i += stride) {
    int64_t off[kMaxIn];
    for (int k = 0; k < p.n_in; ++k) off[k] = 0;
    int64_t r = i;
    for (int d = p.nd - 1; d >= 0; --d) {
      const int64_t c = r % p.size[d];
      r /= p.size[d];
      for (int k = 0; k < p.n_in; ++k) off[k] += c * p.istr[k][d];
    }
    vm_eval<T>(p.prog, v, (T)0, [&](int k) { return load_as<T>(p.in[k], p.in_dt[k], off[k]); });
    for (int o = 0; o < p.n_out; ++o) store_as<T>(p.out[o], p.out_dt[o], i, v[p.out_val[o]]);
  }
}

// ---------------------------------------------------------------------------
template <typename InT, typename OutT, int NIN>
static int ew_fast_launch(const CanonEw &c, const pgb_tensor *in, const pgb_tensor *out, const ChainProg<float> &chain,
                          cudaStream_t stream) {
  using T = float;
  constexpr int V = (sizeof(InT) == 2 && sizeof(OutT) == 2) ? 8 : 4;
  EwFastParams<T, NIN> p{};
  const int nd = c.nd == 0 ? 1 : c.nd;
  p.nd = nd;
  for (int d = 0; d < 4; ++d) p.size[d] = 1;
  for (int d = 0; d < c.nd; ++d) p.size[4 - c.nd + d] = c.size[d];
  if (c.nd == 0) p.size[3] = 1;
  bool vec = (p.size[3] % V) == 0 && (reinterpret_cast<uintptr_t>(out->data) % (V * sizeof(OutT))) == 0;
  for (int k = 0; k < NIN; ++k) {
    p.in[k] = in[k].data;
    for (int d = 0; d < 4; ++d) p.istr[k][d] = 0;
    for (int d = 0; d < c.nd; ++d) p.istr[k][4 - c.nd + d] = c.in[k][d];
    if (p.istr[k][3] == 1) {
      if (reinterpret_cast<uintptr_t>(p.in[k]) % (V * sizeof(InT))) vec = false;
      for (int d = 0; d < 3; ++d) if (p.istr[k][d] % V) vec = false;
    }
  }
  if (!vec) return 0;
  p.out = out->data;
  p.nvec = c.numel / V;
  p.pro = chain;
  const int64_t per_cta = chain.lite ? 256 * (kBatch / V) : 256;
  const int64_t grid = (p.nvec + per_cta - 1) / per_cta;
  if (grid > 2147483647LL || grid == 0) return 0;
  const bool idx32 = c.numel < 2147483647LL;
  if (chain.lite && idx32) ew_fast_kernel<T, InT, OutT, NIN, V, true, uint32_t><<<(unsigned)grid, 256, 0, stream>>>(p);
  else if (chain.lite) ew_fast_kernel<T, InT, OutT, NIN, V, true, int64_t><<<(unsigned)grid, 256, 0, stream>>>(p);
  else if (idx32) ew_fast_kernel<T, InT, OutT, NIN, V, false, uint32_t><<<(unsigned)grid, 256, 0, stream>>>(p);
  else ew_fast_kernel<T, InT, OutT, NIN, V, false, int64_t><<<(unsigned)grid, 256, 0, stream>>>(p);
  count_launch();
  const int st = check_launch("ew_fast_kernel");
  return st == PGB_OK ? 1 : st;
}

template <typename InT, typename OutT>
static int ew_fast_by_nin(const CanonEw &c, const pgb_tensor *in, const pgb_tensor *out, const ChainProg<float> &chain,
                          cudaStream_t stream) {
  switch (c.n_in) {
    case 1: return ew_fast_launch<InT, OutT, 1>(c, in, out, chain, stream);
    case 2: return ew_fast_launch<InT, OutT, 2>(c, in, out, chain, stream);
    case 3: return ew_fast_launch<InT, OutT, 3>(c, in, out, chain, stream);
    default: return 0;
  }
}

static int ew_try_fast(const CanonEw &c, const pgb_tensor *in, int n_in, const pgb_tensor *out, int n_out, const pgb_instr *prog, int n,
                       const int16_t *out_vals, int cdtype, cudaStream_t stream) {
  if (cdtype != PGB_F32 || n_out != 1 || n_in < 1 || n_in > 3 || c.nd > 4) return 0;
  if (out_vals[0] != n - 1) return 0;
  const int dt = in[0].dtype;
  if (dt != PGB_F32 && dt != PGB_F16) return 0;
  for (int k = 0; k < n_in; ++k) {
    if (in[k].dtype != dt) return 0;
    if (c.nd > 0) {
      const int64_t s = c.in[k][c.nd - 1];
      if (s != 0 && s != 1) return 0;
    }
  }
  const int odt = out[0].dtype;
  if (odt != PGB_F32 && odt != PGB_F16) return 0;
  ChainProg<float> chain;
  if (!to_chain<float>(prog, n, chain)) return 0;
  if (dt == PGB_F32 && odt == PGB_F32) return ew_fast_by_nin<float, float>(c, in, out, chain, stream);
  if (dt == PGB_F16 && odt == PGB_F16) return ew_fast_by_nin<__half, __half>(c, in, out, chain, stream);
  if (dt == PGB_F32 && odt == PGB_F16) return ew_fast_by_nin<float, __half>(c, in, out, chain, stream);
  return ew_fast_by_nin<__half, float>(c, in, out, chain, stream);
}

template <typename T>
static int ew_generic(const CanonEw &c, const pgb_tensor *in, int n_in, const pgb_tensor *out, int n_out, const pgb_instr *prog, int n,
                      const int16_t *out_vals, cudaStream_t stream) {
  EwGenParams<T> p{};
  p.n_in = n_in;
  p.n_out = n_out;
  p.nd = c.nd;
  p.numel = c.numel;
  for (int d = 0; d < c.nd; ++d) p.size[d] = c.size[d];
  for (int k = 0; k < n_in; ++k) {
    p.in[k] = in[k].data;
    p.in_dt[k] = in[k].dtype;
    for (int d = 0; d < c.nd; ++d) p.istr[k][d] = c.in[k][d];
  }
  for (int o = 0; o < n_out; ++o) {
    p.out[o] = out[o].data;
    p.out_dt[o] = out[o].dtype;
    p.out_val[o] = out_vals[o];
  }
  to_vm<T>(prog, n, p.prog);
  int64_t grid = (c.numel + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 64;
  if (grid > cap) grid = cap;
  if (grid == 0) return PGB_OK;
  ew_generic_kernel<T><<<(unsigned)grid, 256, 0, stream>>>(p);
  count_launch();
  return check_launch("ew_generic_kernel");
}

// ---------------------------------------------------------------------------
// Copy of a permuted view whose contiguous dim is not the output's inner dim (`as_contiguous`
// of a transpose, csrc/cuda/copy.cu of the reference does it element by element). 64 x 64
// tiles go through shared memory so that both the reads (along the input's contiguous dim i)
// and the writes (along the output's inner dim j) are coalesced; the other dims are a batch.
struct EwTrParams {
  const void *in;
  void *out;
  int nd_b;
  int64_t bsize[3], bin[3], bout[3];
  int64_t ni, nj, in_sj, out_si, tiles_i, tiles_j;
};

template <typename E>
__global__ void __launch_bounds__(256) ew_transpose_kernel(const __grid_constant__ EwTrParams p) {
  __shared__ E tile[64][64 + (sizeof(E) == 2 ? 2 : 1)];  // odd pitch in 32-bit words: conflict-free column reads
  int64_t b = blockIdx.x;
  const int64_t tj = b % p.tiles_j;
  b /= p.tiles_j;
  const int64_t ti = b % p.tiles_i;
  b /= p.tiles_i;
  int64_t ioff = 0, ooff = 0;
  for (int d = p.nd_b - 1; d >= 0; --d) {
    const int64_t c = b % p.bsize[d];
    b /= p.bsize[d];
    ioff += c * p.bin[d];
    ooff += c * p.bout[d];
  }
  const E *src = (const E *)p.in + ioff;
  E *dst = (E *)p.out + ooff;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int64_t i0 = ti * 64, j0 = tj * 64;
#pragma unroll 4
  for (int r = ty; r < 64; r += 4) {
    const int64_t i = i0 + tx, j = j0 + r;
    if (i < p.ni && j < p.nj) tile[r][tx] = src[j * p.in_sj + i];
  }
  __syncthreads();
#pragma unroll 4
  for (int r = ty; r < 64; r += 4) {
    const int64_t i = i0 + r, j = j0 + tx;
    if (i < p.ni && j < p.nj) dst[i * p.out_si + j] = tile[tx][r];
  }
}

// Returns 1 if the transposing copy was launched, 0 if the call is not of that shape.
static int ew_try_transpose(const CanonEw &c, const pgb_tensor *in, int n_in, const pgb_tensor *out, int n_out, const pgb_instr *prog, int n,
                            const int16_t *out_vals, cudaStream_t stream) {
  if (n_in != 1 || n_out != 1 || n != 1 || prog[0].op != PGB_OP_LOAD || prog[0].a != 0 || out_vals[0] != 0) return 0;
  if (in[0].dtype != out[0].dtype || c.nd < 2 || c.nd > 5) return 0;
  const int es = dtype_size(in[0].dtype);
  if (es != 2 && es != 4) return 0;
  const int j = c.nd - 1;
  if (c.in[0][j] == 1 || c.in[0][j] == 0) return 0;
  int t = -1;
  for (int d = 0; d < j; ++d)
    if (c.in[0][d] == 1) t = d;
  if (t < 0) return 0;
  EwTrParams p{};
  p.in = in[0].data;
  p.out = out[0].data;
  int64_t ostride[PGB_MAX_DIMS];
  int64_t acc = 1;
  for (int d = c.nd - 1; d >= 0; --d) { ostride[d] = acc; acc *= c.size[d]; }
  int64_t batch = 1;
  for (int d = 0; d < j; ++d) {
    if (d == t) continue;
    p.bsize[p.nd_b] = c.size[d];
    p.bin[p.nd_b] = c.in[0][d];
    p.bout[p.nd_b] = ostride[d];
    ++p.nd_b;
    batch *= c.size[d];
  }
  p.ni = c.size[t];
  p.nj = c.size[j];
  p.in_sj = c.in[0][j];
  p.out_si = ostride[t];
  p.tiles_i = (p.ni + 63) / 64;
  p.tiles_j = (p.nj + 63) / 64;
  const int64_t grid = p.tiles_i * p.tiles_j * batch;
  if (grid <= 0 || grid > 2147483647LL) return 0;
  if (es == 2) ew_transpose_kernel<uint16_t><<<(unsigned)grid, 256, 0, stream>>>(p);
  else ew_transpose_kernel<uint32_t><<<(unsigned)grid, 256, 0, stream>>>(p);
  count_launch();
  const int st = check_launch("ew_transpose_kernel");
  return st == PGB_OK ? 1 : st;
}

int run_fused_elementwise(const pgb_tensor *in, int n_in, const pgb_tensor *out, int n_out, const pgb_instr *prog, int n,
                          const int16_t *out_vals, cudaStream_t stream) {
  CanonEw c;
  std::string err = canonicalise_elementwise(in, n_in, &out[0], c);
  if (!err.empty()) { set_error(err); return PGB_ERR_INVALID_ARG; }
  if (c.numel == 0) return PGB_OK;
  const int tr = ew_try_transpose(c, in, n_in, out, n_out, prog, n, out_vals, stream);
  if (tr != 0) return tr == 1 ? PGB_OK : tr;
  const int cdtype = compute_dtype(in, n_in, out[0].dtype);
  const int r = ew_try_fast(c, in, n_in, out, n_out, prog, n, out_vals, cdtype, stream);
  if (r != 0) return r == 1 ? PGB_OK : r;
  if (cdtype == PGB_F32) return ew_generic<float>(c, in, n_in, out, n_out, prog, n, out_vals, stream);
  if (cdtype == PGB_F64) return ew_generic<double>(c, in, n_in, out, n_out, prog, n, out_vals, stream);
  return ew_generic<int>(c, in, n_in, out, n_out, prog, n, out_vals, stream);
}

}  // namespace pgb
