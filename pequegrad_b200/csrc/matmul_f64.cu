// fp64 matmul. tcgen05 has no fp64 kind, so this dtype (cublasDgemm in the reference,
// csrc/cuda/matmul.cu:122-140) runs on the fp64 units: 64 x 64 output tiles, 16-deep K slices through
// shared memory, a 4 x 4 register block per thread. Operands are read through their strides (any
// view), up to six leading batch dims; a 2-D b is shared by all batches. Correctness first: the
// fp64 rate of this part is a small fraction of its tensor rate whatever the kernel.
#include "gemm.hpp"
#include "reduce_common.cuh"

namespace pgb {

struct F64Params {
  const double *a, *b;
  double *c;
  const double *bias, *res;
  int64_t M, N, K;
  int64_t a_rs, a_cs, b_rs, b_cs, c_rs, r_rs;  // row / column strides in elements (c and residual: N contiguous)
  int n_lead;
  int64_t lead[6], a_ls[6], b_ls[6], c_ls[6], r_ls[6];
  double alpha;
  int act;
};

__global__ void __launch_bounds__(256) matmul_f64_kernel(const __grid_constant__ F64Params p) {
  __shared__ double As[16][64 + 1], Bs[16][64 + 1];
  int64_t bz = blockIdx.z, ao = 0, bo = 0, co = 0, ro = 0;
  for (int d = p.n_lead - 1; d >= 0; --d) {
    const int64_t i = bz % p.lead[d];
    bz /= p.lead[d];
    ao += i * p.a_ls[d]; bo += i * p.b_ls[d]; co += i * p.c_ls[d]; ro += i * p.r_ls[d];
  }
  const double *A = p.a + ao, *B = p.b + bo;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
  double acc[4][4] = {};
  for (int64_t k0 = 0; k0 < p.K; k0 += 16) {
    // 64 x 16 of A and 16 x 64 of B: 1024 elements each, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + 256 * i;
      {
        // the fast index follows the contiguous dim of the operand
        const int kk = p.a_cs == 1 ? e & 15 : e >> 6, mm = p.a_cs == 1 ? e >> 4 : e & 63;
        const int64_t m = m0 + mm, k = k0 + kk;
        As[kk][mm] = (m < p.M && k < p.K) ? A[m * p.a_rs + k * p.a_cs] : 0.0;
      }
      {
        const int kk = p.b_cs == 1 ? e >> 6 : e & 15, nn = p.b_cs == 1 ? e & 63 : e >> 4;
        const int64_t n = n0 + nn, k = k0 + kk;
        Bs[kk][nn] = (n < p.N && k < p.K) ? B[k * p.b_rs + n * p.b_cs] : 0.0;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      double av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      double v = acc[i][j] * p.alpha;
      if (p.bias) v += p.bias[n];
      if (p.act == ACT_RELU) v = v > 0.0 ? v : 0.0;
      else if (p.act == ACT_GELU_TANH) v = 0.5 * v * (1.0 + tanh(0.7978845608028654 * (v + 0.044715 * v * v * v)));
      if (p.res) v += p.res[ro + m * p.r_rs + n];
      p.c[co + m * p.c_rs + n] = v;
    }
  }
}

int run_matmul_f64(const double *a, const double *b, double *c, const double *bias, const double *res, int64_t M, int64_t N, int64_t K,
                   const int64_t strides[6], int n_lead, const int64_t *lead, const int64_t *a_ls, const int64_t *b_ls, const int64_t *c_ls,
                   const int64_t *r_ls, double alpha, int act, cudaStream_t stream) {
  F64Params p{};
  p.a = a; p.b = b; p.c = c; p.bias = bias; p.res = res;
  p.M = M; p.N = N; p.K = K;
  p.a_rs = strides[0]; p.a_cs = strides[1]; p.b_rs = strides[2]; p.b_cs = strides[3]; p.c_rs = strides[4]; p.r_rs = strides[5];
  p.n_lead = n_lead;
  int64_t batch = 1;
  for (int d = 0; d < n_lead; ++d) {
    p.lead[d] = lead[d]; p.a_ls[d] = a_ls[d]; p.b_ls[d] = b_ls[d]; p.c_ls[d] = c_ls[d]; p.r_ls[d] = r_ls ? r_ls[d] : 0;
    batch *= lead[d];
  }
  p.alpha = alpha;
  p.act = act;
  if (M <= 0 || N <= 0 || batch <= 0) return PGB_OK;
  const int64_t gx = (N + 63) / 64, gy = (M + 63) / 64;
  if (gy > 65535 || batch > 65535 || gx > 2147483647LL) { set_error("matmul: fp64 problem too large for one launch"); return PGB_ERR_UNSUPPORTED; }
  matmul_f64_kernel<<<dim3((unsigned)gx, (unsigned)gy, (unsigned)batch), 256, 0, stream>>>(p);
  count_launch();
  return check_launch("matmul_f64_kernel");
}

}  // namespace pgb
