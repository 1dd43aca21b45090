// fp32 matmul on the tensor cores: operand preparation for the 3 x tf32 scheme.
//
// The reference's fp32 MatMul is a cuBLAS sgemm (csrc/cuda/matmul.cu:100-120). tcgen05 has no fp32 kind; kind::tf32
// keeps 10 mantissa bits. Splitting x = big + small with big = tf32(x), small = tf32(x - big) and summing
// big*big + big*small + small*big in the fp32 accumulator recovers ~21 bits per product (the dropped small*small
// term is below 2^-22). Laid out along K, A' = [small | big | big] and B' = [big | small | big] turn the three
// products into ONE tf32 GEMM of contraction length 3 * Kp (the two small cross terms first, while the accumulator
// is still small: the tensor core truncates when it adds into the fp32 accumulator, so what it loses per step
// scales with the accumulator's magnitude), which is what this kernel prepares: it also makes both
// operands K-major whatever the strides of the views were (32 x 32 tiles through shared memory, so reads are
// coalesced along whichever of the two dims is contiguous and writes along K).
#include "gemm.hpp"
#include "reduce_common.cuh"

namespace pgb {

struct PackParams {
  const float *in;
  float *out;
  int n_lead;
  int64_t lead_size[6], lead_stride[6];
  int64_t rows, K, Kp, row_stride, col_stride;
  int second_small;  // segment order: 0 = [small, big, big], 1 = [big, small, big]
};

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

template <bool COLS_CONTIG>
__global__ void __launch_bounds__(256) pack_tf32x3_kernel(const __grid_constant__ PackParams p) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t k0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  int64_t b = blockIdx.z, off = 0;
  for (int d = p.n_lead - 1; d >= 0; --d) {
    off += (b % p.lead_size[d]) * p.lead_stride[d];
    b /= p.lead_size[d];
  }
  const float *src = p.in + off;
#pragma unroll
  for (int i = ty; i < 32; i += 8) {
    // the fast thread index runs along the dim that is contiguous in the input
    const int64_t r = r0 + (COLS_CONTIG ? i : tx), k = k0 + (COLS_CONTIG ? tx : i);
    float v = 0.f;
    if (r < p.rows && k < p.K) v = src[r * p.row_stride + k * p.col_stride];
    tile[COLS_CONTIG ? i : tx][COLS_CONTIG ? tx : i] = v;
  }
  __syncthreads();
  float *dst = p.out + (int64_t)blockIdx.z * p.rows * 3 * p.Kp;
  const int64_t k = k0 + tx;
  if (k >= p.Kp) return;
#pragma unroll
  for (int i = ty; i < 32; i += 8) {
    const int64_t r = r0 + i;
    if (r >= p.rows) continue;
    const float x = tile[i][tx];
    const float big = tf32_round(x), small = tf32_round(x - big);
    float *row = dst + r * 3 * p.Kp + k;
    row[0] = p.second_small ? big : small;
    row[p.Kp] = p.second_small ? small : big;
    row[2 * p.Kp] = big;
  }
}

// The same re-layout without the split, for 16-bit operands whose view is not K-major or not 16-byte aligned
// (the reference contiguises such inputs too, csrc/cuda/matmul.cu:80-93): out[b, r, 0..Kp) = in[b, r, 0..K), zero padded.
template <bool COLS_CONTIG>
__global__ void __launch_bounds__(256) pack_copy16_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out, const __grid_constant__ PackParams p) {
  __shared__ uint16_t tile[32][34];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t k0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  int64_t b = blockIdx.z, off = 0;
  for (int d = p.n_lead - 1; d >= 0; --d) {
    off += (b % p.lead_size[d]) * p.lead_stride[d];
    b /= p.lead_size[d];
  }
  const uint16_t *src = in + off;
#pragma unroll
  for (int i = ty; i < 32; i += 8) {
    const int64_t r = r0 + (COLS_CONTIG ? i : tx), k = k0 + (COLS_CONTIG ? tx : i);
    uint16_t v = 0;
    if (r < p.rows && k < p.K) v = src[r * p.row_stride + k * p.col_stride];
    tile[COLS_CONTIG ? i : tx][COLS_CONTIG ? tx : i] = v;
  }
  __syncthreads();
  uint16_t *dst = out + (int64_t)blockIdx.z * p.rows * p.Kp;
  const int64_t k = k0 + tx;
  if (k >= p.Kp) return;
#pragma unroll
  for (int i = ty; i < 32; i += 8) {
    const int64_t r = r0 + i;
    if (r < p.rows) dst[r * p.Kp + k] = tile[i][tx];
  }
}

int run_pack_copy16(const void *in, void *out, int n_lead, const int64_t *lead_size, const int64_t *lead_stride, int64_t rows, int64_t K, int64_t Kp,
                    int64_t row_stride, int64_t col_stride, cudaStream_t stream) {
  PackParams p{};
  p.n_lead = n_lead;
  int64_t batch = 1;
  for (int d = 0; d < n_lead; ++d) { p.lead_size[d] = lead_size[d]; p.lead_stride[d] = lead_stride[d]; batch *= lead_size[d]; }
  p.rows = rows; p.K = K; p.Kp = Kp; p.row_stride = row_stride; p.col_stride = col_stride;
  if (rows <= 0 || Kp <= 0 || batch <= 0) return PGB_OK;
  const int64_t gy = (rows + 31) / 32;
  if (batch > 65535 || gy > 65535) { set_error("matmul: too many batches or rows for the operand re-layout"); return PGB_ERR_UNSUPPORTED; }
  const dim3 grid((unsigned)((Kp + 31) / 32), (unsigned)gy, (unsigned)batch);
  if (col_stride == 1 || K == 1) pack_copy16_kernel<true><<<grid, 256, 0, stream>>>((const uint16_t *)in, (uint16_t *)out, p);
  else pack_copy16_kernel<false><<<grid, 256, 0, stream>>>((const uint16_t *)in, (uint16_t *)out, p);
  count_launch();
  return check_launch("pack_copy16_kernel");
}

int run_pack_tf32x3(const float *in, float *out, int n_lead, const int64_t *lead_size, const int64_t *lead_stride, int64_t rows, int64_t K,
                    int64_t Kp, int64_t row_stride, int64_t col_stride, bool second_small, cudaStream_t stream) {
  PackParams p{};
  p.in = in;
  p.out = out;
  p.n_lead = n_lead;
  int64_t batch = 1;
  for (int d = 0; d < n_lead; ++d) { p.lead_size[d] = lead_size[d]; p.lead_stride[d] = lead_stride[d]; batch *= lead_size[d]; }
  p.rows = rows; p.K = K; p.Kp = Kp; p.row_stride = row_stride; p.col_stride = col_stride;
  p.second_small = second_small ? 1 : 0;
  if (rows <= 0 || Kp <= 0 || batch <= 0) return PGB_OK;
  const int64_t gy = (rows + 31) / 32;
  if (batch > 65535 || gy > 65535) { set_error("matmul: too many batches or rows for the fp32 operand preparation"); return PGB_ERR_UNSUPPORTED; }
  const dim3 grid((unsigned)((Kp + 31) / 32), (unsigned)gy, (unsigned)batch);
  if (col_stride == 1 || K == 1) pack_tf32x3_kernel<true><<<grid, 256, 0, stream>>>(p);
  else pack_tf32x3_kernel<false><<<grid, 256, 0, stream>>>(p);
  count_launch();
  return check_launch("pack_tf32x3_kernel");
}

}  // namespace pgb
