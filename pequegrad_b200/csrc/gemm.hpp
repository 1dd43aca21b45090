// Shared between the tensor-core GEMM kernels (gemm_sm100.cu) and their entry
// points (gemm_abi.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pgb {

enum { GEMM_I8 = 0, GEMM_F16 = 1, GEMM_BF16 = 2 };
enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_TANH = 2 };

// What happens to the accumulator of C[m, n] before it is stored.
struct GemmEpilogue {
  // i8: v = float(acc) * (a_scale * col_scale[n]); f16 / bf16: v = acc
  const float *col_scale;    // [N] or null
  const float *a_scale_dev;  // device scalar holding max|activation|; if null a_scale is used
  float a_scale;
  const void *bias;  // [N], dtype bias_dtype, or null
  int bias_dtype;
  int act;
  const void *residual;  // laid out like the output, or null
  int res_dtype;
  int64_t res_ld, res_batch;
  void *out;      // or null
  int out_dtype;  // f32 / f16 / bf16
  int64_t ldc, out_batch;
  int32_t *acc_out;  // raw int32 accumulators (i8 only), or null
  int64_t ld_acc;
  float *absmax;  // running max |v| over the whole output (atomicMax on the bit pattern), or null
};

// a: [batch, M, K], b: [batch, N, K], both K contiguous; strides in elements.
int run_gemm_tc(int kind, const void *a, int64_t lda, int64_t a_batch, const void *b, int64_t ldb, int64_t b_batch, int64_t M, int64_t N,
                int64_t K, int64_t batch, const GemmEpilogue &epi, cudaStream_t stream);
int run_absmax_f32(const float *x, int64_t n, float *out, cudaStream_t stream);
int run_quantize_i8(const float *x, int64_t n, const float *absmax_dev, float scale, int8_t *q, cudaStream_t stream);
int read_gemm_error(int *out, bool reset);

}  // namespace pgb
