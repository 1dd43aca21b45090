// Shared between the tensor-core GEMM kernels (gemm_sm100.cu) and their entry
// points (gemm_abi.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pgb {

enum { GEMM_I8 = 0, GEMM_F16 = 1, GEMM_BF16 = 2, GEMM_TF32 = 3 };
inline int gemm_elem_size(int kind) { return kind == GEMM_I8 ? 1 : (kind == GEMM_TF32 ? 4 : 2); }
enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_TANH = 2 };

// What happens to the accumulator of C[m, n] before it is stored.
struct GemmEpilogue {
  // i8: v = float(acc) * (a_scale * col_scale[n]); f16 / bf16: v = acc
  const float *col_scale;    // [N] or null
  const float *a_scale_dev;  // device scalar holding max|activation|; if null a_scale is used
  float a_scale;
  float alpha;  // f16 / bf16: v = acc * alpha (1 = off), e.g. the 1/sqrt(d) of attention scores
  const void *bias;  // [N], dtype bias_dtype, or null
  int bias_dtype;
  int act;
  const void *residual;  // laid out like the output, or null
  int res_dtype;
  int64_t res_ld, res_batch, res_batch0;  // row pitch, inner and outer batch strides (elements)
  void *out;      // or null
  int out_dtype;  // f32 / f16 / bf16; i8 (i8 kind only): v is quantised with requant_absmax
  const float *requant_absmax;  // device scalar: q = clip(rint(v / (max(*requant_absmax, 1e-6) / 127)), -127, 127)
  int64_t ldc, out_batch, out_batch0;
  int32_t *acc_out;  // raw int32 accumulators (i8 only), or null
  int64_t ld_acc;
  float *absmax;  // running max |v| over the whole output (atomicMax on the bit pattern), or null
};

// a: [nb0, nb1, M, K], b: [nb0, nb1, N, K], both K contiguous; all strides in elements
// (bs0 / bs1 = strides of the outer / inner batch dim).
int run_gemm_tc(int kind, const void *a, int64_t lda, int64_t a_bs0, int64_t a_bs1, const void *b, int64_t ldb, int64_t b_bs0, int64_t b_bs1,
                int64_t M, int64_t N, int64_t K, int64_t nb0, int64_t nb1, const GemmEpilogue &epi, cudaStream_t stream);
// out[b, r, :] = [small | big | big] (second_small = false) or [big | small | big] (true) of in[b, r, 0..K), each
// segment Kp wide (zero padded): big = x rounded to tf32, small = (x - big) rounded to tf32. Concatenated along K,
// a tf32 GEMM of two such operands sums small*big + big*small + big*big: near-fp32 accuracy from three tf32 products.
// Leading dims (up to 6) and the row / column strides of `in` are arbitrary; strides in elements.
int run_pack_tf32x3(const float *in, float *out, int n_lead, const int64_t *lead_size, const int64_t *lead_stride, int64_t rows, int64_t K,
                    int64_t Kp, int64_t row_stride, int64_t col_stride, bool second_small, cudaStream_t stream);
// out[b, r, 0..Kp) = in[b, r, 0..K) (zero padded) for 2-byte elements: a K-major, 16-byte aligned copy of any view.
int run_pack_copy16(const void *in, void *out, int n_lead, const int64_t *lead_size, const int64_t *lead_stride, int64_t rows, int64_t K, int64_t Kp,
                    int64_t row_stride, int64_t col_stride, cudaStream_t stream);
// fp64 matmul on the fp64 units (any strides; strides = {a row, a col, b row, b col, c row, residual row} in elements).
int run_matmul_f64(const double *a, const double *b, double *c, const double *bias, const double *res, int64_t M, int64_t N, int64_t K,
                   const int64_t strides[6], int n_lead, const int64_t *lead, const int64_t *a_ls, const int64_t *b_ls, const int64_t *c_ls,
                   const int64_t *r_ls, double alpha, int act, cudaStream_t stream);
int run_absmax_f32(const float *x, int64_t n, float *out, cudaStream_t stream);
int run_quantize_i8(const float *x, int64_t n, const float *absmax_dev, float scale, int8_t *q, cudaStream_t stream);
int read_gemm_error(int *out, bool reset);
int set_gemm_pair_mode(int mode);  // < 0: query; returns the previous mode
void set_next_gemm_wait_test(uint32_t spin_limit, int skip_loads);
// Reads and clears the drill of this host thread (0 polls = none): the next tensor-core GEMM or attention launch takes it.
void take_next_wait_test(uint32_t *spin_limit, int *skip_loads);
// The device error word of the current device (set by a kernel whose bounded wait ran out), or null.
int *gemm_error_word();
// 4-D tensor map with a 128B-swizzled box (dims innermost first, strides in bytes for dims 1..3). False on failure.
bool encode_map_4d(CUtensorMap *map, CUtensorMapDataType dt, const void *ptr, const uint64_t dims[4], const uint64_t strides[3],
                   const uint32_t box[4]);
int run_attention(const void *q, const void *k, const void *v, void *out, int is_half, int64_t B, int64_t H, int64_t T, int64_t Tk,
                  const int64_t q_str[3], const int64_t k_str[3], const int64_t v_str[3], const int64_t o_str[3], float scale, int causal,
                  cudaStream_t stream);

}  // namespace pgb
