// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points that launch the reference's OWN CUDA kernels on the GPU, as a second oracle and as the
// "reference CUDA on the same B200" comparator of the benchmark. The kernel bodies are the reference's
// templates and macros, compiled from where they lie (the include path points into the reference
// checkout; nothing is copied). Built by oracle/build.py into oracle/_ref_cuda/libpgrefcuda.so.
//   cuda::sum_kernel / max_kernel / mean_kernel      csrc/cuda/reduce.cuh:23-163
//     launch geometry: one 64-thread block per output, 16 bytes of shared memory per dim
//                                                    csrc/cuda/reduce.cu:31-41
//   DEF_BIN_OP_KERNEL (mult, add, max)               csrc/cuda/binary.cuh:7-40, instantiated as in
//     csrc/cuda/binary.cu:12,18,42; geometry 256 threads per block, one thread per element
//                                                    csrc/cuda/binary.cu:66-76
//   DEF_UNARY_OP_KERNEL_DENSE (exp)                  csrc/cuda/unary.cuh:50-63, as csrc/cuda/unary.cu:162;
//     geometry 256 threads per block                 csrc/cuda/unary.cu:66-76
//   DEF_TERNARY_OP_KERNEL (where)                    csrc/cuda/ternary.cuh:18-38, as csrc/cuda/ternary.cu:10
//   the generated kernel of the README fusion case   README.md:93-119, cut out of the README at build time
//     into readme_kernel.inc; geometry maxThreadsPerBlock / 2 threads per block
//                                                    csrc/compiler/ir.cpp:1577-1581
// Shape / stride / axis arrays are DEVICE pointers (the reference uploads them before every launch,
// csrc/cuda/reduce.cu:26-30); callers here upload them once, so that what is timed is the kernel.
#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

#include "cuda/binary.cuh"
#include "cuda/reduce.cuh"
#include "cuda/ternary.cuh"
#include "cuda/unary.cuh"

// the reference keeps its stream in a singleton whose storage lives in one of its .cpp files
GlobalState *GlobalState::instance = nullptr;

namespace pg {
namespace cuda {
DEF_BIN_OP_KERNEL(add_kernel, x + y, float)
DEF_BIN_OP_KERNEL(mult_kernel, x *y, float)
DEF_BIN_OP_KERNEL(element_wise_max_kernel, x > y ? x : y, float)
DEF_UNARY_OP_KERNEL_DENSE(exp_kernel_dense, exp((float)x), float)
DEF_TERNARY_OP_KERNEL(where_kernel, x ? y : z, float)
}  // namespace cuda
}  // namespace pg

#include "readme_kernel.inc"  // __global__ reduce_kernel(arg0, arg1, arg2), written by oracle/build.py

#define REF_API extern "C" __attribute__((visibility("default")))

static int last_error() { return cudaGetLastError() == cudaSuccess ? 0 : -3; }

// op: 0 sum, 1 max, 2 mean. in_strides in bytes; red_axes as stride_t, like the reference passes them.
REF_API int refcuda_reduce_f32(int op, const float *in, float *out, const long *d_in_strides, const size_t *d_in_shape, int n_dims,
                               const long *d_red_axes, int n_red_axes, int total_out, int red_elements, void *stream) {
  dim3 block(REDUCE_N_WARPS * REDUCE_WARP_SIZE), grid(total_out);
  size_t smem = sizeof(size_t) * n_dims + sizeof(stride_t) * n_dims;
  cudaStream_t s = (cudaStream_t)stream;
  if (op == 0) pg::cuda::sum_kernel<float><<<grid, block, smem, s>>>(in, out, d_in_strides, d_in_shape, n_dims, d_red_axes, n_red_axes, total_out, red_elements);
  else if (op == 1) pg::cuda::max_kernel<float><<<grid, block, smem, s>>>(in, out, d_in_strides, d_in_shape, n_dims, d_red_axes, n_red_axes, total_out, red_elements);
  else if (op == 2) pg::cuda::mean_kernel<float><<<grid, block, smem, s>>>(in, out, d_in_strides, d_in_shape, n_dims, d_red_axes, n_red_axes, total_out, red_elements);
  else return -1;
  return last_error();
}

// op: 0 add, 1 mul, 2 elementwise max. Both operands already have the output's shape (broadcast dims have stride 0).
REF_API int refcuda_binary_f32(int op, const long *d_lhs_strides, const long *d_rhs_strides, const size_t *d_shape, int n_dims,
                               const float *lhs, const float *rhs, float *out, long numel, void *stream) {
  dim3 block(DEFAULT_BLOCK_SIZE), grid((unsigned)((numel + block.x - 1) / block.x));
  size_t smem = sizeof(stride_t) * n_dims * 2 + sizeof(size_t) * n_dims;
  cudaStream_t s = (cudaStream_t)stream;
  if (op == 0) pg::cuda::add_kernel<<<grid, block, smem, s>>>(d_lhs_strides, d_rhs_strides, d_shape, n_dims, lhs, rhs, out);
  else if (op == 1) pg::cuda::mult_kernel<<<grid, block, smem, s>>>(d_lhs_strides, d_rhs_strides, d_shape, n_dims, lhs, rhs, out);
  else if (op == 2) pg::cuda::element_wise_max_kernel<<<grid, block, smem, s>>>(d_lhs_strides, d_rhs_strides, d_shape, n_dims, lhs, rhs, out);
  else return -1;
  return last_error();
}

REF_API int refcuda_exp_dense_f32(const float *in, float *out, long numel, void *stream) {
  dim3 block(DEFAULT_BLOCK_SIZE), grid((unsigned)((numel + block.x - 1) / block.x));
  pg::cuda::exp_kernel_dense<<<grid, block, 0, (cudaStream_t)stream>>>((size_t)numel, in, out);
  return last_error();
}

REF_API int refcuda_where_f32(const long *d_s0, const long *d_s1, const long *d_s2, const size_t *d_shape, int n_dims, const float *a,
                              const float *b, const float *c, float *out, long numel, void *stream) {
  dim3 block(DEFAULT_BLOCK_SIZE), grid((unsigned)((numel + block.x - 1) / block.x));
  pg::cuda::where_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(d_s0, d_s1, d_s2, d_shape, n_dims, a, b, c, out);
  return last_error();
}

// The README case: x is the [1000,20,100] buffer (read through its permuted strides inside the kernel),
// y [1000,100,20], out [1000,100]. The shapes are baked into the generated source.
REF_API int refcuda_readme_kernel(const float *x, const float *y, float *out, void *stream) {
  // the reference queries the device once, when it first compiles the kernel (csrc/compiler/ir.cpp:1577-1579)
  static int threads = 0;
  if (threads == 0) {
    int dev = 0, max_threads = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&max_threads, cudaDevAttrMaxThreadsPerBlock, dev) != cudaSuccess) return -3;
    threads = max_threads / 2;
  }
  const int n_out = 100000;
  reduce_kernel<<<(n_out + threads - 1) / threads, threads, 0, (cudaStream_t)stream>>>(x, y, out);
  return last_error();
}
