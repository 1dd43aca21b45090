/*
 * pgb200 — C ABI of the B200 (sm_100a) kernels that sit behind pequegrad's
 * `ADPrimitive::dispatch_cuda` seam (reference: csrc/ad_primitives.hpp:37-38,
 * type switch csrc/dispatch.hpp:38-44).
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; no C++ or torch types cross this boundary;
 *   - tensors are described the way the reference's `View` describes them
 *     (csrc/tensor.hpp:263-273): base pointer (storage + byte offset), shape,
 *     strides in BYTES (0 = broadcast, any permutation, negative not allowed);
 *   - outputs are allocated by the caller (the reference's dispatch functions
 *     call `view_ptr()->allocate()` first, csrc/cuda/binary.cu:59) and must be
 *     contiguous in the logical order of their shape;
 *   - every call only enqueues work on `stream` and returns; nothing synchronises;
 *   - the return value is a pgb_status; on failure `pgb_last_error()` holds a
 *     message in the reference's wording where one exists
 *     ("<name> not implemented for <dtype>", csrc/dispatch.hpp:22-24);
 *   - there is no CPU fallback: without a CUDA device every compute entry
 *     point returns PGB_ERR_CUDA.
 */
#ifndef PGB200_H
#define PGB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define PGB_API __attribute__((visibility("default")))
#else
#define PGB_API
#endif

#define PGB_MAX_DIMS 8
#define PGB_MAX_INPUTS 6
#define PGB_MAX_INSTRS 32
#define PGB_MAX_OUTPUTS 4
#define PGB_MAX_PEERS 16

/* dtype codes: 0..3 follow the reference enum order (csrc/dtype.hpp:9-14);
 * 4 and 5 are additions the int8 and bf16 paths need. */
typedef enum {
  PGB_I32 = 0,
  PGB_F16 = 1,
  PGB_F32 = 2,
  PGB_F64 = 3,
  PGB_I8 = 4,
  PGB_BF16 = 5
} pgb_dtype;

typedef enum {
  PGB_OK = 0,
  PGB_ERR_INVALID_ARG = -1, /* reference: std::invalid_argument (PG_CHECK_ARG, csrc/utils.hpp:10-25) */
  PGB_ERR_UNSUPPORTED = -2, /* reference: "... not implemented for <dtype>" runtime_error */
  PGB_ERR_CUDA = -3,        /* reference: CHECK_CUDA runtime_error (csrc/cuda/cuda_utils.cuh:14-23) */
  PGB_ERR_TIMEOUT = -4,     /* a bounded device-side wait gave up */
  PGB_ERR_WORKSPACE = -5    /* caller-provided workspace too small */
} pgb_status;

typedef struct {
  void *data;      /* device pointer to element [0,...,0] of the view */
  int32_t dtype;   /* pgb_dtype */
  int32_t ndim;    /* 0..PGB_MAX_DIMS; 0 = scalar */
  int64_t shape[PGB_MAX_DIMS];
  int64_t stride_bytes[PGB_MAX_DIMS];
} pgb_tensor;

/* Expression programs: a flat SSA list; instruction i defines value i and may
 * only read values < i. The op set is the reference fuser's linear IR
 * (csrc/compiler/ir.hpp:72 unary, :93 binary, :140 ternary) plus the eager
 * comparison/unary kernels the IR lacks (csrc/cuda/binary.cu:12-47,
 * csrc/cuda/unary.cu:152-177) and explicit casts.
 * All values are held in the region's compute type: f64 if any operand is
 * f64, i32 if all are i32, f32 otherwise (f16/bf16 are widened on load). */
typedef enum {
  PGB_OP_LOAD = 0, /* a = index of the input tensor (element at this position) */
  PGB_OP_IMM = 1,  /* imm; the reference folds Fill constants the same way (csrc/compiler/ir.cpp:235-255) */
  PGB_OP_ACC = 2,  /* epilogue only: the reduction result for this output element */
  /* unary: a */
  PGB_OP_LOG = 8,
  PGB_OP_EXP = 9,
  PGB_OP_SIN = 10,
  PGB_OP_COS = 11,
  PGB_OP_CAST_F16 = 12, /* round to half and widen again */
  PGB_OP_CAST_F32 = 13,
  PGB_OP_CAST_I32 = 14, /* C truncation toward zero, as astype does (csrc/cuda/unary.cuh:104-117) */
  PGB_OP_CAST_BF16 = 15,
  /* binary: a, b. Comparisons yield 0/1 in the compute type (csrc/cuda/binary.cu:24-41) */
  PGB_OP_ADD = 16,
  PGB_OP_MUL = 17,
  PGB_OP_MAX = 18, /* x > y ? x : y (csrc/cuda/binary.cu:42-44) */
  PGB_OP_SUB = 19,
  PGB_OP_DIV = 20, /* C division; truncating for i32 */
  PGB_OP_GT = 21,
  PGB_OP_LT = 22,
  PGB_OP_MOD = 23,
  PGB_OP_EQ = 24,
  PGB_OP_POW = 25,
  PGB_OP_LTE = 26,
  PGB_OP_NEQ = 27,
  PGB_OP_GTE = 28,
  /* ternary: a ? b : c (csrc/cuda/ternary.cu:10-12) */
  PGB_OP_WHERE = 32
} pgb_opcode;

typedef struct {
  uint8_t op; /* pgb_opcode */
  uint8_t reserved;
  int16_t a, b, c; /* value indices (or the input index for LOAD) */
  double imm;
} pgb_instr;

typedef enum {
  PGB_REDUCE_SUM = 0,   /* Sum::dispatch_cuda, csrc/cuda/reduce.cu:11-47 */
  PGB_REDUCE_MAX = 1,   /* MaxReduce::dispatch_cuda, csrc/cuda/reduce.cu:87-125 */
  PGB_REDUCE_MEAN = 2,  /* Mean::dispatch_cuda, csrc/cuda/reduce.cu:49-85: sum, then one divide by the count */
  PGB_REDUCE_ARGMAX = 3 /* first index of the maximum along ONE axis, int32 out; the reference only has
                           the Python composite pequegrad/ops.py:968-978 (float index, ties summed) */
} pgb_reduce_op;

PGB_API const char *pgb_status_string(int status);
/* Message of the last failing call made by this thread ("" if none). */
PGB_API const char *pgb_last_error(void);
PGB_API const char *pgb_version(void);
/* Number of kernels this library has launched in this process (all threads). */
PGB_API uint64_t pgb_launch_count(void);

/*
 * Fused elementwise kernel. Replaces the JIT `elementwise_kernel`
 * (csrc/compiler/ir.cpp:1395-1403, launched by Compiled::dispatch_cuda,
 * csrc/compiler/ir.cpp:1560-1606) and, with one-instruction programs, the
 * eager binary / unary / where / astype kernels (csrc/cuda/binary.cu:51-79,
 * csrc/cuda/unary.cu:11-149, csrc/cuda/ternary.cu:16-45,
 * csrc/cuda/view_helpers.cu:282-302).
 *   in[0..n_in)     same shape as the outputs, arbitrary byte strides
 *   out[0..n_out)   contiguous, same shape; out_vals[j] = program value stored to out[j]
 */
PGB_API int pgb_fused_elementwise(const pgb_tensor *in, int n_in, const pgb_tensor *out,
                          int n_out, const pgb_instr *prog, int n_instr,
                          const int16_t *out_vals, void *stream);

/*
 * Fused prologue -> reduce -> epilogue kernel. Replaces the JIT
 * `reduce_kernel` (csrc/compiler/ir.cpp:839-1151, sample README.md:93-119)
 * and, with a one-LOAD prologue and empty epilogue, the eager
 * Sum / MaxReduce / Mean kernels (csrc/cuda/reduce.cu:11-125).
 *   in[0..n_in)          all of the pre-reduce shape (stride-0 dims allowed)
 *   prologue             last value is what gets accumulated
 *   axes                 reduced axes, negative allowed (csrc/cuda/reduce.cu:22-25)
 *   out                  contiguous, keepdims shape (reduced dims = 1) or the
 *                        squeezed shape; dtype i32 for ARGMAX
 *   epi_in[0..n_epi_in)  tensors broadcastable to out's keepdims shape (same ndim as in[0]), LOAD k in the
 *                        epilogue reads epi_in[k]
 *   epilogue             may be empty (n_epi = 0): the result is stored as is
 *   workspace            scratch for split reductions; if NULL the library
 *                        allocates and frees it stream-ordered
 *                        (cudaMallocAsync, as the reference allocates outputs,
 *                        csrc/cuda/mem.cu:184-192). Query the size with
 *                        pgb_fused_reduce_workspace().
 */
PGB_API int pgb_fused_reduce(const pgb_tensor *in, int n_in, const pgb_tensor *out,
                     int reduce_op, const int32_t *axes, int n_axes,
                     const pgb_instr *prologue, int n_pro,
                     const pgb_tensor *epi_in, int n_epi_in,
                     const pgb_instr *epilogue, int n_epi, void *workspace,
                     size_t workspace_bytes, void *stream);

/* Bytes of workspace the call above would use for these arguments (0 = none). */
PGB_API int pgb_fused_reduce_workspace(const pgb_tensor *in, int n_in,
                               const pgb_tensor *out, int reduce_op,
                               const int32_t *axes, int n_axes,
                               size_t *bytes_out);

/* Which kernel family and launch geometry the planner picks; written as a short
 * human-readable line ("row g=32 vec=4 split=1 grid=..."). For tests and bench. */
PGB_API int pgb_fused_reduce_describe(const pgb_tensor *in, int n_in,
                              const pgb_tensor *out, int reduce_op,
                              const int32_t *axes, int n_axes,
                              const pgb_instr *prologue, int n_pro,
                              char *buf, size_t buf_len);

/*
 * pgb_fused_reduce for callers that cannot allocate device memory. This entry
 * point has no counterpart in the reference (whose dispatch functions allocate
 * freely, csrc/cuda/reduce.cu:26-30).
 *
 * Same arguments and results as pgb_fused_reduce, minus the workspace: the
 * partial results of a split reduction go to a fixed array of
 * PGB_NOALLOC_SCRATCH_BYTES that is part of the library image on every device
 * that loads it. The call performs no cudaMalloc / cudaFree / cudaMallocAsync
 * and calls no allocating library routine; it is meant for hosts that gave the
 * whole device to their own arena, for serving loops that forbid allocator
 * calls on the hot path, and for plugins that are only handed pointers.
 *
 *   - A reduction whose partials do not fit is refused with
 *     PGB_ERR_WORKSPACE and a message naming both sizes; nothing is launched.
 *   - The first call on a device that needs the scratch looks its address up
 *     (cudaGetSymbolAddress, once per device, with that device current); make
 *     that first call before starting any stream capture.
 *   - Every call on a device shares the one array. It keeps the previous
 *     call's partials, which is harmless (every partial is rewritten before it
 *     is read), but two calls that may overlap on the GPU (different streams,
 *     no dependency between them) race on it: order such calls.
 */
#define PGB_NOALLOC_SCRATCH_BYTES (4u << 20)
PGB_API int pgb_fused_reduce_noalloc(const pgb_tensor *in, int n_in, const pgb_tensor *out,
                     int reduce_op, const int32_t *axes, int n_axes,
                     const pgb_instr *prologue, int n_pro,
                     const pgb_tensor *epi_in, int n_epi_in,
                     const pgb_instr *epilogue, int n_epi, void *stream);

/*
 * Row softmax over the last axis, one kernel. Replaces the composite
 * pequegrad/ops.py:259-267 (max_reduce, sub, exp, sum, div) and the mask
 * `where(mask, s, -1e9)` of pequegrad/ops.py:807-814 when causal != 0
 * (column j > row i of the last two dims is excluded; excluded outputs are 0).
 * x, y: same shape, last dim contiguous, dtype f16 / bf16 / f32; math in f32.
 */
PGB_API int pgb_softmax_rows(const pgb_tensor *x, const pgb_tensor *y, int causal,
                     void *stream);

/*
 * LayerNorm over the last axis, one kernel. Replaces the composite
 * pequegrad/ops.py:515-551 (mean; biased variance via pequegrad/ops.py:480-501
 * with correction 0; (x-mean)/sqrt(var+eps); *gamma; +beta).
 * gamma / beta may be NULL. f32 or f16 io, math in f32.
 */
PGB_API int pgb_layernorm_rows(const pgb_tensor *x, const pgb_tensor *gamma,
                       const pgb_tensor *beta, float eps, const pgb_tensor *y,
                       void *stream);

/*
 * Token + position embedding: out[r, :] = wte[ids[r], :] + wpe[r % T, :]  (wpe may be NULL).
 * Replaces the index-tensor Select gather and the add of pequegrad/modules.py:329-337 and
 * examples/gpt2.py:365-372. ids int32 [rows], tables [V, C] / [>= T, C] f16 / bf16 / f32 contiguous.
 */
PGB_API int pgb_embedding_rows(const pgb_tensor *ids, const pgb_tensor *wte, const pgb_tensor *wpe, int64_t T,
                               const pgb_tensor *out, void *stream);

/*
 * Dense matmul on the tensor cores (tcgen05 + TMEM, TMA-fed): out = act(alpha * (a @ b) + bias) + residual.
 * Replaces MatMul::dispatch_cuda (csrc/cuda/matmul.cu:72-163: cuBLAS strided-batched
 * GEMM; for half inputs the reference accumulates in fp16, here the accumulator
 * is fp32) and FusedLinearBiasAct::dispatch_cuda (csrc/cuda/other.cu:19-166).
 *   a         [.., M, K], f16 or bf16 with K contiguous (fp32: see below)
 *   b         [.., K, N]. Read in place when it is the view whose K dim is the contiguous one,
 *             i.e. the transposed view of an [.., N, K] array (a Linear weight stored transposed
 *             once, or k.transpose(-2,-1) in attention); any other view of a or b (row-major
 *             [K, N], pitches that are not multiples of 16 bytes) is first copied K-major into
 *             a stream-ordered scratch buffer, as the reference contiguises its inputs.
 *             A 2-D b is shared by all batches of a;
 *             otherwise the leading dims must reduce to at most two strided batch dims
 *   alpha     scale of the product (1 for a plain matmul; 1/sqrt(d) for attention scores,
 *             pequegrad/ops.py:792-818 divides after the matmul)
 *   bias      [N] or NULL;  act: 0 none, 1 ReLU (max(x,0), pequegrad/tensor.py:162-163),
 *             2 GELU, tanh form (pequegrad/ops.py:109-118)
 *   residual  same shape as out, or NULL
 *   out       [.., M, N] f16 / bf16 / f32, N contiguous
 * fp32 operands (the reference's cublasSgemm path, csrc/cuda/matmul.cu:100-120) are accepted with ANY
 * strides for a and b: both are split into tf32 big / small parts and packed K-major into a
 * stream-ordered scratch buffer, and one tf32 tensor-core GEMM over [small|big|big] x
 * [big|small|big] sums three products per term in the fp32 accumulator: the error stays below
 * 1e-5 * sum_k |a_ik b_kj| (the classical fp32 dot-product bound for K = 170), ~1e-6 of it in practice.
 * fp64 operands (cublasDgemm in the reference) run on the fp64 units, any strides, fp64 bias / residual / output.
 * int32 operands return PGB_ERR_UNSUPPORTED ("matmul_cuda not implemented for int32"), as in the reference.
 */
PGB_API int pgb_matmul(const pgb_tensor *a, const pgb_tensor *b, const pgb_tensor *bias, int act, float alpha,
                       const pgb_tensor *residual, const pgb_tensor *out, void *stream);

/*
 * Fused scaled-dot-product attention: out = softmax(scale * q @ k^T [+ causal mask]) @ v in ONE
 * kernel; the [T, Tk] scores stay in tensor memory. Replaces the composite of the reference's
 * GPT-2 block (examples/gpt2.py:168-186: matmul, mask add, softmax of pequegrad/ops.py:259-267,
 * matmul), i.e. MatMul::dispatch_cuda twice (csrc/cuda/matmul.cu:72-163) around the softmax chain.
 *   q    [B, H, T, 64]   f16 or bf16, any view with a contiguous last dim (e.g. a slice of a packed
 *   k,v  [B, H, Tk, 64]  qkv buffer seen as [B, T, H, 64] and permuted); fewer leading dims are allowed
 *   out  [B, H, T, 64]   same dtype, a view with a contiguous last dim
 *   causal != 0: key j takes part in query row i only if j <= i (the -inf mask above the diagonal)
 * Base addresses and the row / head / batch pitches must be multiples of 16 bytes; other head
 * dims and dtypes return PGB_ERR_UNSUPPORTED. fp32 accumulation and fp32 softmax statistics; the
 * exponentials are the hardware's ex2.approx and, for a quarter of the scores, a cubic on the FMA
 * pipe (relative error 7.5e-5, below the rounding of the 16-bit probabilities that feed the second
 * product).
 */
PGB_API int pgb_attention(const pgb_tensor *q, const pgb_tensor *k, const pgb_tensor *v, float scale, int causal, const pgb_tensor *out,
                          void *stream);

/*
 * int8 quantized linear: acc = a_i8 @ w_i8^T in int32 (exact), then
 *   out = act(float(acc) * (a_scale * w_scale[n]) + bias[n])   in fp32, in that association.
 * The reference has no int8 type; its quantized example fake-quantizes weights in
 * fp32 (examples/quantized_mlp.py:28-48). This is the real-int8 form of that layer.
 *   a             [M, K] int8, K contiguous;  w  [N, K] int8 (per-output-channel quantized weight)
 *   w_scale       device pointer to N floats
 *   a_scale       per-tensor activation scale, used when a_absmax_dev is NULL; otherwise the
 *                 scale is max(*a_absmax_dev, 1e-6) / 127 read on the device (no host round trip)
 *   bias          [N] f32 or NULL;  relu != 0 applies max(x, 0)
 *   out           [M, N] f32 / f16 / bf16, or NULL
 *   acc_i32       [M, N] int32 raw accumulators, or NULL
 *   out_absmax_dev  if not NULL, max |out| is folded into it with atomicMax (the caller zeroes
 *                 it), ready to be the next layer's a_absmax_dev
 * Two more modes let a hidden layer hand int8 activations to the next layer without ever
 * writing its fp32 output (same accumulators and arithmetic, so the int8 values are the ones
 * the three-step route absmax -> pgb_quantize_i8 would give):
 *   out == NULL, acc_i32 == NULL, out_absmax_dev != NULL   only max |out| is computed;
 *   out of dtype int8 (more than 128 output channels, 16-byte aligned rows): out =
 *                 clip(rint(v / s), -127, 127) with s = max(*out_absmax_dev, 1e-6) / 127, where
 *                 *out_absmax_dev is READ here: the result of an earlier output-less pass
 */
PGB_API int pgb_qlinear_i8(const pgb_tensor *a, const pgb_tensor *w, const float *w_scale, float a_scale,
                           const float *a_absmax_dev, const pgb_tensor *bias, int relu, const pgb_tensor *out,
                           const pgb_tensor *acc_i32, float *out_absmax_dev, void *stream);

/* max |x| of a contiguous f32 tensor into *absmax_dev (zeroed by this call first). */
PGB_API int pgb_absmax_f32(const pgb_tensor *x, float *absmax_dev, void *stream);

/* q = clip(rint(x / s), -127, 127) with s = max(*absmax_dev, 1e-6) / 127, or s = scale when
 * absmax_dev is NULL; round half to even, true fp32 division. x f32, q int8, contiguous. */
PGB_API int pgb_quantize_i8(const pgb_tensor *x, const float *absmax_dev, float scale, const pgb_tensor *q,
                            void *stream);

/* Error word of the kernels' bounded device-side waits (every mbarrier wait of the tensor-core GEMMs and of the fused
 * attention gives up after a fixed number of polls instead of hanging). Synchronises with the device. *code = 0 and
 * PGB_OK when no wait ran out; else *code = (role << 16) | block (roles: 1 producer, 2 MMA issuer, 3 epilogue of the
 * GEMM kernels; 10, 11 the peer collectives; 16-26 the attention kernel's producer, MMA issuer and softmax waits) and
 * the return value is PGB_ERR_TIMEOUT. While the word is set, later launches of those kernels return at once without
 * computing; `reset` clears it. Replaces nothing in the reference, whose kernels never wait on one another. */
PGB_API int pgb_device_error(int *code, int reset);

/* Which GEMMs run on CTA pairs (tcgen05.mma.cta_group::2, 256 x 256 tiles): 0 = none, 1 = the measured default
 * (large aligned f16 / bf16 / tf32 problems), 2 = also the absmax-only pass of int8 layers, 3 = also every int8
 * pass (both measured slower than the one-CTA kernel on 65536 x 1024 x 1024: 73.9 vs 65.6 us and 88.1 vs 80.0 us;
 * kept for measurement and for the tests that compare the two kernels bit for bit), negative = only query.
 * Returns the previous mode. A tuning switch in the manner of cublasSetMathMode; the reference has no counterpart. */
PGB_API int pgb_gemm_pair_mode(int mode);

/* Failure-detection drill: the NEXT tensor-core GEMM or fused attention launched from this host thread polls each of
 * its waits at most `polls` times and, with skip_loads != 0, its producer issues no loads, so the wait of its MMA
 * warp runs out: the kernel records the error word above, frees its tensor memory and returns; nothing faults or
 * hangs. Used by the tests to exercise the timeout path; no counterpart in the reference. */
PGB_API int pgb_gemm_wait_drill(unsigned int polls, int skip_loads);

/* ---- Collectives of the batch-sharded path over peer memory (one process per GPU of one box) -------------------
 * The reference's pequegrad/distrib runs its "devices" one after another on one GPU and reduces in a Python loop
 * (pequegrad/distrib/__init__.py:4-62); these entry points have no counterpart there. They serve the two exchanges
 * the sharded workloads need (a max of one float, a gather of small slabs) as single kernels that store into the
 * peers' memory and poll their own, instead of a library collective per exchange.
 *
 * Set-up, once: every rank allocates a control block of pgb_peer_ctrl_bytes() bytes (and, for gathers, a receive
 * buffer of world x slab bytes) with pgb_peer_alloc, exports both with pgb_peer_export, passes the 64-byte handles
 * to the other ranks by any host channel, and opens the others' with pgb_peer_open. peer_ctrl[r] / peer_dst[r] are
 * then rank r's control block / receive buffer as mapped in THIS process (its own allocation for r == rank).
 * Every rank must issue the same sequence of collective calls. A rank whose peer does not arrive within the poll
 * limit (one to two seconds by default) records the error word of pgb_device_error (roles 10 and 11) and its kernel
 * returns. */
PGB_API size_t pgb_peer_ctrl_bytes(void);
/* Polls per wait of the two collective kernels below (default 2^21, one to two seconds); 0 only queries. Returns the
 * previous value. Captured graphs keep the limit they were captured with. */
PGB_API unsigned int pgb_peer_poll_limit(unsigned int polls);
PGB_API int pgb_peer_alloc(size_t bytes, void **ptr);   /* zero-filled device memory that other processes can map */
PGB_API int pgb_peer_free(void *ptr);
PGB_API int pgb_peer_export(const void *ptr, unsigned char handle[64]);
PGB_API int pgb_peer_open(const unsigned char handle[64], void **ptr);
PGB_API int pgb_peer_close(void *ptr);
/* *value (a non-negative float in this rank's memory) becomes the maximum over all ranks. */
PGB_API int pgb_peer_allreduce_max_f32(float *value, void *const *peer_ctrl, int rank, int world, void *stream);
/* Every rank's `bytes` at `src` land at offset rank * bytes of every rank's receive buffer; when the kernel has
 * finished on a rank, all slabs have arrived there. src 16-byte aligned, bytes a multiple of 16. */
PGB_API int pgb_peer_allgather(const void *src, size_t bytes, void *const *peer_dst, void *const *peer_ctrl, int rank,
                               int world, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PGB200_H */
