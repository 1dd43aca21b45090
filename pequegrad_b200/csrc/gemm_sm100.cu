// Dense contractions on the 5th-generation tensor cores: tcgen05.mma with the
// accumulators in TMEM, operands staged in shared memory by TMA (no multicast),
// mbarrier pipelines, warp-specialised roles, persistent CTAs. One kernel
// template, two instruction kinds:
//   kind::i8   int8 x int8 -> int32   (quantized linear, fused dequant + bias + ReLU)
//   kind::f16  f16 / bf16 -> f32      (matmul / linear with bias, ReLU / GELU, residual)
//
// Replaces MatMul::dispatch_cuda (cuBLAS strided-batched GEMM with a handle
// created and destroyed per call, and fp16 ACCUMULATION for half inputs,
// csrc/cuda/matmul.cu:72-163) and FusedLinearBiasAct::dispatch_cuda (CUTLASS 2.x
// Sm75 tiles, csrc/cuda/other.cu:19-166). The reference has no int8 path.
//
// Both operands are K-major: A is [M, K] and B is [N, K], K contiguous
// (a Linear weight is passed as its transpose, prepared once). One CTA per SM
// loops over 128 x BN tiles of C:
//   warp 0     TMA producer: 128-byte-wide K slabs of A and B per stage, 128B swizzle
//   warp 1     allocates TMEM, issues tcgen05.mma (one thread), commits to mbarriers
//   warps 2-9  epilogue: tcgen05.ld the accumulator (one row per thread), apply the
//              fused epilogue, transpose through shared memory, coalesced 128-bit stores
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue
// of tile i overlaps the MMAs of tile i+1.
// Every wait is bounded: on a timeout the kernel records an error word that
// pgb_device_error() reads, skips the rest of its work and frees its TMEM.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <string>

#include "gemm_epilogue.cuh"

namespace pgb {

template <int KIND, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                    const __grid_constant__ CUtensorMap tmap_b,
                                                                    const __grid_constant__ GemmParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  // a kernel of an earlier launch gave up on a wait: do nothing until the host has read and cleared the error
  if (*(volatile int *)&g_gemm_error != 0) return;
  // 1024-byte alignment for the 128B-swizzled tiles
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  uint8_t *tiles = smem;
  uint32_t *epi_stage = reinterpret_cast<uint32_t *>(smem + STAGES * Cfg::kStageBytes);
  float *col_stash = reinterpret_cast<float *>(smem + STAGES * Cfg::kStageBytes + kEpiStageBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * Cfg::kStageBytes + kEpiStageBytes + kColStashBytes);
  uint64_t *full = bars;                   // [STAGES]  TMA -> MMA
  uint64_t *empty = bars + STAGES;         // [STAGES]  MMA -> TMA
  uint64_t *acc_full = bars + 2 * STAGES;  // [2]       MMA -> epilogue
  uint64_t *acc_empty = acc_full + 2;      // [2]       epilogue -> MMA
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int ES = (KIND == GEMM_I8) ? 1 : 2;
  constexpr int SLAB_ELEMS = kSlabBytes / ES;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_batch * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kEpiWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
      uint32_t phase = 0;
      int s = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int bz = tile / tiles_per_batch, rem = tile - bz * tiles_per_batch;
        const int m0 = (rem / p.tiles_n) * kBM, n0 = (rem % p.tiles_n) * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(&g_gemm_error, 0, (1 << 16) | (blockIdx.x & 0xffff));
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], Cfg::kStageBytes);
          uint8_t *sa = tiles + s * Cfg::kStageBytes;
          tma_load_4d(sa, &tmap_a, kb * SLAB_ELEMS, m0, bz % p.nb1, bz / p.nb1, &full[s]);
          tma_load_4d(sa + kTileABytes, &tmap_b, kb * SLAB_ELEMS, n0, bz % p.nb1, bz / p.nb1, &full[s]);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc<KIND, BN>();
      uint32_t phase = 0;
      int s = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        // the epilogue must have drained this accumulator (its use two tiles ago)
        if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_gemm_error, 0, (4 << 16) | (blockIdx.x & 0xffff));
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full[s], phase, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(&g_gemm_error, 0, (2 << 16) | (blockIdx.x & 0xffff));
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + s * Cfg::kStageBytes);
          const uint64_t da = make_kmajor_sw128_desc(sa), db = make_kmajor_sw128_desc(sa + kTileABytes);
#pragma unroll
          for (int kk = 0; kk < kSlabBytes / 32; ++kk)  // one MMA consumes 32 bytes of K: +2 in 16-byte units
            tc_mma<KIND>(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
          tc_commit(&empty[s]);  // frees the stage when these MMAs have read it
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;  // a warp may read TMEM lanes 32*(warp%4) .. +31
    const int ew = warp - 2;  // 0..7; warps ew and ew+4 share a lane group and split the columns
    gemm_epilogue_warp<KIND, BN>(p, tmem_base, epi_stage + ew * 32 * kStagePitch, col_stash + ew * 512, ew >> 2, acc_full, acc_empty, abort_flag, q, lane, num_tiles,
                                 tiles_per_batch);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ---- host side ---------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// [nb0, nb1, rows, K] K-major operand -> 4-D tensor map with a {128 bytes of K, box_rows, 1, 1} box, 128B swizzle
static int make_operand_map(CUtensorMap *map, const void *ptr, int kind, int64_t rows, int64_t K, int64_t ld_elems, int64_t nb0, int64_t nb1,
                            int64_t bs0, int64_t bs1, int box_rows, const char *what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("matmul: cuTensorMapEncodeTiled is not available from this driver"); return PGB_ERR_CUDA; }
  const int es = kind == GEMM_I8 ? 1 : 2;
  // a batch dim of extent 1 has no stride of its own: give it a valid one
  if (nb1 <= 1) bs1 = rows * ld_elems;
  if (nb0 <= 1) bs0 = std::max<int64_t>(nb1, 1) * bs1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld_elems * es) % 16 || (bs1 * es) % 16 || (bs0 * es) % 16) {
    set_error(std::string("matmul: operand ") + what + " must be 16-byte aligned with row and batch pitches that are multiples of 16 bytes");
    return PGB_ERR_UNSUPPORTED;
  }
  const CUtensorMapDataType dt = kind == GEMM_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                 : (kind == GEMM_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  const cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(nb1, 1), (cuuint64_t)std::max<int64_t>(nb0, 1)};
  const cuuint64_t strides[3] = {(cuuint64_t)(ld_elems * es), (cuuint64_t)(bs1 * es), (cuuint64_t)(bs0 * es)};
  const cuuint32_t box[4] = {(cuuint32_t)(kSlabBytes / es), (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(std::string("matmul: cuTensorMapEncodeTiled failed for operand ") + what + " (code " + std::to_string((int)r) + ")");
    return PGB_ERR_CUDA;
  }
  return PGB_OK;
}

template <int KIND, int BN>
static int launch_gemm(const CUtensorMap &ma, const CUtensorMap &mb, const GemmParams &p, int grid, cudaStream_t stream) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_tc_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, TileCfg<BN>::kSmem);
  });
  if (attr_err != cudaSuccess) {
    set_error(std::string("matmul: cannot raise the shared-memory limit: ") + cudaGetErrorString(attr_err));
    return PGB_ERR_CUDA;
  }
  gemm_tc_kernel<KIND, BN><<<grid, kGemmThreads, TileCfg<BN>::kSmem, stream>>>(ma, mb, p);
  count_launch();
  return check_launch("gemm_tc_kernel");
}

template <int KIND>
static int launch_gemm_bn(int bn, const CUtensorMap &ma, const CUtensorMap &mb, const GemmParams &p, int grid, cudaStream_t stream) {
  if (bn == 256) return launch_gemm<KIND, 256>(ma, mb, p, grid, stream);
  if (bn == 128) return launch_gemm<KIND, 128>(ma, mb, p, grid, stream);
  return launch_gemm<KIND, 32>(ma, mb, p, grid, stream);
}

// a: [nb0, nb1, M, K], b: [nb0, nb1, N, K], both K contiguous; strides in elements.
int run_gemm_tc(int kind, const void *a, int64_t lda, int64_t a_bs0, int64_t a_bs1, const void *b, int64_t ldb, int64_t b_bs0, int64_t b_bs1,
                int64_t M, int64_t N, int64_t K, int64_t nb0, int64_t nb1, const GemmEpilogue &epi, cudaStream_t stream) {
  const int64_t batch = nb0 * nb1;
  if (M <= 0 || N <= 0 || batch <= 0) return PGB_OK;
  if (K <= 0) { set_error("matmul: empty contraction dim"); return PGB_ERR_INVALID_ARG; }
  int bn = N > 128 ? 256 : (N > 32 ? 128 : 32);
  if (const char *e = getenv("PGB_GEMM_BN")) {  // tuning aid
    const int v = atoi(e);
    if (v == 32 || v == 128 || v == 256) bn = v;
  }
  const int64_t tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + bn - 1) / bn;
  if (M > 2147483647LL || N > 2147483647LL || K > 2147483647LL || tiles_m * tiles_n * batch > 2147483647LL) {
    set_error("matmul: problem too large for one launch");
    return PGB_ERR_UNSUPPORTED;
  }
  CUtensorMap ma, mb;
  int st = make_operand_map(&ma, a, kind, M, K, lda, nb0, nb1, a_bs0, a_bs1, kBM, "A");
  if (st != PGB_OK) return st;
  st = make_operand_map(&mb, b, kind, N, K, ldb, nb0, nb1, b_bs0, b_bs1, bn, "B");
  if (st != PGB_OK) return st;
  GemmParams p{};
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  const int es = kind == GEMM_I8 ? 1 : 2;
  p.num_kb = (int)((K * es + kSlabBytes - 1) / kSlabBytes);
  p.tiles_m = (int)tiles_m;
  p.tiles_n = (int)tiles_n;
  p.batch = (int)batch;
  p.nb1 = (int)std::max<int64_t>(nb1, 1);
  p.epi = epi;
  if (const char *e = getenv("PGB_GEMM_DBG")) p.dbg = atoi(e);
  const int64_t num_tiles = tiles_m * tiles_n * batch;
  const int grid = (int)std::min<int64_t>(num_tiles, sm_count());
  if (kind == GEMM_I8) return launch_gemm_bn<GEMM_I8>(bn, ma, mb, p, grid, stream);
  if (kind == GEMM_F16) return launch_gemm_bn<GEMM_F16>(bn, ma, mb, p, grid, stream);
  return launch_gemm_bn<GEMM_BF16>(bn, ma, mb, p, grid, stream);
}

int read_gemm_error(int *out, bool reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return PGB_ERR_CUDA; }
  if (reset && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  }
  *out = v;
  return PGB_OK;
}

}  // namespace pgb
