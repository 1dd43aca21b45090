// The persistent tcgen05 GEMM kernel and its launcher, instantiated once per instruction kind
// (gemm_kind_*.cu) so that the kinds compile in parallel. Overview in gemm_sm100.cu.
#pragma once
#include <mutex>
#include <string>

#include "gemm_epilogue.cuh"

namespace pgb {

// TMA_EPI: the output is stored with TMA tile stores (small epilogue staging, deeper operand ring); else the
// plain-store epilogue for outputs TMA cannot address.
template <int KIND, int BN, bool TMA_EPI>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                    const __grid_constant__ CUtensorMap tmap_b,
                                                                    const __grid_constant__ CUtensorMap tmap_out,
                                                                    const __grid_constant__ CUtensorMap tmap_res,
                                                                    const __grid_constant__ GemmParams p) {
  using Cfg = TileCfg<BN, TMA_EPI>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ __align__(1024) uint8_t smem[];  // the 128B-swizzled tiles need 1024-byte alignment
  // a kernel of an earlier launch gave up on a wait: do nothing until the host has read and cleared the error
  if (*(volatile int *)p.err != 0) return;
  if (smem_u32(smem) & 1023u) {  // never seen; every thread takes this exit together
    if (threadIdx.x == 0) atomicCAS(p.err, 0, (7 << 16) | (int)(blockIdx.x & 0xffff));
    return;
  }
  uint8_t *tiles = smem;
  uint8_t *epi_stage = smem + STAGES * Cfg::kStageBytes;  // 1024-aligned: every stage is a multiple of 1024 bytes
  float *col_stash = reinterpret_cast<float *>(epi_stage + Cfg::kEpiStageBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(epi_stage + Cfg::kEpiStageBytes + Cfg::kStashBytes);
  uint64_t *full = bars;                   // [STAGES]  TMA -> MMA
  uint64_t *empty = bars + STAGES;         // [STAGES]  MMA -> TMA
  uint64_t *acc_full = bars + 2 * STAGES;  // [2]       MMA -> epilogue
  uint64_t *acc_empty = acc_full + 2;      // [2]       epilogue -> MMA
  uint64_t *res_bars = acc_empty + 2;      // [kEpiWarps] TMA -> epilogue warp: its residual box has landed
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(res_bars + kEpiWarps);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int ES = (KIND == GEMM_I8) ? 1 : (KIND == GEMM_TF32 ? 4 : 2);
  constexpr int SLAB_ELEMS = kSlabBytes / ES;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_batch * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kEpiWarps); }
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&res_bars[w], 1);
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
          if (p.skip_loads) { ok = false; break; }  // test hook: nothing is loaded, the MMA warp's wait runs out
          if (!mbar_wait(&empty[s], phase ^ 1, abort_flag, p.spin_limit)) {
            report_error(p, abort_flag, 1);
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
        if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.spin_limit)) {
          report_error(p, abort_flag, 4);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full[s], phase, abort_flag, p.spin_limit)) {
            report_error(p, abort_flag, 2);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + s * Cfg::kStageBytes);
          const uint64_t da = make_kmajor_sw128_desc(sa), db = make_kmajor_sw128_desc(sa + kTileABytes);
          const int n_mma = kb == p.num_kb - 1 ? p.last_mmas : kSlabBytes / 32;
#pragma unroll
          for (int kk = 0; kk < kSlabBytes / 32; ++kk)  // one MMA consumes 32 bytes of K: +2 in 16-byte units
            if (kk < n_mma) tc_mma<KIND>(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
          tc_commit(&empty[s]);  // frees the stage when these MMAs have read it
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;   // a warp may read TMEM lanes 32*(warp%4) .. +31
    const int ew = warp - 2;  // 0..15; the four warps of a lane quadrant split the tile's columns
    if (lane == 0 && p.out_tma) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_out) : "memory");
      if (p.epi.residual) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_res) : "memory");
    }
    gemm_epilogue_warp<KIND, BN, TMA_EPI>(p, &tmap_out, &tmap_res, tmem_base, epi_stage, col_stash, res_bars + ew, ew, acc_full, acc_empty, abort_flag,
                                          q, lane, num_tiles, tiles_per_batch);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int KIND, int BN, bool TMA_EPI>
static int launch_gemm(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mo, const CUtensorMap &mr, const GemmParams &p, int grid, cudaStream_t stream) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_tc_kernel<KIND, BN, TMA_EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TileCfg<BN, TMA_EPI>::kSmem);
  });
  if (attr_err != cudaSuccess) {
    set_error(std::string("matmul: cannot raise the shared-memory limit: ") + cudaGetErrorString(attr_err));
    return PGB_ERR_CUDA;
  }
  gemm_tc_kernel<KIND, BN, TMA_EPI><<<grid, kGemmThreads, TileCfg<BN, TMA_EPI>::kSmem, stream>>>(ma, mb, mo, mr, p);
  count_launch();
  return check_launch("gemm_tc_kernel");
}

// p.out_tma != 0 selects the TMA-store kernel (128- and 256-column tiles only).
template <int KIND>
int launch_gemm_bn(int bn, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mo, const CUtensorMap &mr, const GemmParams &p, int grid,
                   cudaStream_t stream) {
  if (p.out_tma) {
    if (bn == 256) return launch_gemm<KIND, 256, true>(ma, mb, mo, mr, p, grid, stream);
    return launch_gemm<KIND, 128, true>(ma, mb, mo, mr, p, grid, stream);
  }
  if (bn == 256) return launch_gemm<KIND, 256, false>(ma, mb, mo, mr, p, grid, stream);
  if (bn == 128) return launch_gemm<KIND, 128, false>(ma, mb, mo, mr, p, grid, stream);
  return launch_gemm<KIND, 32, false>(ma, mb, mo, mr, p, grid, stream);
}

}  // namespace pgb
