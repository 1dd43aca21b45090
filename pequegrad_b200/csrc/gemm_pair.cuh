// The CTA-pair form of the persistent tcgen05 GEMM: a cluster of two CTAs on neighbouring SMs computes one
// 256 x 256 tile with `tcgen05.mma.cta_group::2`. Each CTA loads its own 128 rows of A and HALF of the tile's B
// columns (32 KB per stage instead of 48, so the ring is six stages deep and every B byte crosses L2 -> shared
// memory once per pair instead of once per CTA), holds its own 128 accumulator lanes in TMEM and runs its own
// epilogue. The leader (cluster rank 0) issues every MMA; barriers that both CTAs feed live in the leader:
//   full[s]       leader: both CTAs' TMA loads count their bytes there
//   empty[s]      one per CTA: the leader commits the MMAs that read the stage to both
//   acc_full[b]   one per CTA: the leader commits the finished accumulator to both
//   acc_empty[b]  leader: the epilogue warps of both CTAs arrive there
// Every wait is bounded as in the one-CTA kernel; the two cluster-wide barriers (start, end) are reached by every
// thread of both CTAs on every path, so that neither CTA leaves while the other may still signal into its memory.
#pragma once
#include <mutex>
#include <string>

#include "gemm_epilogue.cuh"
#include "gemm_pair_ptx.cuh"

namespace pgb {

constexpr int kPairBN = 256;
constexpr int kPairStageBytes = kTileABytes + (kPairBN / 2) * kSlabBytes;  // 16 KB of A + 16 KB of B per CTA
constexpr int kPairStages = (kSmemLimit - kBarrierBytes - kTmaStageBytes - kTmaStashBytes) / kPairStageBytes;
constexpr int kPairSmem = kPairStages * kPairStageBytes + kTmaStageBytes + kTmaStashBytes + kBarrierBytes;
static_assert(kPairStages >= 4 && kPairStages <= 8, "ring depth");
static_assert((2 * kPairStages + 4 + kEpiWarps) * 8 + 16 <= kBarrierBytes, "barrier region");

template <int KIND>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_res,
                        const __grid_constant__ GemmParams p) {
  constexpr int STAGES = kPairStages;
  constexpr int BN = kPairBN;
  constexpr int TMEM_COLS = 2 * BN;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t *tiles = smem;
  uint8_t *epi_stage = smem + STAGES * kPairStageBytes;
  float *col_stash = reinterpret_cast<float *>(epi_stage + kTmaStageBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(epi_stage + kTmaStageBytes + kTmaStashBytes);
  uint64_t *full = bars;                   // [STAGES]  used in the leader
  uint64_t *empty = bars + STAGES;         // [STAGES]  one per CTA
  uint64_t *acc_full = bars + 2 * STAGES;  // [2]       one per CTA
  uint64_t *acc_empty = acc_full + 2;      // [2]       used in the leader
  uint64_t *res_bars = acc_empty + 2;      // [kEpiWarps]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(res_bars + kEpiWarps);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile uint32_t *skip_flag = reinterpret_cast<volatile uint32_t *>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  constexpr int ES = (KIND == GEMM_I8) ? 1 : (KIND == GEMM_TF32 ? 4 : 2);
  constexpr int SLAB_ELEMS = kSlabBytes / ES;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_batch * p.batch;
  const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * kEpiWarps); }
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&res_bars[w], 1);
    *abort_flag = 0;
    // an earlier launch gave up on a wait (do nothing until the host has read and cleared the error), or the
    // swizzled tiles are not 1024-byte aligned (never seen)
    uint32_t skip = (*(volatile int *)p.err != 0) ? 1u : 0u;
    if (smem_u32(smem) & 1023u) {
      atomicCAS(p.err, 0, (7 << 16) | (int)(blockIdx.x & 0xffff));
      skip = 1u;
    }
    *skip_flag = skip;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anything signals them
  // the pair works or leaves together: nothing has been allocated or signalled yet
  const uint32_t skip = *skip_flag | ld_shared_cluster_u32(map_to_cta(smem_u32((const void *)skip_flag), rank ^ 1u));
  cluster_sync();  // the peer has read this CTA's flag
  if (skip) return;

  if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
      const uint32_t leader_full = map_to_cta(smem_u32(full), 0);
      uint32_t phase = 0;
      int s = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        const int bz = tile / tiles_per_batch, rem = tile - bz * tiles_per_batch;
        const int m0 = (rem / p.tiles_n) * (2 * kBM) + (int)rank * kBM;      // this CTA's rows of A
        const int n0 = (rem % p.tiles_n) * BN + (int)rank * (BN / 2);        // this CTA's half of the B columns
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) {
            report_error(p, abort_flag, 1);
            ok = false;
            break;
          }
          // the leader expects the bytes of both CTAs (the peer's may be counted before this: the count goes
          // negative for a moment, the phase cannot complete before this arrival)
          if (rank == 0) mbar_expect_tx(&full[s], 2 * kPairStageBytes);
          uint8_t *sa = tiles + s * kPairStageBytes;
          const uint32_t bar = leader_full + 8u * (uint32_t)s;
          tma_load_4d_pair(sa, &tmap_a, kb * SLAB_ELEMS, m0, bz % p.nb1, bz / p.nb1, bar);
          tma_load_4d_pair(sa + kTileABytes, &tmap_b, kb * SLAB_ELEMS, n0, bz % p.nb1, bz / p.nb1, bar);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc<KIND, BN, 2 * kBM>();
      const uint32_t my_empty = smem_u32(empty), peer_empty = map_to_cta(my_empty, 1);
      const uint32_t my_accf = smem_u32(acc_full), peer_accf = map_to_cta(my_accf, 1);
      uint32_t phase = 0;
      int s = 0, it = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++it) {
        const int buf = it & 1;
        // the epilogues of both CTAs must have drained this accumulator (its use two tiles ago)
        if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) {
          report_error(p, abort_flag, 4);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full[s], phase, abort_flag)) {
            report_error(p, abort_flag, 2);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + s * kPairStageBytes);
          const uint64_t da = make_kmajor_sw128_desc(sa), db = make_kmajor_sw128_desc(sa + kTileABytes);
          const int n_mma = kb == p.num_kb - 1 ? p.last_mmas : kSlabBytes / 32;
#pragma unroll
          for (int kk = 0; kk < kSlabBytes / 32; ++kk)
            if (kk < n_mma) tc_mma_pair<KIND>(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
          // frees the stage in both CTAs when these MMAs have read it
          tc_commit_pair(my_empty + 8u * (uint32_t)s);
          tc_commit_pair(peer_empty + 8u * (uint32_t)s);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) {
          tc_commit_pair(my_accf + 8u * (uint32_t)buf);
          tc_commit_pair(peer_accf + 8u * (uint32_t)buf);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int ew = warp - 2;
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_out) : "memory");
      if (p.epi.residual) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_res) : "memory");
    }
    gemm_epilogue_warp<KIND, BN, true>(p, &tmap_out, &tmap_res, tmem_base, epi_stage, col_stash, res_bars + ew, ew, acc_full, acc_empty, abort_flag, q,
                                       lane, num_tiles, tiles_per_batch);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // no signal of either CTA is still on its way into the other
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// Launch configuration of `grid` CTAs in clusters of two.
struct PairLaunch {
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute at{};
  PairLaunch(int grid, cudaStream_t stream) {
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = kPairSmem;
    cfg.stream = stream;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
  }
  PairLaunch(const PairLaunch &) = delete;
};

// How many CTA pairs can run at once (the SMs of a pair share a cluster, and not every SM has a partner free).
template <int KIND>
static int pair_clusters() {
  static std::once_flag once;
  static int clusters = 0;
  std::call_once(once, [] {
    if (cudaFuncSetAttribute(gemm_tc_pair_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    PairLaunch l(2 * sm_count(), nullptr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<KIND>, &l.cfg) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    clusters = n;
  });
  return clusters;
}

// p.pair == 2, p.tiles_m counts 256-row tiles. Returns PGB_ERR_UNSUPPORTED (nothing launched) when pairs cannot run here.
template <int KIND>
int launch_gemm_pair(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mo, const CUtensorMap &mr, const GemmParams &p,
                     cudaStream_t stream) {
  const int clusters = pair_clusters<KIND>();
  if (clusters < 1) return PGB_ERR_UNSUPPORTED;
  const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n * p.batch;
  PairLaunch l(2 * (int)std::min<int64_t>(num_tiles, clusters), stream);
  const cudaError_t e = cudaLaunchKernelEx(&l.cfg, gemm_tc_pair_kernel<KIND>, ma, mb, mo, mr, p);
  if (e != cudaSuccess) {
    set_error(std::string("matmul: launch of the CTA-pair kernel failed: ") + cudaGetErrorString(e));
    return PGB_ERR_CUDA;
  }
  count_launch();
  return check_launch("gemm_tc_pair_kernel");
}

}  // namespace pgb
