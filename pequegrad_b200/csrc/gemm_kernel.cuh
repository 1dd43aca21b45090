// The persistent tcgen05 GEMM kernel (see gemm_sm100.cu for the overview).
#pragma once
#include "gemm_ptx.cuh"
#include "reduce_common.cuh"

namespace pgb {

constexpr int kBM = 128;
constexpr int kSlabBytes = 128;  // bytes of K per stage = one 128B swizzle atom row
constexpr int kTileABytes = kBM * kSlabBytes;
constexpr int kEpiGroups = 4;              // column groups: epilogue warps per TMEM lane quadrant
constexpr int kEpiWarps = 4 * kEpiGroups;  // each takes a quarter of the tile's columns for its 32 rows
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
constexpr int kStagePitch = 36;  // words per staged row: 32 + 4 keeps 128-bit accesses conflict-free
constexpr int kStoreBoxBytes = 32 * 128;  // the TMA-store box of one epilogue warp: 32 rows x (at most) 128 bytes
constexpr int kEpiStageBytes = kEpiWarps * kStoreBoxBytes;
constexpr int kPlainWarps = 8;  // the plain-store epilogue splits a tile's columns in two: eight warps work, eight only hand over
constexpr int kPlainStageBytes = 32 * kStagePitch * 4;
static_assert(kPlainWarps * kPlainStageBytes <= kEpiStageBytes, "the plain-store path stages 32 x 36-word blocks in the same area");
constexpr int kColStashBytes = kPlainWarps * 2 * 256 * 4;  // per plain-store warp: scale and bias of the tile's columns (the TMA path needs less)
constexpr int kSmemBudget = 150 * 1024;  // for the operand ring

template <int BN>
struct TileCfg {
  static constexpr int kTileBBytes = BN * kSlabBytes;
  static constexpr int kStageBytes = kTileABytes + kTileBBytes;
  static constexpr int kStages = (kSmemBudget / kStageBytes) > 8 ? 8 : (kSmemBudget / kStageBytes);
  static constexpr int kTmemCols = (2 * BN) < 32 ? 32 : 2 * BN;  // two accumulators; a power of two >= 32
  static constexpr int kSmem = kStages * kStageBytes + kEpiStageBytes + kColStashBytes + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

struct GemmParams {
  int M, N, K;  // K in elements
  int num_kb;   // K slabs
  int tiles_m, tiles_n, batch;  // batch = nb0 * nb1
  int nb1;                      // extent of the inner batch dim
  int out_tma;  // 0: plain stores; 2 / 4: the output goes through TMA tile stores, value = its element size
  int res_vec;  // the residual rows can be read with 16-byte loads
  int *err;     // device error word: 0 = ok; else (role << 16) | block index bits
  GemmEpilogue epi;
};

__device__ __forceinline__ void report_error(const GemmParams &p, volatile int *abort_flag, int role) {
  *abort_flag = 1;
  atomicCAS(p.err, 0, (role << 16) | (int)(blockIdx.x & 0xffff));
}

// Instruction descriptor: c format [4,6) (1 = f32, 2 = s32), a format [7,10), b format [10,13)
// (f16 kinds: 0 f16, 1 bf16; i8: 1 = signed), a/b major [15],[16] (0 = K-major),
// N >> 3 at [17,23), M >> 4 at [24,29).
template <int KIND, int BN>
__device__ __forceinline__ uint32_t make_idesc() {
  uint32_t d = 0;
  const uint32_t cfmt = (KIND == GEMM_I8) ? 2u : 1u;
  const uint32_t abfmt = (KIND == GEMM_F16) ? 0u : 1u;  // i8 signed = 1, bf16 = 1, f16 = 0
  d |= cfmt << 4;
  d |= abfmt << 7;
  d |= abfmt << 10;
  d |= (uint32_t)(BN >> 3) << 17;
  d |= (uint32_t)(kBM >> 4) << 24;
  return d;
}

// Writes a warp's 32-row block (thread = row, w = that row's 32-bit words) to global memory with
// coalesced 128-bit stores, going through the warp's staging area in shared memory.
// WORDS = words per row: 32 for 4-byte outputs, 16 for packed 2-byte outputs.
template <int WORDS>
__device__ __forceinline__ void stage_and_store(uint32_t *stage, const uint32_t (&w)[32], uint8_t *gbase, int64_t row_pitch_bytes, int row0,
                                                int M, int lane) {
#pragma unroll
  for (int i = 0; i < WORDS; i += 4) *reinterpret_cast<uint4 *>(stage + lane * kStagePitch + i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
  __syncwarp();
  constexpr int LPR = WORDS / 4;  // lanes per row (16 bytes each)
  constexpr int RPI = 32 / LPR;   // rows per store instruction
#pragma unroll
  for (int r0 = 0; r0 < 32; r0 += RPI) {
    const int r = r0 + lane / LPR, c4 = (lane % LPR) * 4;
    const uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kStagePitch + c4);
    if (row0 + r < M) *reinterpret_cast<uint4 *>(gbase + (int64_t)r * row_pitch_bytes + c4 * 4) = v;
  }
  __syncwarp();
}

// Scalar store of the first n elements of this thread's row (ragged right edge, unaligned rows).
// ES = element size: 4 (one word each) or 2 (two per word). All register indices are static.
template <int ES>
__device__ __forceinline__ void store_tail(const uint32_t (&w)[32], uint8_t *gbase_row0, int64_t row_pitch_bytes, int lane, int n) {
  uint8_t *dst = gbase_row0 + (int64_t)lane * row_pitch_bytes;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if (i < n) {
      if (ES == 4) reinterpret_cast<uint32_t *>(dst)[i] = w[i];
      else reinterpret_cast<uint16_t *>(dst)[i] = (uint16_t)((i & 1) ? (w[i >> 1] >> 16) : (w[i >> 1] & 0xffffu));
    }
  }
}

}  // namespace pgb
