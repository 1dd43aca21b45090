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
constexpr int kStagePitch = 36;  // plain-store path: words per staged row, 32 + 4 keeps 128-bit accesses conflict-free
constexpr int kSmemLimit = 232448;  // 227 KB: the most dynamic shared memory one CTA can have
constexpr int kBarrierBytes = 512;  // up to 8 + 8 ring barriers, 4 accumulator barriers, 16 residual barriers, two words
// TMA-store epilogue: one 32-row x 64-byte box (64B swizzle) per warp, one copy of the tile's column operands per CTA
constexpr int kStoreBoxBytes = 32 * 64;
constexpr int kTmaStageBytes = kEpiWarps * kStoreBoxBytes;
constexpr int kTmaStashBytes = 2 * 256 * 4;  // scale[256], bias[256]
// plain-store epilogue: splits a tile's columns in two, so eight warps work and eight only hand the accumulator over
constexpr int kPlainWarps = 8;
constexpr int kPlainStageBytes = 32 * kStagePitch * 4;
constexpr int kPlainStashBytes = kPlainWarps * 2 * 256 * 4;

// The operand ring takes whatever the epilogue leaves of the 227 KB: with 128 x 256 tiles (48 KB per stage) four
// stages beside the TMA-store epilogue, three beside the plain-store one. The ring's depth is what bounds the
// mainloop (a refill takes ~2000 cycles, a stage is consumed in 512): three stages ran the tensor pipe at 41-52 %,
// four at 28 % more.
template <int BN, bool TMA_EPI>
struct TileCfg {
  static constexpr int kTileBBytes = BN * kSlabBytes;
  static constexpr int kStageBytes = kTileABytes + kTileBBytes;
  static constexpr int kEpiStageBytes = TMA_EPI ? kTmaStageBytes : kPlainWarps * kPlainStageBytes;
  static constexpr int kStashBytes = TMA_EPI ? kTmaStashBytes : kPlainStashBytes;
  static constexpr int kRingBudget = kSmemLimit - kBarrierBytes - kEpiStageBytes - kStashBytes;
  static constexpr int kStages = (kRingBudget / kStageBytes) > 8 ? 8 : (kRingBudget / kStageBytes);
  static constexpr int kTmemCols = (2 * BN) < 32 ? 32 : 2 * BN;  // two accumulators; a power of two >= 32
  static constexpr int kSmem = kStages * kStageBytes + kEpiStageBytes + kStashBytes + kBarrierBytes;
  static_assert(kStages >= 2, "the operand ring needs at least two stages");
};

struct GemmParams {
  int M, N, K;  // K in elements
  int num_kb;   // K slabs
  int tiles_m, tiles_n, batch;  // batch = nb0 * nb1
  int nb1;                      // extent of the inner batch dim
  int out_tma;  // 0: plain stores; 2 / 4: the output goes through TMA tile stores, value = its element size
  int res_vec;  // the residual rows can be read with 16-byte loads
  int pair;     // CTAs per tile: 1, or 2 for the CTA-pair kernel (256-row tiles, tiles_m counts those)
  int last_mmas;        // MMAs the last K slab needs (1..4): K need not fill it
  uint32_t spin_limit;  // polls per bounded wait
  int skip_loads;       // test hook: the producer issues no loads, so the first wait of the MMA warp runs out
  int *err;     // device error word: 0 = ok; else (role << 16) | block index bits
  GemmEpilogue epi;
};

__device__ __forceinline__ void report_error(const GemmParams &p, volatile int *abort_flag, int role) {
  *abort_flag = 1;
  atomicCAS(p.err, 0, (role << 16) | (int)(blockIdx.x & 0xffff));
}

// Instruction descriptor: c format [4,6) (1 = f32, 2 = s32), a format [7,10), b format [10,13)
// (f16 kinds: 0 f16, 1 bf16; tf32 kind: 2; i8: 1 = signed), a/b major [15],[16] (0 = K-major),
// N >> 3 at [17,23), M >> 4 at [24,29).
template <int KIND, int BN, int BM = kBM>
__device__ __forceinline__ uint32_t make_idesc() {
  uint32_t d = 0;
  const uint32_t cfmt = (KIND == GEMM_I8) ? 2u : 1u;
  const uint32_t abfmt = (KIND == GEMM_F16) ? 0u : (KIND == GEMM_TF32 ? 2u : 1u);  // f16 = 0, bf16 = 1, tf32 = 2; i8 signed = 1
  d |= cfmt << 4;
  d |= abfmt << 7;
  d |= abfmt << 10;
  d |= (uint32_t)(BN >> 3) << 17;
  d |= (uint32_t)(BM >> 4) << 24;
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
