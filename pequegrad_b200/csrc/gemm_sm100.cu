// Dense contractions on the 5th-generation tensor cores: tcgen05.mma with the
// accumulators in TMEM, operands staged in shared memory by TMA (every CTA loads its own tiles),
// mbarrier pipelines, warp-specialised roles, persistent CTAs. One kernel
// template, two instruction kinds:
//   kind::i8   int8 x int8 -> int32   (quantized linear, fused dequant + bias + ReLU)
//   kind::f16  f16 / bf16 -> f32      (matmul / linear with bias, ReLU / GELU, residual)
//   kind::tf32 tf32 -> f32            (fp32 matmul as three tf32 products of split operands, gemm_pack.cu)
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
//   warps 2-17 epilogue: tcgen05.ld the accumulator (one row per thread), apply the fused
//              epilogue in registers, write 32-row x 128-byte boxes to shared memory and
//              TMA-store them (plain coalesced stores for outputs TMA cannot address)
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue
// of tile i overlaps the MMAs of tile i+1.
// Every wait is bounded: on a timeout the kernel records an error word that
// pgb_device_error() reads, skips the rest of its work and frees its TMEM.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <string>

#include "gemm_kernel.cuh"

namespace pgb {

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

// Encoding a tensor map costs a microsecond or two of host time, four of them per launch; a map depends only on the
// address, the extents, the pitches and the box, so the last encodings are kept and reused (what matters when a
// launch is tens of microseconds: the 8192-row MLP shards of an 8-GPU run, decode-sized GEMMs).
struct MapKey {
  const void *ptr;
  int dt, swizzle, promo;
  uint64_t dims[4], strides[3];
  uint32_t box[4];
  bool operator==(const MapKey &o) const {
    if (ptr != o.ptr || dt != o.dt || swizzle != o.swizzle || promo != o.promo) return false;
    for (int i = 0; i < 4; ++i) if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
    for (int i = 0; i < 3; ++i) if (strides[i] != o.strides[i]) return false;
    return true;
  }
};

static CUresult encode_cached(CUtensorMap *map, CUtensorMapDataType dt, const void *ptr, const cuuint64_t dims[4], const cuuint64_t strides[3],
                              const cuuint32_t box[4], CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo) {
  constexpr int kSlots = 128;
  static std::mutex mu;
  static MapKey keys[kSlots];
  static CUtensorMap maps[kSlots];
  static int used = 0, next = 0;
  MapKey k{};
  k.ptr = ptr; k.dt = (int)dt; k.swizzle = (int)swizzle; k.promo = (int)promo;
  for (int i = 0; i < 4; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i < 3; ++i) k.strides[i] = strides[i];
  {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
      if (keys[i] == k) { *map = maps[i]; return CUDA_SUCCESS; }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    std::lock_guard<std::mutex> lock(mu);
    const int slot = used < kSlots ? used++ : (next = (next + 1) % kSlots);
    keys[slot] = k;
    maps[slot] = *map;
  }
  return r;
}

// [nb0, nb1, rows, K] K-major operand -> 4-D tensor map with a {128 bytes of K, box_rows, 1, 1} box, 128B swizzle
static int make_operand_map(CUtensorMap *map, const void *ptr, int kind, int64_t rows, int64_t K, int64_t ld_elems, int64_t nb0, int64_t nb1,
                            int64_t bs0, int64_t bs1, int box_rows, const char *what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("matmul: cuTensorMapEncodeTiled is not available from this driver"); return PGB_ERR_CUDA; }
  const int es = gemm_elem_size(kind);
  // a batch dim of extent 1 has no stride of its own: give it a valid one
  if (nb1 <= 1) bs1 = rows * ld_elems;
  if (nb0 <= 1) bs0 = std::max<int64_t>(nb1, 1) * bs1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld_elems * es) % 16 || (bs1 * es) % 16 || (bs0 * es) % 16) {
    set_error(std::string("matmul: operand ") + what + " must be 16-byte aligned with row and batch pitches that are multiples of 16 bytes");
    return PGB_ERR_UNSUPPORTED;
  }
  const CUtensorMapDataType dt = kind == GEMM_I8     ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : kind == GEMM_F16  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : kind == GEMM_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(nb1, 1), (cuuint64_t)std::max<int64_t>(nb0, 1)};
  const cuuint64_t strides[3] = {(cuuint64_t)(ld_elems * es), (cuuint64_t)(bs1 * es), (cuuint64_t)(bs0 * es)};
  const cuuint32_t box[4] = {(cuuint32_t)(kSlabBytes / es), (cuuint32_t)box_rows, 1, 1};
  const CUresult r = encode_cached(map, dt, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
  if (r != CUDA_SUCCESS) {
    set_error(std::string("matmul: cuTensorMapEncodeTiled failed for operand ") + what + " (code " + std::to_string((int)r) + ")");
    return PGB_ERR_CUDA;
  }
  return PGB_OK;
}

bool encode_map_4d(CUtensorMap *map, CUtensorMapDataType dt, const void *ptr, const uint64_t dims[4], const uint64_t strides[3],
                   const uint32_t box[4]) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  const cuuint64_t s[3] = {strides[0], strides[1], strides[2]};
  const cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
  return encode_cached(map, dt, ptr, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) == CUDA_SUCCESS;
}

// The output as a 4-D tensor map for TMA tile stores: {N, M, nb1, nb0} with a {128 bytes, 32 rows, 1, 1} box, 128B swizzle.
// Returns false (and leaves the plain-store epilogue in charge) when the layout does not meet TMA's alignment rules.
static bool make_box_map(CUtensorMap *map, void *ptr, int dtype, int64_t ld, int64_t bs0, int64_t bs1, int64_t M, int64_t N, int64_t nb0, int64_t nb1);
static bool make_output_map(CUtensorMap *map, const GemmEpilogue &e, int64_t M, int64_t N, int64_t nb0, int64_t nb1, int bn) {
  (void)bn;
  return make_box_map(map, e.out, e.out_dtype, e.ldc, e.out_batch0, e.out_batch, M, N, nb0, nb1);
}
// [nb0, nb1, M, N] with N contiguous -> 4-D tensor map with the epilogue's 32-row x 64-byte box (64B swizzle).
static bool make_box_map(CUtensorMap *map, void *ptr, int dtype, int64_t ld, int64_t bs0, int64_t bs1, int64_t M, int64_t N, int64_t nb0, int64_t nb1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || !ptr) return false;
  GemmEpilogue e{};
  e.out = ptr; e.out_dtype = dtype; e.ldc = ld;
  const int es = dtype == PGB_F32 ? 4 : (dtype == PGB_I8 ? 1 : 2);
  if (nb1 <= 1) bs1 = M * ld;
  if (nb0 <= 1) bs0 = std::max<int64_t>(nb1, 1) * bs1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld * es) % 16 || (bs1 * es) % 16 || (bs0 * es) % 16 || ld < N) return false;
  const CUtensorMapDataType dt = e.out_dtype == PGB_F32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : e.out_dtype == PGB_I8  ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : e.out_dtype == PGB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)std::max<int64_t>(nb1, 1), (cuuint64_t)std::max<int64_t>(nb0, 1)};
  const cuuint64_t strides[3] = {(cuuint64_t)(e.ldc * es), (cuuint64_t)(bs1 * es), (cuuint64_t)(bs0 * es)};
  // the epilogue's box: 32 rows x 64 bytes, 64B swizzle (gemm_epilogue_tma.cuh)
  const cuuint32_t box[4] = {(cuuint32_t)(64 / es), 32, 1, 1};
  return encode_cached(map, dt, e.out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE) == CUDA_SUCCESS;
}

// The device error word that a kernel sets when one of its bounded waits runs out (one per device).
static __device__ int g_gemm_error;

int *gemm_error_word() {
  static std::mutex mu;
  static int *ptrs[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_gemm_error) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    ptrs[dev] = static_cast<int *>(p);
  }
  return ptrs[dev];
}

// one instantiation per instruction kind, each in its own translation unit (gemm_kind_*.cu)
template <int KIND>
int launch_gemm_bn(int bn, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mo, const CUtensorMap &mr, const GemmParams &p, int grid,
                   cudaStream_t stream);
extern template int launch_gemm_bn<GEMM_I8>(int, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, cudaStream_t);
extern template int launch_gemm_bn<GEMM_F16>(int, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, cudaStream_t);
extern template int launch_gemm_bn<GEMM_BF16>(int, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, cudaStream_t);
extern template int launch_gemm_bn<GEMM_TF32>(int, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, cudaStream_t);

template <int KIND>
int launch_gemm_pair(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mo, const CUtensorMap &mr, const GemmParams &p, cudaStream_t stream);
extern template int launch_gemm_pair<GEMM_I8>(const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, cudaStream_t);
extern template int launch_gemm_pair<GEMM_F16>(const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, cudaStream_t);
extern template int launch_gemm_pair<GEMM_BF16>(const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, cudaStream_t);
extern template int launch_gemm_pair<GEMM_TF32>(const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const GemmParams &, cudaStream_t);

// Which problems go to the CTA-pair kernel: 0 none (every GEMM on the one-CTA kernel), 1 the measured default below.
// Set through pgb_gemm_pair_mode() (A/B timing, and the tests that compare the two kernels).
static std::atomic<int> g_pair_mode{1};
int set_gemm_pair_mode(int mode) {
  if (mode < 0) return g_pair_mode.load();
  return g_pair_mode.exchange(mode > 3 ? 1 : mode);
}
static bool pair_enabled() { return g_pair_mode.load(std::memory_order_relaxed) != 0; }
// modes 2 / 3 (measurement only): int8 layers too, 2 = their absmax-only pass, 3 = every pass
static bool pair_int8(bool absmax_only) {
  const int m = g_pair_mode.load(std::memory_order_relaxed);
  return m == 3 || (m == 2 && absmax_only);
}

// A test hook: the next launch of the one-CTA kernel on this thread uses this many polls per wait instead of the
// default and, if `skip_loads`, its producer issues no loads, so that the first wait runs out (nothing faults, nothing
// hangs: the kernel records the error word and returns). Cleared by that launch.
static thread_local uint32_t t_next_spin_limit = 0;
static thread_local int t_next_skip_loads = 0;
void set_next_gemm_wait_test(uint32_t spin_limit, int skip_loads) {
  t_next_spin_limit = spin_limit;
  t_next_skip_loads = skip_loads;
}
void take_next_wait_test(uint32_t *spin_limit, int *skip_loads) {
  *spin_limit = t_next_spin_limit;
  *skip_loads = t_next_skip_loads;
  t_next_spin_limit = 0;
  t_next_skip_loads = 0;
}

// a: [nb0, nb1, M, K], b: [nb0, nb1, N, K], both K contiguous; strides in elements.
int run_gemm_tc(int kind, const void *a, int64_t lda, int64_t a_bs0, int64_t a_bs1, const void *b, int64_t ldb, int64_t b_bs0, int64_t b_bs1,
                int64_t M, int64_t N, int64_t K, int64_t nb0, int64_t nb1, const GemmEpilogue &epi, cudaStream_t stream) {
  const int64_t batch = nb0 * nb1;
  if (M <= 0 || N <= 0 || batch <= 0) return PGB_OK;
  if (K <= 0) { set_error("matmul: empty contraction dim"); return PGB_ERR_INVALID_ARG; }
  const int bn = N > 128 ? 256 : (N > 32 ? 128 : 32);
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
  const int es = gemm_elem_size(kind);
  p.num_kb = (int)((K * es + kSlabBytes - 1) / kSlabBytes);
  // MMAs (32 bytes of K each) that the last slab needs: the zero fill beyond K is not worth multiplying
  p.last_mmas = (int)((K * es - (int64_t)(p.num_kb - 1) * kSlabBytes + 31) / 32);
  uint32_t drill_polls = 0;
  take_next_wait_test(&drill_polls, &p.skip_loads);
  p.spin_limit = drill_polls ? drill_polls : kSpinLimit;
  p.tiles_m = (int)tiles_m;
  p.tiles_n = (int)tiles_n;
  p.batch = (int)batch;
  p.nb1 = (int)std::max<int64_t>(nb1, 1);
  p.epi = epi;
  p.err = gemm_error_word();
  if (!p.err) { set_error("matmul: cannot resolve the device error word"); return PGB_ERR_CUDA; }
  // TMA-store epilogue: the output (and the residual, read with 16-byte loads in the output's dtype) must be aligned for it;
  // raw int32 accumulators and 32-column tiles stay on the plain-store epilogue
  CUtensorMap mo = ma;
  const bool absmax_only = !epi.out && !epi.acc_out && epi.absmax;
  const int oes = absmax_only ? 4 : (epi.out_dtype == PGB_F32 ? 4 : (epi.out_dtype == PGB_I8 ? 1 : 2));
  bool fast = bn >= 128 && (epi.out || absmax_only) && !epi.acc_out;
  if (kind == GEMM_I8 && oes == 2) fast = false;
  if (oes == 1 && (kind != GEMM_I8 || bn != 256 || !epi.requant_absmax)) fast = false;
  if (fast && epi.residual) {
    const int64_t rb1 = nb1 <= 1 ? 0 : epi.res_batch, rb0 = nb0 <= 1 ? 0 : epi.res_batch0;
    fast = epi.res_dtype == epi.out_dtype && !(reinterpret_cast<uintptr_t>(epi.residual) & 15) && (epi.res_ld * oes) % 16 == 0 &&
           (rb1 * oes) % 16 == 0 && (rb0 * oes) % 16 == 0;
  }
  if (fast && !absmax_only) fast = make_output_map(&mo, epi, M, N, nb0, nb1, bn);
  CUtensorMap mr = mo;
  if (fast && epi.residual)
    fast = make_box_map(&mr, const_cast<void *>(epi.residual), epi.res_dtype, epi.res_ld, epi.res_batch0, epi.res_batch, M, N, nb0, nb1);
  if (oes == 1 && !fast) {
    set_error("qlinear: an int8 output needs more than 128 output channels, a 16-byte aligned base and row pitch, and a device absmax");
    return PGB_ERR_UNSUPPORTED;
  }
  p.out_tma = fast ? oes : 0;
  p.res_vec = fast && epi.residual;
  p.pair = 1;
  // Large aligned 16-bit / tf32 problems: CTA pairs on 256 x 256 tiles (each CTA loads half of the tile's B columns,
  // the ring is six stages deep). Measured against the one-CTA kernel on 32768-row problems: 10-17 % faster for
  // contractions of 768 with wide outputs (qkv, lm_head), level (+-3 %) for long contractions and heavy epilogues,
  // 40 % slower when a tile is a single K slab (attention scores, K = 64), and 6-9 % slower for the int8 layers,
  // whose short tiles are bound by the epilogue's arithmetic and suffer from the coupling of two CTAs' epilogues.
  if (fast && bn == 256 && M % (2 * kBM) == 0 && (kind != GEMM_I8 || pair_int8(absmax_only)) && p.num_kb >= 4 && pair_enabled() && !p.skip_loads) {
    CUtensorMap mb_half;
    if (make_operand_map(&mb_half, b, kind, N, K, ldb, nb0, nb1, b_bs0, b_bs1, bn / 2, "B") == PGB_OK) {
      GemmParams pp = p;
      pp.pair = 2;
      pp.tiles_m = (int)(M / (2 * kBM));
      int r;
      if (kind == GEMM_I8) r = launch_gemm_pair<GEMM_I8>(ma, mb_half, mo, mr, pp, stream);
      else if (kind == GEMM_F16) r = launch_gemm_pair<GEMM_F16>(ma, mb_half, mo, mr, pp, stream);
      else if (kind == GEMM_TF32) r = launch_gemm_pair<GEMM_TF32>(ma, mb_half, mo, mr, pp, stream);
      else r = launch_gemm_pair<GEMM_BF16>(ma, mb_half, mo, mr, pp, stream);
      if (r != PGB_ERR_UNSUPPORTED) return r;  // else: pairs cannot be scheduled on this device
    }
  }
  const int64_t num_tiles = tiles_m * tiles_n * batch;
  const int grid = (int)std::min<int64_t>(num_tiles, sm_count());
  if (kind == GEMM_I8) return launch_gemm_bn<GEMM_I8>(bn, ma, mb, mo, mr, p, grid, stream);
  if (kind == GEMM_F16) return launch_gemm_bn<GEMM_F16>(bn, ma, mb, mo, mr, p, grid, stream);
  if (kind == GEMM_TF32) return launch_gemm_bn<GEMM_TF32>(bn, ma, mb, mo, mr, p, grid, stream);
  return launch_gemm_bn<GEMM_BF16>(bn, ma, mb, mo, mr, p, grid, stream);
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
