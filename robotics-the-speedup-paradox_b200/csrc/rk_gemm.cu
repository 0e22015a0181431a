// Host side of the tcgen05 GEMM entry points: argument checks, tile / split-K selection,
// TMA tensor-map construction (cached), launches.

#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "rk_attn.cuh"
#include "rk_gemm_tc.cuh"
#include "rk_gemm_tc2.cuh"
#include "rk_gemm_w4.cuh"
#include "rk_gemm_w4fold.cuh"
#include "rk_gemm_w4fold2.cuh"
#include "rk_gemv_w4.cuh"
#include "rk_host.h"

namespace rk {
namespace {

constexpr int kSmemBudget = 227 * 1024 - 2048;  // dynamic shared memory we ask for at most (static barriers excluded)
constexpr int kNumSms = 148;

// Programmatic dependent launch lets a GEMM's on-chip set-up overlap the tail of the kernel before
// it in the stream.  RK_B200_PDL=0 in the environment turns it off.
// Test aid (rk_debug_wait_expiry): a shortened spin limit and a first pipeline stage whose byte
// count is never met, so that the bounded waits of the next GEMM launches run out.
int g_debug_wait_limit = 0;
int g_debug_stall = 0;

// ------------------------------------------------------------------ tensor maps
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t inner, rows, pitch;
  uint64_t planes, plane_pitch;  // third dimension (0 for 2-D maps)
  uint32_t box_inner, box_rows;
  uint32_t box_planes;
  int dtype, swizzle;
  int pad;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return static_cast<size_t>(h);
  }
};

// 2-D row-major matrix [rows, inner] (elements), row pitch in bytes, box {box_inner, box_rows}.
int make_map_2d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner,
                uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr;
  key.inner = inner;
  key.rows = rows;
  key.pitch = pitch_bytes;
  key.box_inner = box_inner;
  key.box_rows = box_rows;
  key.dtype = static_cast<int>(dtype);
  key.swizzle = static_cast<int>(swizzle);
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return RK_OK;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(RK_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (!aligned16(ptr) || pitch_bytes % 16 != 0) return fail(RK_EINVAL, "matrix base and row pitch must be 16-byte aligned");
  (void)elem_bytes;
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(RK_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return RK_OK;
}

// 3-D view [planes, rows, inner] (elements) of a row-major matrix: `planes` consecutive slices of
// `inner` elements along each row, `plane_pitch_bytes` apart.  One box {box_inner, box_rows,
// box_planes} then lands in shared memory as box_planes blocks of box_rows x box_inner, which is how
// one copy fetches several swizzle-width column blocks of a tile.
int make_map_3d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dtype, uint64_t inner, uint64_t rows,
                uint64_t planes, uint64_t pitch_bytes, uint64_t plane_pitch_bytes, uint32_t box_inner,
                uint32_t box_rows, uint32_t box_planes, CUtensorMapSwizzle swizzle) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr;
  key.inner = inner;
  key.rows = rows;
  key.pitch = pitch_bytes;
  key.planes = planes;
  key.plane_pitch = plane_pitch_bytes;
  key.box_inner = box_inner;
  key.box_rows = box_rows;
  key.box_planes = box_planes;
  key.dtype = static_cast<int>(dtype);
  key.swizzle = static_cast<int>(swizzle);
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return RK_OK;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(RK_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (!aligned16(ptr) || pitch_bytes % 16 != 0 || plane_pitch_bytes % 16 != 0)
    return fail(RK_EINVAL, "matrix base and pitches must be 16-byte aligned");
  const cuuint64_t dims[3] = {inner, rows, planes};
  const cuuint64_t strides[2] = {pitch_bytes, plane_pitch_bytes};
  const cuuint32_t box[3] = {box_inner, box_rows, box_planes};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(RK_ECUDA, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d", static_cast<int>(r));
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return RK_OK;
}

// ------------------------------------------------------------------ workspace layout
// [0, 256) status area (word 0 = status, word 16 = amax staging) | op-specific scratch
struct Workspace {
  int* status;
};

int carve_workspace(void* ws, size_t bytes, Workspace* out, const char* who) {
  if (!ws || bytes < RK_WORKSPACE_HEADER) return fail(RK_EWORKSPACE, "%s: workspace missing or too small", who);
  if (!aligned16(ws)) return fail(RK_EWORKSPACE, "%s: workspace must be 16-byte aligned", who);
  out->status = reinterpret_cast<int*>(ws);
  return RK_OK;
}

int pow2_at_least(int v, int lo) {
  int r = lo;
  while (r < v) r <<= 1;
  return r;
}

// ------------------------------------------------------------------ tile selection
struct Plan {
  int swap, bn, tiles_a, tiles_b, splits, stages, tmem_cols, acc_stride, acc_bufs, out_bufs, smem_bytes, grid_x;
  int sfb_blocks;
};

// Block-scaled kinds, rows on the MMA N axis cut into equal tiles of `bn` rows.  Scale factors live in
// 128-row blocks with one 32-bit TMEM column per 32 rows; the kernel fetches the (up to two) blocks a
// tile touches and offsets the scale-factor column address of the MMA.  That offset must be EVEN:
// tcgen05.mma raised "misaligned address" for a B scale-factor address at an odd column on B200, so
// tiles start on multiples of 64 rows.  Tiles of at most 192 rows leave room in TMEM for two
// accumulator buffers next to the scale columns, which lets the epilogue of one tile overlap the
// MMAs of the next.
int block_scaled_tile_rows(int64_t rows) {
  constexpr int align = 64;
  if (rows <= 192) return static_cast<int>(round_up(rows, 32));
  int best = 128;
  double best_cost = 1e30;
  for (int bn = 192; bn >= 64; bn -= align) {
    const int64_t tiles = (rows + bn - 1) / bn;
    // operand traffic from L2 per tile is proportional to (128 + bn); tensor time to bn
    const double cost = static_cast<double>(tiles) * (0.5 * (128 + bn) + bn);
    if (cost < best_cost) best_cost = cost, best = bn;
  }
  return best;
}

// `tactic` only nudges the shape of the decomposition (it can never change integer results and
// only reorders fp32 partial sums): bit 0 forbids swap, bit 1 forbids split-K, bit 2 halves bn.
Plan make_plan(int kind, int64_t m, int64_t n, int kblocks, int tactic) {
  Plan pl{};
  const bool block_scaled = kind == KIND_MXF8 || kind == KIND_NVF4;
  // Weights on the 128-lane axis whenever the activation row count fits one or a few
  // B-role tiles; otherwise activations take the 128-lane axis and weights use wide tiles.
  pl.swap = (m <= 1024 && !(tactic & 1)) ? 1 : 0;
  pl.sfb_blocks = 0;
  const bool rewriting = kind == KIND_I4 || kind == KIND_F8P || kind == KIND_MX48;
  if (rewriting) {
    // raw operands are rewritten in shared memory: activations on the 128-lane axis, 128-row weight
    // tiles (their raw rows and the rewritten tile both live in the stage), persistent schedule
    pl.swap = 0;
    pl.bn = n < 128 ? static_cast<int>(round_up(n, 64)) : 128;
    pl.tiles_a = static_cast<int>((m + 127) / 128);
    pl.tiles_b = static_cast<int>((n + pl.bn - 1) / pl.bn);
    pl.sfb_blocks = kind == KIND_MX48 ? 1 : 0;
    if (kind == KIND_MX48) tactic |= 2;  // block scales: no split-K
  } else if (block_scaled) {
    // A-role tiles are whole 128-row scale blocks; B-role tiles start on multiples of 64 rows
    const int64_t rows_b = pl.swap ? m : n;
    pl.bn = block_scaled_tile_rows(rows_b);
    if ((tactic & 4) && pl.bn > 128) pl.bn = 128;
    if (!pl.swap) pl.bn = static_cast<int>(round_up(pl.bn, 64)) > 192 ? 192 : static_cast<int>(round_up(pl.bn, 64));
    pl.tiles_a = static_cast<int>(((pl.swap ? n : m) + 127) / 128);
    pl.tiles_b = static_cast<int>((rows_b + pl.bn - 1) / pl.bn);
    // blocks a tile can touch: worst case over the tile starts j * bn
    int worst = 1;
    for (int j = 0; j < pl.tiles_b && j < 8; ++j) {
      const int first = (j * pl.bn) >> 7, last = (j * pl.bn + pl.bn - 1) >> 7;
      if (last - first + 1 > worst) worst = last - first + 1;
    }
    pl.sfb_blocks = worst;
  } else if (pl.swap) {
    // fewest <=256-row chunks; a lone chunk may be any multiple of 16 rows (32 when block-scaled),
    // several chunks must be multiples of 32 rows (the TMA store works on 32-row boxes)
    int chunks = static_cast<int>((m + 255) / 256);
    // When the 128-row weight tiles alone cannot occupy the machine, cut the activation rows
    // into more (<=128-row) chunks before resorting to split-K: the split-K exchange moves
    // bn x 128 x 4 bytes per CTA through distributed shared memory, so narrow tiles keep it cheap.
    const long long wide_tiles = ((n + 127) / 128) * chunks;
    if (!block_scaled && m > 128 && wide_tiles * 2 <= kNumSms) chunks = static_cast<int>((m + 127) / 128);
    const int q = (block_scaled || chunks > 1) ? 32 : 16;
    int bn = static_cast<int>(round_up((m + chunks - 1) / chunks, q));
    if ((tactic & 4) && bn >= 64 && !block_scaled) bn = static_cast<int>(round_up(bn / 2, 32));
    // A CTA's K loop runs at the pace of its issuing threads (a few hundred cycles per K block whatever
    // the tile width), so while the machine is not full, narrower activation chunks - more CTAs, each
    // with the same loop - beat both wide tiles and split-K (whose exchange costs more than it saves
    // unless the tiles are very few).
    if (!block_scaled && !(tactic & 4) && bn >= 64) {
      const int half = static_cast<int>(round_up(bn / 2, 32));
      if (((n + 127) / 128) * ((m + half - 1) / half) <= kNumSms) bn = half;
    }
    pl.bn = bn;
    pl.tiles_a = static_cast<int>((n + 127) / 128);
    pl.tiles_b = static_cast<int>((m + bn - 1) / bn);
  } else {
    // the TMA store of this layout works on 64-column boxes: bn is a multiple of 64
    pl.bn = (tactic & 4) ? 128 : 256;
    if (n < pl.bn) pl.bn = static_cast<int>(round_up(n, 64));
    pl.tiles_a = static_cast<int>((m + 127) / 128);
    pl.tiles_b = static_cast<int>((n + pl.bn - 1) / pl.bn);
  }
  // TMEM: accumulator buffers (+ scale-factor columns for the block-scaled kinds: 16 for the A
  // role, then 4 per K chunk and 128-row block of the B role)
  pl.acc_stride = static_cast<int>(round_up(pl.bn, 32));
  const int sf_cols = (block_scaled || kind == KIND_MX48) ? 16 + 4 * (kind == KIND_NVF4 ? 4 : 1) * pl.sfb_blocks : 0;
  pl.acc_bufs = (2 * pl.acc_stride + sf_cols <= 512) ? 2 : 1;
  pl.tmem_cols = pow2_at_least(pl.acc_bufs * pl.acc_stride + sf_cols, 32);
  // split-K across a cluster when the tiles cannot occupy the machine; >= 2 K blocks per CTA
  const long long tiles = static_cast<long long>(pl.tiles_a) * pl.tiles_b;
  pl.splits = 1;
  // A split costs a cluster launch and the exchange through distributed shared memory (+1 ... +7 us
  // measured on K loops of 4 ... 16 blocks: 64 x 2048 x 2048 W8A8 6.5 us split eight ways, 5.75 us
  // unsplit), so it is taken only when the K loop it shortens is long: 32 blocks of 128 bytes for the
  // direct kinds, 8 for the rewriting kinds, whose stages take ~1 us each.
  const bool long_loop = rewriting ? kblocks >= 8 : kblocks >= 32;
  if (!(tactic & 2) && tiles * 4 <= kNumSms && long_loop) {  // a two-way split does not pay for its exchange
    int s = static_cast<int>(kNumSms / tiles);
    if (s > 8) s = 8;
    if (s > kblocks / 2) s = kblocks / 2;
    if (s > 1) pl.splits = s;
  }
  // shared memory: pipeline stages + output staging + per-tile vectors
  const int stage = gemm_stage_bytes(kind, pl.bn, pl.sfb_blocks);
  pl.out_bufs = 2;
  int budget = kSmemBudget - kVecBytes - pl.out_bufs * kOutBufBytes;
  if (rewriting || (budget / stage < 4 && (kSmemBudget - kVecBytes - kOutBufBytes) / stage >= 4)) {
    pl.out_bufs = 1;  // one more pipeline stage is worth more than a second staging buffer
    budget = kSmemBudget - kVecBytes - kOutBufBytes;
  }
  pl.stages = budget / stage;
  if (pl.stages > kMaxStages) pl.stages = kMaxStages;
  const int kb_per_cta = (kblocks + pl.splits - 1) / pl.splits;
  if (pl.stages > kb_per_cta) pl.stages = kb_per_cta < 2 ? 2 : kb_per_cta;
  // the split-K exchange parks a bn x 128 x 4-byte tile in the stage memory
  while (pl.splits > 1 && pl.stages * stage < pl.bn * 512) ++pl.stages;
  pl.smem_bytes = pl.stages * stage + pl.out_bufs * kOutBufBytes + kVecBytes + 1024;
  pl.grid_x = pl.splits > 1 ? static_cast<int>(tiles) : static_cast<int>(tiles < kNumSms ? tiles : kNumSms);
  return pl;
}

template <int KIND, bool RESIDUAL = false>
int launch_tc(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_out, const GemmParams& p,
              const Plan& pl, cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_tc_kernel<KIND, RESIDUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.grid_x, 1, pl.splits);
  cfg.blockDim = dim3(KindTraits<KIND>::kThreads);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = pl.splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rk_gemm_tc_kernel<KIND, RESIDUAL>, tm_a, tm_b, tm_out, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "rk_gemm_tc_kernel launch: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

// RK_B200_ISSUE_BLOCK=0 issues every tensor-core instruction under its own predicate instead of the
// straight-line block of the elected lane (kept for comparison).
int issue_block_mode() {
  static const int mode = [] {
    const char* v = std::getenv("RK_B200_ISSUE_BLOCK");
    return (v && v[0] == '0') ? 0 : 1;
  }();
  return mode;
}

// Two-CTA schedule: RK_B200_TWO_CTA=0 never, =1 whenever the kind allows it, unset = for
// activation row counts beyond the swap range.
int two_cta_mode() {
  static const int mode = [] {
    const char* v = std::getenv("RK_B200_TWO_CTA");
    if (!v) return -1;
    return v[0] == '0' ? 0 : 1;
  }();
  return mode;
}

int launch_tc_peer(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const PeerMaps& maps, const GemmParams& p, const Plan& pl,
                   cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_tc_peer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.grid_x, 1, 1);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rk_gemm_tc_peer_kernel, tm_a, tm_b, maps, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "rk_gemm_tc_peer_kernel launch: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

template <int KIND>
int launch_tc2(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_out, const CUtensorMap& tm_sfa,
               const CUtensorMap& tm_sfb, const Gemm2Params& p, int smem, cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_tc2_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int clusters = tiles < kNumSms / 2 ? tiles : kNumSms / 2;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(p.sw_q != nullptr ? kGemm2ThreadsSwiglu : kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rk_gemm_tc2_kernel<KIND>, tm_a, tm_b, tm_out, tm_sfa, tm_sfb, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "rk_gemm_tc2_kernel launch: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

// A box of the 16 x U4 -> 16-byte-aligned tensor-map type writes 128 bytes per row into shared memory
// (8 data bytes + 8 bytes of gap per 16 elements) from 64 bytes of global memory, and the copy
// counts the 64 GLOBAL bytes per row on its barrier (measured: announcing the shared-memory bytes
// leaves the phase incomplete).  A stage therefore announces this much less per 4-bit row.
constexpr int kU4TxDeficitPerRow = 64;

// the column-parallel ("peer") mode of run_tc: see GemmParams::peer_*
struct PeerArgs {
  void* out[8];    // every rank's [m, ld] output as mapped on this GPU (TMA form), or all null
  void* mc_out;    // multicast address of the full output (multimem form), or null
  int64_t ld, col0;
  int* flags[8];
  int* epoch;
  int count, rank;
};

struct TcArgs {
  const PeerArgs* peer = nullptr;
  const void* residual = nullptr;  // gated residual update in the epilogue (GemmParams::residual)
  const void* res_gate = nullptr;
  int64_t res_tokens = 1;
  bool wgt_u4 = false;   // KIND_MXF8 with packed e2m1 weights [n, k / 2]: TMA expands them into the MMA's padded layout
  void* swiglu_q = nullptr;   // KIND_NVF4, interleaved gate/up weights: the epilogue packs silu(gate) * up to NVFP4
  void* swiglu_sf = nullptr;  //   (codes and swizzled scale factors) instead of writing bf16
  int swiglu_mode = 0;  // Gemm2Params::sw_mode
  const void* swiglu_table = nullptr;  // KIND_MXF8 with a SiLU table: the epilogue packs bf16(table[gate] * up) to MXFP8 instead
  int kind;
  const void* act;       // [m, k_bytes] bytes
  const void* wgt;       // [n, k_bytes] bytes
  int64_t m, n, k_bytes; // bytes of K per row (the row pitch)
  int mma_bytes_last;    // valid bytes of K in the last 128-byte block
  const float* scale_act;
  const float* scale_wgt;
  const uint8_t* sf_act;
  const uint8_t* sf_wgt;
  int sf_kt;
  const void* bias;
  void* out;
  int* acc_out;
  int tactic;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
  const char* who;
};

int run_tc(const TcArgs& a) {
  if (!a.act || !a.wgt || (!a.out && !a.acc_out && !a.peer && !a.swiglu_q)) return fail(RK_EINVAL, "%s: null pointer", a.who);
  if (a.m < 1 || a.n < 1 || a.k_bytes < 16) return fail(RK_EINVAL, "%s: empty problem", a.who);
  if (a.m > (1 << 24) || a.n > (1 << 24) || a.k_bytes > (1 << 24)) return fail(RK_EUNSUPPORTED, "%s: dimension too large", a.who);
  if (a.n % 8 != 0) return fail(RK_EINVAL, "%s: n must be a multiple of 8", a.who);
  Workspace ws;
  int rc = carve_workspace(a.workspace, a.workspace_bytes, &ws, a.who);
  if (rc != RK_OK) return rc;
  const int kblocks = static_cast<int>((a.k_bytes + kStageKBytes - 1) / kStageKBytes);
  const bool block_scaled = a.kind == KIND_MXF8 || a.kind == KIND_NVF4;
  const bool two_cta_kind = a.acc_out == nullptr && (a.out != nullptr || a.swiglu_q != nullptr) && a.kind <= KIND_NVF4 && a.peer == nullptr &&
                            a.residual == nullptr;  // the residual epilogue lives in the one-CTA kernel
  const int mode = two_cta_mode();
  // CTA pairs: from 512 activation rows on for the block-scaled kinds, whose main loop is paced by
  // the issuing thread (scale copies + MMAs: up to 17 tensor-core instructions per stage; one
  // instruction of a pair drives two SMs), beyond 1024 rows for the others (no gain below: measured)
  static const int64_t pair_min_env = [] {
    const char* v = std::getenv("RK_B200_TWO_CTA_MIN_M");
    return v ? static_cast<int64_t>(std::atoll(v)) : static_cast<int64_t>(0);
  }();
  const int64_t pair_min_m = pair_min_env > 0 ? pair_min_env : (block_scaled ? 512 : 1025);
  if (two_cta_kind && ((mode != 0 && ((mode == 1 && a.m > 256) || a.m >= pair_min_m) && a.n >= 128) || a.swiglu_q != nullptr)) {
    Gemm2Params p2{};
    p2.m = static_cast<int>(a.m);
    p2.n = static_cast<int>(a.n);
    p2.kblocks = kblocks;
    p2.k_valid_mmas_last = (a.mma_bytes_last + 31) / 32;
    if (p2.k_valid_mmas_last < 1 || p2.k_valid_mmas_last > 4) p2.k_valid_mmas_last = 4;
    static const int bn_env = [] {
      const char* v = std::getenv("RK_B200_PAIR_BN");
      return v ? std::atoi(v) : 0;
    }();
    if (!block_scaled) {
      p2.bn = ((a.tactic & 4) || a.n < 256) ? 128 : 256;
      p2.acc_bufs = 2;
    } else {
      // The scale factors need tensor-memory columns of their own: 128- and 192-column tiles keep two
      // accumulator buffers (the epilogue overlaps the next tile's MMAs), 256-column tiles have one
      // and pay for it with an exposed epilogue.  A stage costs the larger of the issuing thread's
      // time (about 50 cycles per tensor-core instruction: 4 MMAs, the scale copies, the commit) and
      // the tensor pipe's (bn / 2 cycles per MMA); the tile width with the least estimated time over
      // all rounds of the 74 pairs wins.  (Measured: 816 x 16384 x 2048 NVFP4 19.4 us at 192 against
      // 21.6 at 256; 4096 x 8192 x 8192 107 us at 256 against 126 at 192.)
      const int chunks = a.kind == KIND_NVF4 ? 4 : 1;
      const int64_t tiles_m = (a.m + 255) / 256;
      int64_t best = -1;
      p2.bn = 128;
      for (int bn : {256, 192, 128}) {
        if (bn > 128 && ((a.tactic & 4) || a.n < 192)) continue;
        // the re-packing epilogue is as long as the tile's MMAs: it needs the second accumulator buffer to hide behind them
        if (a.swiglu_q != nullptr && bn != 128) continue;
        const int sfb = bn == 128 ? 1 : 2;
        const int64_t issue = 50 * (4 + chunks * (1 + sfb) + 1);
        const int64_t pipe = 4 * (bn / 2);
        const int64_t stage = issue > pipe ? issue : pipe;
        const int64_t tiles = tiles_m * ((a.n + bn - 1) / bn);
        const int64_t rounds = (tiles + kNumSms / 2 - 1) / (kNumSms / 2);
        const int64_t epilogue = 10 * bn;  // exposed after every tile without a second buffer, else after the last
        const int64_t cost = rounds * (kblocks * stage + (bn == 256 ? epilogue : 0)) + (bn == 256 ? 0 : epilogue);
        if (best < 0 || cost < best) best = cost, p2.bn = bn;
      }
      if (bn_env == 128 || bn_env == 192 || bn_env == 256) p2.bn = bn_env;
      p2.acc_bufs = p2.bn == 256 ? 1 : 2;
    }
    p2.sfb_blocks = block_scaled ? (p2.bn == 128 ? 1 : 2) : 0;
    p2.sf_kt = a.sf_kt;
    p2.issue_block = issue_block_mode();
    p2.tiles_m = static_cast<int>((a.m + 255) / 256);
    p2.tiles_n = static_cast<int>((a.n + p2.bn - 1) / p2.bn);
    const int stage = gemm2_stage_bytes(a.kind, p2.bn, p2.sfb_blocks);
    p2.out_bufs = 2;
    p2.stages = (kSmemBudget - kVecBytes - 2 * kOutBufBytes) / stage;
    if (p2.stages > kMaxStages) p2.stages = kMaxStages;
    if (p2.stages > kblocks) p2.stages = kblocks < 2 ? 2 : kblocks;
    p2.ldo = a.n;
    p2.scale_act = a.scale_act;
    p2.scale_wgt = a.scale_wgt;
    p2.bias = static_cast<const __nv_bfloat16*>(a.bias);
    p2.out = static_cast<__nv_bfloat16*>(a.out);
    p2.sw_q = static_cast<uint8_t*>(a.swiglu_q);
    p2.sw_sf = static_cast<uint8_t*>(a.swiglu_sf);
    p2.sw_table = static_cast<const __nv_bfloat16*>(a.swiglu_table);
    p2.sw_mode = a.swiglu_mode;
    p2.sw_kt = a.swiglu_table != nullptr ? static_cast<int>((a.n / 2 / 32 + 3) / 4) : static_cast<int>(a.n / 128);
    p2.status = ws.status;
    CUtensorMap t_act, t_wgt, t_out, t_sfa, t_sfb;
    rc = make_map_2d(&t_act, a.act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.k_bytes, a.m, a.k_bytes, kStageKBytes, kTileA,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != RK_OK) return rc;
    rc = make_map_2d(&t_wgt, a.wgt, a.wgt_u4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                     a.k_bytes, a.n, a.wgt_u4 ? a.k_bytes / 2 : a.k_bytes, kStageKBytes, static_cast<uint32_t>(p2.bn / 2),
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != RK_OK) return rc;
    p2.fmt_a = FMT_E4M3;
    p2.fmt_b = a.wgt_u4 ? FMT_E2M1_IN_F8 : FMT_E4M3;
    p2.tx_deficit = a.wgt_u4 ? kU4TxDeficitPerRow * (p2.bn / 2) : 0;
    if (a.out != nullptr) {
      rc = make_map_2d(&t_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.n, a.m, a.n * 2, 64, 128,
                       CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != RK_OK) return rc;
    } else {
      t_out = t_act;  // the re-packing epilogue stores with ordinary instructions
    }
    t_sfa = t_act;
    t_sfb = t_act;
    if (block_scaled) {
      // scale buffers as [chunks, 128] 32-bit words; one box = the chunks of one stage and row block
      const uint32_t chunks = a.kind == KIND_NVF4 ? 4 : 1;
      rc = make_map_2d(&t_sfa, a.sf_act, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, 128, ((a.m + 127) / 128) * a.sf_kt, 512, 128,
                       chunks, CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc != RK_OK) return rc;
      rc = make_map_2d(&t_sfb, a.sf_wgt, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, 128, ((a.n + 127) / 128) * a.sf_kt, 512, 128,
                       chunks, CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc != RK_OK) return rc;
    }
    const int smem = p2.stages * stage + 2 * kOutBufBytes + kVecBytes + 1024;
    switch (a.kind) {
      case KIND_I8: return launch_tc2<KIND_I8>(t_act, t_wgt, t_out, t_sfa, t_sfb, p2, smem, a.stream);
      case KIND_F8: return launch_tc2<KIND_F8>(t_act, t_wgt, t_out, t_sfa, t_sfb, p2, smem, a.stream);
      case KIND_MXF8: return launch_tc2<KIND_MXF8>(t_act, t_wgt, t_out, t_sfa, t_sfb, p2, smem, a.stream);
      default: return launch_tc2<KIND_NVF4>(t_act, t_wgt, t_out, t_sfa, t_sfb, p2, smem, a.stream);
    }
  }
  const Plan pl = make_plan(a.kind, a.m, a.n, kblocks, a.tactic);

  CUtensorMap tm_act, tm_wgt, tm_out;
  const uint32_t box_act = pl.swap ? pl.bn : kTileA;
  const uint32_t box_wgt = pl.swap ? kTileA : pl.bn;
  // an operand that is rewritten in shared memory is fetched as raw rows: `raw` bytes of every row per
  // 128 MMA bytes of K, unswizzled; its row pitch is k_bytes * raw / 128
  const int raw_act = gemm_raw_bytes_a(a.kind), raw_wgt = gemm_raw_bytes_b(a.kind);
  if (raw_act)
    rc = make_map_2d(&tm_act, a.act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.k_bytes * raw_act / kStageKBytes, a.m,
                     a.k_bytes * raw_act / kStageKBytes, raw_act, box_act, CU_TENSOR_MAP_SWIZZLE_NONE);
  else
    rc = make_map_2d(&tm_act, a.act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.k_bytes, a.m, a.k_bytes, kStageKBytes, box_act,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  if (raw_wgt)
    rc = make_map_2d(&tm_wgt, a.wgt, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.k_bytes * raw_wgt / kStageKBytes, a.n,
                     a.k_bytes * raw_wgt / kStageKBytes, raw_wgt, box_wgt, CU_TENSOR_MAP_SWIZZLE_NONE);
  else
    rc = make_map_2d(&tm_wgt, a.wgt, a.wgt_u4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                     a.k_bytes, a.n, a.wgt_u4 ? a.k_bytes / 2 : a.k_bytes, kStageKBytes, box_wgt, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  if (a.out != nullptr && a.acc_out == nullptr && a.peer == nullptr) {
    // output tiles leave through TMA: 32 rows x 128 channels (swap) or 128 rows x 64 channels
    if (pl.swap)
      rc = make_map_2d(&tm_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.n, a.m, a.n * 2, 128, 32,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
    else
      rc = make_map_2d(&tm_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.n, a.m, a.n * 2, 64, 128,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != RK_OK) return rc;
  } else {
    tm_out = tm_act;  // unused by the raw-accumulator variant
  }

  GemmParams p{};
  p.m = static_cast<int>(a.m);
  p.n = static_cast<int>(a.n);
  p.kblocks = kblocks;
  p.k_valid_mmas_last = (a.mma_bytes_last + 31) / 32;
  if (p.k_valid_mmas_last < 1 || p.k_valid_mmas_last > 4) p.k_valid_mmas_last = 4;
  p.bn = pl.bn;
  p.swap = pl.swap;
  p.splits = pl.splits;
  p.stages = pl.stages;
  p.tmem_cols = pl.tmem_cols;
  p.acc_stride = pl.acc_stride;
  p.acc_bufs = pl.acc_bufs;
  p.out_bufs = pl.out_bufs;
  p.tiles_a = pl.tiles_a;
  p.tiles_b = pl.tiles_b;
  p.ldo = a.n;
  p.scale_act = a.scale_act;
  p.scale_wgt = a.scale_wgt;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.acc_out = a.acc_out;
  p.sf_act = a.sf_act;
  p.sf_wgt = a.sf_wgt;
  p.sf_kt = a.sf_kt;
  p.sfb_blocks = pl.sfb_blocks;
  p.sf_rows_b = static_cast<int>(pl.swap ? a.m : a.n);
  p.wait_limit = g_debug_wait_limit > 0 ? g_debug_wait_limit : static_cast<int>(kWaitSpinMax);
  p.debug_stall = g_debug_stall;
  p.issue_block = (issue_block_mode() && pl.sfb_blocks <= 2) ? 1 : 0;
  const int fmt_wgt = a.wgt_u4 ? FMT_E2M1_IN_F8 : FMT_E4M3;
  p.fmt_a = pl.swap ? fmt_wgt : FMT_E4M3;
  p.fmt_b = pl.swap ? FMT_E4M3 : fmt_wgt;
  p.tx_deficit = a.wgt_u4 ? kU4TxDeficitPerRow * static_cast<int>(box_wgt) : 0;
  p.residual = static_cast<const __nv_bfloat16*>(a.residual);
  p.res_gate = static_cast<const __nv_bfloat16*>(a.res_gate);
  p.res_magic = a.res_tokens > 1 ? static_cast<unsigned>((1ull << 32) / static_cast<unsigned long long>(a.res_tokens) + 1ull) : 0u;
  if (a.peer != nullptr) {
    for (int g = 0; g < a.peer->count; ++g) p.peer_flags[g] = a.peer->flags[g];
    p.peer_mc = static_cast<__nv_bfloat16*>(a.peer->mc_out);
    p.peer_ld = a.peer->ld;
    p.peer_col0 = a.peer->col0;
    p.peer_count = a.peer->count;
    p.peer_rank = a.peer->rank;
    p.peer_mask = 0xFFu;
    p.peer_epoch = a.peer->epoch;
    p.peer_counter = reinterpret_cast<unsigned*>(ws.status) + 32;  // a word of the workspace header, zero between launches
  }
  p.status = ws.status;
  const CUtensorMap& tm_a = pl.swap ? tm_wgt : tm_act;
  const CUtensorMap& tm_b = pl.swap ? tm_act : tm_wgt;
  if (a.peer != nullptr) {
    PeerMaps maps{};
    for (int g = 0; g < a.peer->count; ++g) {
      maps.m[g] = tm_act;  // placeholder for the multicast form (never dereferenced)
      if (a.peer->mc_out != nullptr) continue;
      // this rank's slab inside rank g's [m, ld] buffer, clipped at the slab's edges: boxes of 32 rows x 128
      // channels when the weights take the 128-lane axis, else of 128 rows x 64 channels
      const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(a.peer->out[g]) + a.peer->col0;
      rc = pl.swap ? make_map_2d(&maps.m[g], base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.n, a.m, a.peer->ld * 2, 128, 32,
                                 CU_TENSOR_MAP_SWIZZLE_NONE)
                   : make_map_2d(&maps.m[g], base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.n, a.m, a.peer->ld * 2, 64, 128,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != RK_OK) return rc;
    }
    return launch_tc_peer(tm_a, tm_b, maps, p, pl, a.stream);
  }
  switch (a.kind) {
    case KIND_I8:
      return a.residual != nullptr ? launch_tc<KIND_I8, true>(tm_a, tm_b, tm_out, p, pl, a.stream)
                                   : launch_tc<KIND_I8>(tm_a, tm_b, tm_out, p, pl, a.stream);
    case KIND_F8: return launch_tc<KIND_F8>(tm_a, tm_b, tm_out, p, pl, a.stream);
    case KIND_MXF8: return launch_tc<KIND_MXF8>(tm_a, tm_b, tm_out, p, pl, a.stream);
    case KIND_NVF4: return launch_tc<KIND_NVF4>(tm_a, tm_b, tm_out, p, pl, a.stream);
    case KIND_I4:
      return a.residual != nullptr ? launch_tc<KIND_I4, true>(tm_a, tm_b, tm_out, p, pl, a.stream)
                                   : launch_tc<KIND_I4>(tm_a, tm_b, tm_out, p, pl, a.stream);
    case KIND_F8P: return launch_tc<KIND_F8P>(tm_a, tm_b, tm_out, p, pl, a.stream);
    default: return launch_tc<KIND_MX48>(tm_a, tm_b, tm_out, p, pl, a.stream);
  }
}

// Two's-complement nibbles (low nibble = even k) -> int8, 16 packed bytes per thread.
__global__ void __launch_bounds__(256) unpack_int4_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                                          long long vectors) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= vectors) return;
  const uint4 v = in[i];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // per-byte sign extension of the even and odd nibbles: (u ^ 8) - 8
    const uint32_t even = __vsub4((w[j] & 0x0F0F0F0Fu) ^ 0x08080808u, 0x08080808u);
    const uint32_t odd = __vsub4(((w[j] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u, 0x08080808u);
    o[2 * j] = __byte_perm(even, odd, 0x5140);      // e0 o0 e1 o1
    o[2 * j + 1] = __byte_perm(even, odd, 0x7362);  // e2 o2 e3 o3
  }
  out[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
  out[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

int unpack_int4(const void* in, void* out, long long packed_bytes, cudaStream_t st) {
  const long long vectors = packed_bytes / 16;
  unpack_int4_kernel<<<static_cast<unsigned>((vectors + 255) / 256), 256, 0, st>>>(
      static_cast<const uint4*>(in), static_cast<uint4*>(out), vectors);
  return check_launch("unpack_int4_kernel");
}

template <int BN, int UW>
int launch_w4(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_s, const CUtensorMap& tm_o,
              const W4Params& p, int tiles_n, int tiles_m, int smem, cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_w4a16_kernel<BN, UW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(tiles_n, tiles_m, 1);
  cfg.blockDim = dim3(w4_threads(UW));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rk_gemm_w4a16_kernel<BN, UW>, tm_w, tm_x, tm_s, tm_o, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "rk_gemm_w4a16_kernel launch: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

}  // namespace
}  // namespace rk

using namespace rk;

extern "C" size_t rk_workspace_bytes(int op, int64_t m, int64_t n, int64_t k) {
  if (m < 1 || n < 1) return 0;
  size_t bytes = RK_WORKSPACE_HEADER;
  if (op == RK_OP_W4A4) bytes += static_cast<size_t>(round_up(m + n, 16)) * static_cast<size_t>(round_up(k, 128));  // int8 copies
  return (bytes + 255) / 256 * 256;
}

namespace {
int noalloc_scratch_address(uint8_t** out);
}

extern "C" int rk_read_status(void* workspace, int* code, void* stream) {
  if (!workspace) {
    // NULL names the scratch array built into the library (the one rk_gemm_int4_noalloc uses)
    uint8_t* builtin = nullptr;
    const int rc = noalloc_scratch_address(&builtin);
    if (rc != RK_OK) return rc;
    workspace = builtin;
  }
  cudaError_t e = cudaStreamSynchronize(as_stream(stream));
  if (e != cudaSuccess) return fail(RK_ECUDA, "rk_read_status: %s", cudaGetErrorString(e));
  int v = 0;
  e = cudaMemcpy(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(RK_ECUDA, "rk_read_status: %s", cudaGetErrorString(e));
  if (code) *code = v;
  if (v != 0) {
    cudaMemset(workspace, 0, sizeof(int));
    return fail(RK_EDEVICE, "a kernel gave up a bounded wait (device code %d)", v);
  }
  return RK_OK;
}

extern "C" int rk_debug_wait_expiry(int on, int spin_limit) {
  if (on && (spin_limit < 64 || spin_limit > (1 << 21))) return fail(RK_EINVAL, "rk_debug_wait_expiry: spin_limit must be 64..2^21");
  g_debug_stall = on ? 1 : 0;
  g_debug_wait_limit = on ? spin_limit : 0;
  return RK_OK;
}

static int gemm_int_common(const void* a, const float* sa, const void* b, const float* sb, const void* bias, void* out,
                           int32_t* acc, int64_t m, int64_t n, int64_t kpad, int bits, int tactic, void* workspace,
                           size_t workspace_bytes, void* stream, const char* who, bool widen_in_scratch = false,
                           const void* residual = nullptr, const void* res_gate = nullptr, int64_t res_tokens = 1) {
  if (bits != 8 && bits != 4) return fail(RK_EINVAL, "%s: bits must be 4 or 8", who);
  if (kpad < 128 || kpad % 128 != 0) return fail(RK_EINVAL, "%s: kpad must be a positive multiple of 128", who);
  if (tactic < 0 || tactic > 7) return fail(RK_EINVAL, "%s: tactic must be 0..7", who);
  if (!acc && (!sa || !sb)) return fail(RK_EINVAL, "%s: null scale pointer", who);
  if (!a || !b) return fail(RK_EINVAL, "%s: null pointer", who);
  if (m < 1 || n < 1 || m > (1 << 24) || n > (1 << 24) || kpad > (1 << 24)) return fail(RK_EINVAL, "%s: bad dimensions", who);
  uint8_t* copies = nullptr;
  size_t copies_bytes = 0;
  if (bits == 4 && !widen_in_scratch) {
    // tcgen05 has no 4-bit integer kind: the kernel fetches the packed nibbles and widens both
    // operands to int8 in shared memory (the products and the int32 sums are identical)
    if (!aligned16(a) || !aligned16(b)) return fail(RK_EINVAL, "%s: operands must be 16-byte aligned", who);
    TcArgs t{};
    t.kind = KIND_I4;
    t.act = a;
    t.wgt = b;
    t.m = m;
    t.n = n;
    t.k_bytes = kpad;
    t.mma_bytes_last = 128;
    t.scale_act = sa;
    t.scale_wgt = sb;
    t.bias = bias;
    t.out = out;
    t.acc_out = acc;
    t.tactic = tactic;
    t.workspace = workspace;
    t.workspace_bytes = workspace_bytes;
    t.stream = as_stream(stream);
    t.who = who;
    t.residual = residual;
    t.res_gate = res_gate;
    t.res_tokens = res_tokens;
    return run_tc(t);
  }
  if (bits == 4) {
    // the variant that widens both operands to int8 in a scratch buffer first and then runs the int8
    // kernel on the copies (kept for rk_gemm_int4_noalloc, whose scratch is built into the library)
    if (!aligned16(a) || !aligned16(b)) return fail(RK_EINVAL, "%s: operands must be 16-byte aligned", who);
    const size_t need = rk_workspace_bytes(RK_OP_W4A4, m, n, kpad);
    if (!workspace || workspace_bytes < need) return fail(RK_EWORKSPACE, "%s: workspace too small for the int8 copies", who);
    uint8_t* a8 = static_cast<uint8_t*>(workspace) + need - static_cast<size_t>(round_up(m + n, 16)) * kpad;
    uint8_t* b8 = a8 + static_cast<size_t>(m) * kpad;
    int rc = unpack_int4(a, a8, m * kpad / 2, as_stream(stream));
    if (rc != RK_OK) return rc;
    rc = unpack_int4(b, b8, n * kpad / 2, as_stream(stream));
    if (rc != RK_OK) return rc;
    a = a8;
    b = b8;
    copies = a8;
    copies_bytes = static_cast<size_t>(round_up(m + n, 16)) * kpad;
    workspace_bytes = need - static_cast<size_t>(round_up(m + n, 16)) * kpad;
  }
  TcArgs t{};
  t.kind = KIND_I8;
  t.act = a;
  t.wgt = b;
  t.m = m;
  t.n = n;
  t.k_bytes = kpad;
  t.mma_bytes_last = 128;
  t.scale_act = sa;
  t.scale_wgt = sb;
  t.bias = bias;
  t.out = out;
  t.acc_out = acc;
  t.tactic = tactic;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = who;
  t.residual = residual;
  t.res_gate = res_gate;
  t.res_tokens = res_tokens;
  int rc = run_tc(t);
  if (rc == RK_OK && copies != nullptr) {
    // leave the whole scratch buffer zero-filled, as every entry point promises
    if (cudaMemsetAsync(copies, 0, copies_bytes, as_stream(stream)) != cudaSuccess)
      return fail(RK_ECUDA, "%s: cudaMemsetAsync failed", who);
  }
  return rc;
}

extern "C" int rk_gemm_int(const void* a, const float* sa, const void* b, const float* sb, const void* bias, void* out,
                           int64_t m, int64_t n, int64_t kpad, int bits, int tactic, void* workspace,
                           size_t workspace_bytes, void* stream) {
  return gemm_int_common(a, sa, b, sb, bias, out, nullptr, m, n, kpad, bits, tactic, workspace, workspace_bytes, stream,
                         "rk_gemm_int");
}

extern "C" int rk_gemm_int_residual(const void* a, const float* sa, const void* b, const float* sb, const void* bias,
                                    const void* residual, const void* gate, int64_t tokens, void* out, int64_t m, int64_t n,
                                    int64_t kpad, int bits, int tactic, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  const char* who = "rk_gemm_int_residual";
  if (!residual || !out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (tokens < 1 || m < 1 || m % tokens != 0) return fail(RK_EINVAL, "%s: m must be a positive multiple of tokens", who);
  if (static_cast<unsigned long long>(m) * static_cast<unsigned long long>(tokens) >= (1ull << 32))
    return fail(RK_EUNSUPPORTED, "%s: m * tokens must stay below 2^32", who);
  if (n % 8 != 0 || (reinterpret_cast<uintptr_t>(residual) & 1u) || (gate && (reinterpret_cast<uintptr_t>(gate) & 1u)))
    return fail(RK_EINVAL, "%s: n must be a multiple of 8 and the bf16 pointers 2-byte aligned", who);
  return gemm_int_common(a, sa, b, sb, bias, out, nullptr, m, n, kpad, bits, tactic, workspace, workspace_bytes, stream, who,
                         false, residual, gate, tokens);
}

extern "C" int rk_gemm_int_acc(const void* a, const void* b, int32_t* acc, int64_t m, int64_t n, int64_t kpad, int bits,
                               int tactic, void* workspace, size_t workspace_bytes, void* stream) {
  if (!acc) return fail(RK_EINVAL, "rk_gemm_int_acc: null pointer");
  return gemm_int_common(a, nullptr, b, nullptr, nullptr, nullptr, acc, m, n, kpad, bits, tactic, workspace,
                         workspace_bytes, stream, "rk_gemm_int_acc");
}

extern "C" int rk_gemm_fp8(const void* a, const float* scale_a, const void* b, const float* scale_b, const void* bias,
                           void* out, int64_t m, int64_t n, int64_t k, int tactic, void* workspace,
                           size_t workspace_bytes, void* stream) {
  if (k < 16 || k % 16 != 0) return fail(RK_EINVAL, "rk_gemm_fp8: k must be a positive multiple of 16");
  if (!scale_a || !scale_b) return fail(RK_EINVAL, "rk_gemm_fp8: null scale pointer");
  TcArgs t{};
  t.kind = KIND_F8;
  t.act = a;
  t.wgt = b;
  t.m = m;
  t.n = n;
  t.k_bytes = k;
  t.mma_bytes_last = static_cast<int>(k % 128 == 0 ? 128 : k % 128);
  t.scale_act = scale_a;
  t.scale_wgt = scale_b;
  t.bias = bias;
  t.out = out;
  t.tactic = tactic & 7;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = "rk_gemm_fp8";
  return run_tc(t);
}

extern "C" int rk_gemm_fp8_producer(const void* x, const void* b, const float* scale_b, const void* bias, void* out,
                                    int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  if (k < 16 || k % 16 != 0) return fail(RK_EINVAL, "rk_gemm_fp8_producer: k must be a positive multiple of 16");
  if (!scale_b) return fail(RK_EINVAL, "rk_gemm_fp8_producer: null scale pointer");
  TcArgs t{};
  t.kind = KIND_F8P;
  t.act = x;
  t.wgt = b;
  t.m = m;
  t.n = n;
  t.k_bytes = k;  // in MMA bytes (e4m3); the bf16 rows are twice as long
  t.mma_bytes_last = static_cast<int>(k % 128 == 0 ? 128 : k % 128);
  t.scale_act = nullptr;  // unit activation scale
  t.scale_wgt = scale_b;
  t.bias = bias;
  t.out = out;
  t.tactic = tactic & 7;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = "rk_gemm_fp8_producer";
  return run_tc(t);
}

extern "C" int rk_gemm_w4a8_mx(const void* a, const void* sfa, const void* b, const void* sfb, const void* bias, void* out,
                               int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                               void* stream) {
  const char* who = "rk_gemm_w4a8_mx";
  if (k < 32 || k % 32 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 32", who);
  if (!sfa || !sfb) return fail(RK_EINVAL, "%s: null scale-factor pointer", who);
  if (!aligned16(sfa) || !aligned16(sfb)) return fail(RK_EINVAL, "%s: scale-factor buffers must be 16-byte aligned", who);
  TcArgs t{};
  // Packed e2m1 rows can go to the tensor core as they are when TMA may expand them into the padded
  // 4-bit layout of kind::mxf8f6f4 (K a multiple of 128, 32-byte aligned rows); otherwise four warps
  // rewrite them to e4m3 in shared memory.
  const bool direct = k % 128 == 0 && reinterpret_cast<uintptr_t>(b) % 32 == 0;
  t.kind = direct ? KIND_MXF8 : KIND_MX48;
  t.wgt_u4 = direct;
  t.act = a;
  t.wgt = b;
  t.m = m;
  t.n = n;
  t.k_bytes = k;  // in MMA bytes (e4m3 after the weights are expanded); packed weight rows are k / 2
  t.mma_bytes_last = static_cast<int>(k % 128 == 0 ? 128 : k % 128);
  t.sf_act = static_cast<const uint8_t*>(sfa);
  t.sf_wgt = static_cast<const uint8_t*>(sfb);
  t.sf_kt = static_cast<int>((k + 127) / 128);
  t.bias = bias;
  t.out = out;
  t.tactic = (tactic & 7) | 2;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = who;
  return run_tc(t);
}

extern "C" int rk_gemm_mxfp8(const void* a, const void* sfa, const void* b, const void* sfb, const void* bias, void* out,
                             int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (k < 32 || k % 32 != 0) return fail(RK_EINVAL, "rk_gemm_mxfp8: k must be a positive multiple of 32");
  if (!sfa || !sfb) return fail(RK_EINVAL, "rk_gemm_mxfp8: null scale-factor pointer");
  if (!aligned16(sfa) || !aligned16(sfb)) return fail(RK_EINVAL, "rk_gemm_mxfp8: scale-factor buffers must be 16-byte aligned");
  TcArgs t{};
  t.kind = KIND_MXF8;
  t.act = a;
  t.wgt = b;
  t.m = m;
  t.n = n;
  t.k_bytes = k;
  t.mma_bytes_last = static_cast<int>(k % 128 == 0 ? 128 : k % 128);
  t.sf_act = static_cast<const uint8_t*>(sfa);
  t.sf_wgt = static_cast<const uint8_t*>(sfb);
  t.sf_kt = static_cast<int>((k + 127) / 128);
  t.bias = bias;
  t.out = out;
  t.tactic = (tactic & 7) | 2;  // no split-K: fp32 partial sums would reorder additions
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = "rk_gemm_mxfp8";
  return run_tc(t);
}

extern "C" int rk_gemm_nvfp4(const void* a, const void* sfa, const float* ga, const void* b, const void* sfb,
                             const float* gb, const void* bias, void* out, int64_t m, int64_t n, int64_t k, int tactic,
                             void* workspace, size_t workspace_bytes, void* stream) {
  if (k < 32 || k % 32 != 0) return fail(RK_EINVAL, "rk_gemm_nvfp4: k must be a positive multiple of 32");
  if (!sfa || !sfb) return fail(RK_EINVAL, "rk_gemm_nvfp4: null scale-factor pointer");
  if (!aligned16(sfa) || !aligned16(sfb)) return fail(RK_EINVAL, "rk_gemm_nvfp4: scale-factor buffers must be 16-byte aligned");
  if (k % 64 != 0) return fail(RK_EUNSUPPORTED, "rk_gemm_nvfp4: k must be a multiple of 64 in this build");
  TcArgs t{};
  t.kind = KIND_NVF4;
  t.act = a;
  t.wgt = b;
  t.m = m;
  t.n = n;
  t.k_bytes = k / 2;
  t.mma_bytes_last = static_cast<int>((k / 2) % 128 == 0 ? 128 : (k / 2) % 128);
  t.scale_act = ga;
  t.scale_wgt = gb;
  t.sf_act = static_cast<const uint8_t*>(sfa);
  t.sf_wgt = static_cast<const uint8_t*>(sfb);
  t.sf_kt = static_cast<int>((k / 16 + 3) / 4);
  t.bias = bias;
  t.out = out;
  t.tactic = (tactic & 7) | 2;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = "rk_gemm_nvfp4";
  return run_tc(t);
}

extern "C" int rk_gemm_nvfp4_swiglu(const void* a, const void* sfa, const float* ga, const void* b_interleaved,
                                    const void* sfb, const float* gb, void* q_out, void* sf_out, int64_t m, int64_t n,
                                    int64_t k, int tactic, void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "rk_gemm_nvfp4_swiglu";
  if (k < 64 || k % 64 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 64", who);
  if (n < 128 || n % 128 != 0) return fail(RK_EINVAL, "%s: n (gate and up rows together) must be a multiple of 128", who);
  if (!sfa || !sfb || !q_out || !sf_out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (!aligned16(sfa) || !aligned16(sfb) || !aligned16(q_out) || !aligned16(sf_out))
    return fail(RK_EINVAL, "%s: buffers must be 16-byte aligned", who);
  TcArgs t{};
  t.kind = KIND_NVF4;
  t.act = a;
  t.wgt = b_interleaved;
  t.m = m;
  t.n = n;
  t.k_bytes = k / 2;
  t.mma_bytes_last = static_cast<int>((k / 2) % 128 == 0 ? 128 : (k / 2) % 128);
  t.scale_act = ga;
  t.scale_wgt = gb;
  t.sf_act = static_cast<const uint8_t*>(sfa);
  t.sf_wgt = static_cast<const uint8_t*>(sfb);
  t.sf_kt = static_cast<int>((k / 16 + 3) / 4);
  t.swiglu_q = q_out;
  t.swiglu_sf = sf_out;
  t.tactic = (tactic & 4) | 2;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = who;
  return run_tc(t);
}

extern "C" int rk_gemm_nvfp4_gated_act(const void* a, const void* sfa, const float* ga, const void* b_interleaved,
                                       const void* sfb, const float* gb, const void* table, float divisor, void* out,
                                       float* scale_out, int64_t m, int64_t n, int64_t k, int tactic, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  const char* who = "rk_gemm_nvfp4_gated_act";
  if (k < 64 || k % 64 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 64", who);
  if (n < 128 || n % 128 != 0) return fail(RK_EINVAL, "%s: n (gate and up rows together) must be a multiple of 128", who);
  if (!sfa || !sfb || !table || !out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (!aligned16(sfa) || !aligned16(sfb) || !aligned16(out)) return fail(RK_EINVAL, "%s: buffers must be 16-byte aligned", who);
  if (scale_out != nullptr && !(divisor > 0.0f)) return fail(RK_EINVAL, "%s: the divisor must be positive", who);
  if (!workspace || workspace_bytes < RK_WORKSPACE_HEADER) return fail(RK_EWORKSPACE, "%s: workspace too small", who);
  unsigned* staging = scale_out != nullptr ? reinterpret_cast<unsigned*>(static_cast<uint8_t*>(workspace) + 64) : nullptr;
  TcArgs t{};
  t.kind = KIND_NVF4;
  t.act = a;
  t.wgt = b_interleaved;
  t.m = m;
  t.n = n;
  t.k_bytes = k / 2;
  t.mma_bytes_last = static_cast<int>((k / 2) % 128 == 0 ? 128 : (k / 2) % 128);
  t.scale_act = ga;
  t.scale_wgt = gb;
  t.sf_act = static_cast<const uint8_t*>(sfa);
  t.sf_wgt = static_cast<const uint8_t*>(sfb);
  t.sf_kt = static_cast<int>((k / 16 + 3) / 4);
  t.swiglu_q = out;
  t.swiglu_sf = staging;
  t.swiglu_table = table;
  t.swiglu_mode = 2;
  t.tactic = (tactic & 4) | 2;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = who;
  const int rc = run_tc(t);
  if (rc != RK_OK || staging == nullptr) return rc;
  return launch_finalize_scale(staging, divisor, scale_out, as_stream(stream));
}

extern "C" int rk_gemm_mxfp8_swiglu(const void* a, const void* sfa, const void* b_interleaved, const void* sfb,
                                    const void* silu_table, void* q_out, void* sf_out, int64_t m, int64_t n, int64_t k,
                                    int tactic, void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "rk_gemm_mxfp8_swiglu";
  if (k < 32 || k % 32 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 32", who);
  if (n < 256 || n % 256 != 0) return fail(RK_EINVAL, "%s: n (gate and up rows together) must be a multiple of 256", who);
  if (!sfa || !sfb || !silu_table || !q_out || !sf_out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (!aligned16(sfa) || !aligned16(sfb) || !aligned16(q_out) || !aligned16(sf_out))
    return fail(RK_EINVAL, "%s: buffers must be 16-byte aligned", who);
  TcArgs t{};
  t.kind = KIND_MXF8;
  t.act = a;
  t.wgt = b_interleaved;
  t.m = m;
  t.n = n;
  t.k_bytes = k;
  t.mma_bytes_last = static_cast<int>(k % 128 == 0 ? 128 : k % 128);
  t.sf_act = static_cast<const uint8_t*>(sfa);
  t.sf_wgt = static_cast<const uint8_t*>(sfb);
  t.sf_kt = static_cast<int>((k + 127) / 128);
  t.swiglu_q = q_out;
  t.swiglu_sf = sf_out;
  t.swiglu_table = silu_table;
  t.swiglu_mode = 1;
  t.tactic = (tactic & 4) | 2;
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = who;
  return run_tc(t);
}

template <int BN>
int launch_w4_fold(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_s, const CUtensorMap& tm_o,
                   const W4Params& p, int tiles_n, int tiles_m, int smem, cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_w4a16_fold_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(tiles_n, tiles_m, 1);
  cfg.blockDim = dim3(kW4fThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rk_gemm_w4a16_fold_kernel<BN>, tm_w, tm_x, tm_s, tm_o, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "rk_gemm_w4a16_fold_kernel launch: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

// The pair kernel: a cluster of two CTAs per 256 channels x 256 activation rows.
int launch_w4_fold2(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_s, const CUtensorMap& tm_o,
                    const W4Params& p, int tiles_n, int tiles_m, int smem, cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_w4a16_fold2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(tiles_n, tiles_m, 1);
  cfg.blockDim = dim3(kW4fThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rk_gemm_w4a16_fold2_kernel, tm_w, tm_x, tm_s, tm_o, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "rk_gemm_w4a16_fold2_kernel launch: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

// Activation batches above 64 rows: scale folded into the expanded weights, one accumulator for all of K.
int run_w4_fold(const void* x, const void* q, const void* scales, W4Params p, int64_t m, int64_t n, int64_t k,
                int scales_bytes, int tactic, cudaStream_t st, const char* who) {
  const int bn = m > 128 ? 256 : 128;
  const int tiles_n = static_cast<int>((n + 127) / 128);
  const int tiles_m = static_cast<int>((m + bn - 1) / bn);
  // tactic bit 3: 256-row tiles on CTA pairs (each CTA stages half of the activation tile), when
  // the channel tiles pair up
  const bool pair = bn == 256 && tiles_n % 2 == 0 && (tactic & 8);
  const int x_bytes = pair ? kW4f2XBytes : bn * 128;
  const int slots = pair ? kW4f2Slots : w4f_slots(bn);
  const int copies = (p.groups + 1) / 2;
  int w_stages = (kSmemBudget - scales_bytes - slots * x_bytes) / kW4PairBytes;
  if (w_stages > kW4MaxW) w_stages = kW4MaxW;
  if (w_stages > copies) w_stages = copies;
  if (w_stages < 1) return fail(RK_EUNSUPPORTED, "%s: shared memory budget exceeded", who);
  p.w_stages = w_stages;
  const int smem = slots * x_bytes + w_stages * kW4PairBytes + scales_bytes + 1024;
  CUtensorMap tm_w, tm_x, tm_s, tm_o;
  const uint32_t group_box = static_cast<uint32_t>(p.groups < 256 ? p.groups : 256);
  int rc = make_map_2d(&tm_s, scales, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n, k / 128, n * 2, 128, group_box,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != RK_OK) return rc;
  rc = make_map_2d(&tm_w, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k / 2, n, k / 2, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  rc = make_map_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, m, k * 2, 64, pair ? 128 : bn,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  // output tiles leave through TMA: 32 rows x 128 channels per store, clipped at the matrix edges
  rc = make_map_2d(&tm_o, p.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n, m, n * 2, 128, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != RK_OK) return rc;
  if (pair) return launch_w4_fold2(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
  return bn == 256 ? launch_w4_fold<256>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st)
                   : launch_w4_fold<128>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
}

extern "C" int rk_gemm_w4a16_g128(const void* x, const void* q, const void* scales, const void* bias, void* out,
                                  int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  const char* who = "rk_gemm_w4a16_g128";
  if (!x || !q || !scales || !out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (m < 1 || n < 1 || k < 128 || k % 128 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 128", who);
  if (n % 8 != 0) return fail(RK_EINVAL, "%s: n must be a multiple of 8", who);
  if (tactic < 0 || tactic > 63) return fail(RK_EINVAL, "%s: tactic must be 0..63", who);
  if (m > (1 << 24) || n > (1 << 24) || k > (1 << 24)) return fail(RK_EUNSUPPORTED, "%s: dimension too large", who);
  Workspace ws;
  int rc = carve_workspace(workspace, workspace_bytes, &ws, who);
  if (rc != RK_OK) return rc;
  // activation rows per CTA: the smallest of 16/32/64/128 that covers m in the fewest tiles
  int bn = 128;
  if (m <= 16) bn = 16;
  else if (m <= 32) bn = 32;
  else if (m <= 64) bn = 64;
  if ((tactic & 4) && bn > 16) bn /= 2;
  const int tiles_n = static_cast<int>((n + 127) / 128);
  const int tiles_m = static_cast<int>((m + bn - 1) / bn);
  W4Params p{};
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.groups = static_cast<int>(k / 128);
  const int scales_bytes = static_cast<int>(round_up((k / 128) * 256, 1024));  // [groups][128] bf16 in shared memory
  if (scales_bytes > 64 * 1024) return fail(RK_EUNSUPPORTED, "%s: k > 32768", who);
  if (!aligned16(scales)) return fail(RK_EINVAL, "%s: scales must be 16-byte aligned", who);
  const int64_t gemv_slabs = k / kGemvSlab;
  const bool gemv_shape = k % kGemvSlab == 0 && (gemv_slabs == 1 || gemv_slabs == 2 || gemv_slabs == 4 || gemv_slabs % 8 == 0);
  if (m == 1 && tactic == 0 && gemv_shape && aligned16(x) && aligned16(q) && aligned16(out)) {
    // one activation row: byte-streaming work for the CUDA cores (any tactic bit keeps the tensor-core kernels)
    GemvParams g{};
    g.q = static_cast<const uint8_t*>(q);
    g.scales = static_cast<const __nv_bfloat16*>(scales);
    g.x = static_cast<const __nv_bfloat16*>(x);
    g.bias = static_cast<const __nv_bfloat16*>(bias);
    g.out = static_cast<__nv_bfloat16*>(out);
    g.n = static_cast<int>(n);
    g.k = static_cast<int>(k);
    const int slabs = static_cast<int>(k / kGemvSlab);
    const int share = slabs < kGemvWarps ? slabs : kGemvWarps;
    const int batches = static_cast<int>(n / kGemvRows);
    const int per_cta = kGemvWarps / share;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((batches + per_cta - 1) / per_cta);
    cfg.blockDim = dim3(kGemvWarps * 32);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, rk_gemv_w4a16_kernel, g);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(RK_ECUDA, "rk_gemv_w4a16_kernel launch: %s", cudaGetErrorString(e));
    }
    return RK_OK;
  }
  if (m > 64 && !(tactic & 2)) {  // tactic bit 1 keeps the per-group-accumulator kernel for any m
    p.ldo = n;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.status = ws.status;
    return run_w4_fold(x, q, scales, p, m, n, k, scales_bytes, tactic, as_stream(stream), who);
  }
  // shared memory: the activation tiles of the slot ring first, the rest goes to the raw-weight
  // ring (group pairs of 16 KB), whose depth is what keeps enough HBM requests in flight
  const int x_bytes = 2 * bn * 128;
  const int slots = w4_slots(bn);
  const int pairs = (p.groups + 1) / 2;
  int w_stages = (kSmemBudget - scales_bytes - slots * x_bytes) / kW4PairBytes;
  if (w_stages > kW4MaxW) w_stages = kW4MaxW;
  if (w_stages > pairs) w_stages = pairs;
  if (w_stages < 1) return fail(RK_EUNSUPPORTED, "%s: shared memory budget exceeded", who);
  p.w_stages = w_stages;
  p.ldo = n;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = ws.status;
  const int smem = slots * x_bytes + w_stages * kW4PairBytes + scales_bytes + 1024;
  if (!aligned16(scales)) return fail(RK_EINVAL, "%s: scales must be 16-byte aligned", who);
  CUtensorMap tm_w, tm_x, tm_s;
  const uint32_t group_box = static_cast<uint32_t>(p.groups < 256 ? p.groups : 256);
  rc = make_map_2d(&tm_s, scales, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n, k / 128, n * 2, 128, group_box,
                   CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != RK_OK) return rc;
  // raw weights: 128 bytes (two K groups) of 128 rows per copy
  rc = make_map_2d(&tm_w, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k / 2, n, k / 2, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  // activations as [k / 64][m][64]: one box {64, bn, 2} is both 64-element column blocks of a K group
  rc = make_map_3d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 64, m, k / 64, k * 2, 128, 64, bn, 2,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  // output rows leave through TMA stores of up to 32 rows x 128 channels, clipped at the matrix edges
  CUtensorMap tm_o;
  rc = make_map_2d(&tm_o, out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n, m, n * 2, 128, static_cast<uint32_t>(bn < 32 ? bn : 32),
                   CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != RK_OK) return rc;
  cudaStream_t st = as_stream(stream);
  if (tactic & 1) {  // four unpack warps instead of eight
    switch (bn) {
      case 16: return launch_w4<16, 4>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
      case 32: return launch_w4<32, 4>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
      case 64: return launch_w4<64, 4>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
      default: break;
    }
  }
  // Sixteen unpack warps put four K groups in flight at once, which shortens the ramp at the start of
  // the K loop; the register file allows them for activation tiles of up to 32 rows.  Chosen by
  // default for K <= 4096 (the ramp is a smaller share of longer loops, which run a little faster
  // with eight); tactic bit 4 forces sixteen, bit 5 forces eight.
  const bool sixteen = (tactic & 16) || (!(tactic & 32) && p.groups <= 32);
  if (sixteen) {
    switch (bn) {
      case 16: return launch_w4<16, 16>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
      case 32: return launch_w4<32, 16>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
      default: break;
    }
  }
  switch (bn) {
    case 16: return launch_w4<16, 8>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
    case 32: return launch_w4<32, 8>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
    case 64: return launch_w4<64, 8>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
    default: return launch_w4<128, 4>(tm_w, tm_x, tm_s, tm_o, p, tiles_n, tiles_m, smem, st);
  }
}

// ------------------------------------------------------------------ W4A4 GEMM without caller scratch
// The int4 GEMM widens both operands to int8 before the tensor-core kernel runs, which normally
// happens in the caller's workspace.  Callers that cannot obtain device memory at call time -
// for example code running inside a fixed memory plan, or a host thread that must not enter the
// allocator - get this variant: the widened copies live in a device array that is part of the
// library image.  Every GPU that loads the library carries the array until the process exits.
constexpr size_t kNoAllocScratchBytes = (8u << 20) + 4096;  // 8 MiB of int8 copies + header
static __device__ __align__(256) uint8_t g_noalloc_scratch[kNoAllocScratchBytes];

namespace {
// The array's name is only a host-side handle; kernels need its device address, which differs
// per device.  Looked up once per device (with that device current) and kept.
int noalloc_scratch_address(uint8_t** out) {
  static std::mutex mu;
  static uint8_t* per_device[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return rk::fail(RK_ECUDA, "cudaGetDevice failed");
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return rk::fail(RK_ECUDA, "cudaGetSymbolAddress(g_noalloc_scratch): %s", cudaGetErrorString(e));
    per_device[dev] = static_cast<uint8_t*>(ptr);
  }
  *out = per_device[dev];
  return RK_OK;
}
}  // namespace

extern "C" int rk_gemm_int4_noalloc(const void* a, const float* sa, const void* b, const float* sb, const void* bias,
                                    void* out, int64_t m, int64_t n, int64_t kpad, int tactic, void* stream) {
  const char* who = "rk_gemm_int4_noalloc";
  if (m < 1 || n < 1 || kpad < 128 || kpad % 128 != 0) return rk::fail(RK_EINVAL, "%s: bad dimensions", who);
  const size_t need = rk_workspace_bytes(RK_OP_W4A4, m, n, kpad);
  if (need > kNoAllocScratchBytes)
    return rk::fail(RK_EUNSUPPORTED,
                    "%s: 256 + round_up(m + n, 16) * kpad, rounded up to 256, = %zu bytes exceed the built-in "
                    "%zu-byte scratch; use rk_gemm_int with a caller workspace",
                    who, need, kNoAllocScratchBytes);
  uint8_t* scratch = nullptr;
  int rc = noalloc_scratch_address(&scratch);
  if (rc != RK_OK) return rc;
  // the status word at the head of the scratch must start at zero; the copies are overwritten anyway
  if (cudaMemsetAsync(scratch, 0, RK_WORKSPACE_HEADER, rk::as_stream(stream)) != cudaSuccess)
    return rk::fail(RK_ECUDA, "%s: cudaMemsetAsync failed", who);
  return gemm_int_common(a, sa, b, sb, bias, out, nullptr, m, n, kpad, 4, tactic, scratch, need, stream, who, true);
}

// ------------------------------------------------------------------ attention over a cached prefix
extern "C" int rk_attention_prefix(const void* q, const void* k_cache, const void* vt_cache, void* out, int64_t batch,
                                   int64_t tokens, int64_t heads, int64_t kv_heads, int64_t head_dim, int64_t cache_rows,
                                   int64_t vt_pitch, int64_t kv_len, float scaling, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  const char* who = "rk_attention_prefix";
  if (!q || !k_cache || !vt_cache || !out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (head_dim != kAttnDim) return fail(RK_EUNSUPPORTED, "%s: head_dim must be %d", who, kAttnDim);
  if (batch < 1 || batch > 65535 || tokens < 1 || tokens > 128 || heads < 1 || kv_heads < 1 || heads % kv_heads != 0)
    return fail(RK_EINVAL, "%s: bad batch / tokens (1..128) / heads", who);
  if (kv_len < 1 || kv_len > cache_rows || kv_len > vt_pitch || vt_pitch % 8 != 0)
    return fail(RK_EINVAL, "%s: kv_len must fit the caches and vt_pitch must be a multiple of 8", who);
  if (kv_len > 2048) return fail(RK_EUNSUPPORTED, "%s: more than 2048 keys", who);
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(vt_cache) || !aligned16(out))
    return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  Workspace ws;
  int rc = carve_workspace(workspace, workspace_bytes, &ws, who);
  if (rc != RK_OK) return rc;
  // query heads per 128-lane tile: as many heads of one KV group as fit
  const int per_kv = static_cast<int>(heads / kv_heads);
  int group = 1;
  for (int g = per_kv; g >= 1; --g)
    if (per_kv % g == 0 && g * tokens <= 128) {
      group = g;
      break;
    }
  const int tiles = static_cast<int>(heads / group);
  // key slices: enough CTAs to occupy the machine, at most 256 keys each, a power of two up to 8
  int splits = 1;
  while (splits < 8 && (tiles * batch * splits * 2 <= kNumSms || (kv_len + splits - 1) / splits > 256)) splits *= 2;
  const int keys = static_cast<int>(round_up((kv_len + splits - 1) / splits, 32));
  if (keys > 256) return fail(RK_EUNSUPPORTED, "%s: key slices above 256 keys", who);
  CUtensorMap tm_q, tm_k, tm_vt;
  // queries [batch * tokens, heads, 256]: a box is 64 dimensions x `group` heads x `tokens` rows
  rc = make_map_3d(&tm_q, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, kAttnDim, heads, batch * tokens, kAttnDim * 2,
                   heads * kAttnDim * 2, 64, static_cast<uint32_t>(group), static_cast<uint32_t>(tokens),
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  // keys [batch * kv_heads, cache_rows, 256]; rows past kv_len are masked in the kernel, rows past cache_rows read as zero
  rc = make_map_3d(&tm_k, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, kAttnDim, cache_rows, batch * kv_heads, kAttnDim * 2,
                   cache_rows * kAttnDim * 2, 64, static_cast<uint32_t>(keys), 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  // transposed values [batch * kv_heads, 256, vt_pitch]: a box is 64 keys x 256 dimensions
  rc = make_map_3d(&tm_vt, vt_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, vt_pitch, kAttnDim, batch * kv_heads, vt_pitch * 2,
                   kAttnDim * vt_pitch * 2, 64, kAttnDim, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  AttnParams p{};
  p.tokens = static_cast<int>(tokens);
  p.heads = static_cast<int>(heads);
  p.kv_heads = static_cast<int>(kv_heads);
  p.group = group;
  p.kv_len = static_cast<int>(kv_len);
  p.keys = keys;
  p.splits = splits;
  p.scaling = scaling;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = ws.status;
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured_dev[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(rk_attn_prefix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured_dev[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(splits, tiles, static_cast<unsigned>(batch));
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = kAttnSmem;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rk_attn_prefix_kernel, tm_q, tm_k, tm_vt, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "rk_attn_prefix_kernel launch: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

// ------------------------------------------------------------------ column-parallel FP8 GEMM with a fused exchange
namespace rk {
// One warp; lane g watches rank g's entry of this rank's flag array until it reaches the number of
// this wait (the kernel keeps its own call counter, so it does not depend on anything the GEMM of
// the same call writes except the flags themselves, this rank's own flag included).  It is
// launched as a programmatic dependent of that GEMM: it may start while the GEMM still runs - every
// CTA of the GEMM is resident by then - and returns when the last slab has arrived.  The kernel
// launched after it overlaps its prologue with all of that and is released when this one ends.
__global__ void wait_peer_flags_kernel(const int* flags, int ranks, int* wait_counter, int spin_max, int* status) {
  pdl_launch_dependents();
  const int g = threadIdx.x;
  int expected = 0;
  if (g == 0) {
    expected = *wait_counter + 1;
    *wait_counter = expected;
  }
  expected = __shfl_sync(0xffffffffu, expected, 0);
  if (g >= ranks) return;
  const int* flag = flags + g;
  for (int it = 0; it < spin_max; ++it) {
    int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v - expected >= 0) return;  // counters only grow (wrap-around safe comparison)
    __nanosleep(it < 64 ? 40 : 400);
  }
  atomicCAS(status, 0, 107);  // a slab did not arrive in time
}
}  // namespace rk

extern "C" int rk_gemm_fp8_column_parallel(const void* a, const float* scale_a, const void* b, const float* scale_b,
                                           const void* bias, int64_t m, int64_t n_local, int64_t k,
                                           void* const* out_ptrs, void* multicast_out, int64_t ld_total, int64_t col0,
                                           void* const* flag_ptrs, int rank, int ranks, void* epoch_counter,
                                           void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "rk_gemm_fp8_column_parallel";
  if (!flag_ptrs || !scale_a || !scale_b || !epoch_counter) return fail(RK_EINVAL, "%s: null pointer", who);
  if ((out_ptrs == nullptr) == (multicast_out == nullptr))
    return fail(RK_EINVAL, "%s: give the ranks' output pointers or the multicast address, not both", who);
  if (ranks < 1 || ranks > 8 || rank < 0 || rank >= ranks) return fail(RK_EINVAL, "%s: 1..8 ranks", who);
  if (k < 16 || k % 16 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 16", who);
  if (col0 < 0 || col0 % 8 != 0 || ld_total % 8 != 0 || n_local % 8 != 0 || col0 + n_local > ld_total)
    return fail(RK_EINVAL, "%s: the slab must lie inside the output and start on a multiple of 8 columns", who);
  if (multicast_out != nullptr && !aligned16(multicast_out)) return fail(RK_EINVAL, "%s: misaligned multicast address", who);
  PeerArgs peer{};
  for (int g = 0; g < ranks; ++g) {
    if (!flag_ptrs[g]) return fail(RK_EINVAL, "%s: bad pointer for rank %d", who, g);
    peer.flags[g] = static_cast<int*>(flag_ptrs[g]);
  }
  for (int g = 0; g < ranks && out_ptrs != nullptr; ++g) {
    if (!out_ptrs[g] || !aligned16(out_ptrs[g])) return fail(RK_EINVAL, "%s: bad output pointer for rank %d", who, g);
    peer.out[g] = out_ptrs[g];
  }
  peer.mc_out = multicast_out;
  peer.ld = ld_total;
  peer.col0 = col0;
  peer.count = ranks;
  peer.rank = rank;
  peer.epoch = static_cast<int*>(epoch_counter);
  TcArgs t{};
  t.peer = &peer;
  t.kind = KIND_F8;
  t.act = a;
  t.wgt = b;
  t.m = m;
  t.n = n_local;
  t.k_bytes = k;
  t.mma_bytes_last = static_cast<int>(k % 128 == 0 ? 128 : k % 128);
  t.scale_act = scale_a;
  t.scale_wgt = scale_b;
  t.bias = bias;
  t.tactic = 2;  // no split-K: every CTA stores finished values
  t.workspace = workspace;
  t.workspace_bytes = workspace_bytes;
  t.stream = as_stream(stream);
  t.who = who;
  return run_tc(t);
}

extern "C" int rk_wait_peers(const void* flags, int ranks, void* wait_counter, void* workspace, size_t workspace_bytes,
                             void* stream) {
  const char* who = "rk_wait_peers";
  if (!flags || !wait_counter) return fail(RK_EINVAL, "%s: null pointer", who);
  if (ranks < 1 || ranks > 8) return fail(RK_EINVAL, "%s: 1..8 ranks", who);
  Workspace ws;
  int rc = carve_workspace(workspace, workspace_bytes, &ws, who);
  if (rc != RK_OK) return rc;
  const int limit = g_debug_wait_limit > 0 ? g_debug_wait_limit : (1 << 21);  // with 400 ns sleeps: roughly a second
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, wait_peer_flags_kernel, static_cast<const int*>(flags), ranks,
                                     static_cast<int*>(wait_counter), limit, ws.status);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "%s: %s", who, cudaGetErrorString(e));
  }
  return RK_OK;
}
