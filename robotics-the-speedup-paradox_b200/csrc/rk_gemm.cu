// Host side of the tcgen05 GEMM entry points: argument checks, tile / split-K selection,
// TMA tensor-map construction (cached), launches.

#include <cuda.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

#include "rk_gemm_tc.cuh"
#include "rk_gemm_w4.cuh"
#include "rk_host.h"

namespace rk {
namespace {

constexpr int kSmemBudget = 227 * 1024 - 2048;  // dynamic shared memory we ask for at most (static barriers excluded)
constexpr int kNumSms = 148;

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
  uint32_t box_inner, box_rows;
  int dtype, swizzle;
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

// ------------------------------------------------------------------ workspace layout
// [0, 256) status area (word 0 = status, word 16 = amax staging) | counters | partial sums
constexpr size_t kMaxCounters = 8192;
constexpr size_t kCounterBytes = kMaxCounters * sizeof(unsigned);

struct Workspace {
  int* status;
  unsigned* counters;
  int* partial;
  size_t partial_bytes;
};

int carve_workspace(void* ws, size_t bytes, Workspace* out, const char* who) {
  if (!ws || bytes < RK_WORKSPACE_HEADER + kCounterBytes) return fail(RK_EWORKSPACE, "%s: workspace missing or too small", who);
  if (!aligned16(ws)) return fail(RK_EWORKSPACE, "%s: workspace must be 16-byte aligned", who);
  uint8_t* p = static_cast<uint8_t*>(ws);
  out->status = reinterpret_cast<int*>(p);
  out->counters = reinterpret_cast<unsigned*>(p + RK_WORKSPACE_HEADER);
  out->partial = reinterpret_cast<int*>(p + RK_WORKSPACE_HEADER + kCounterBytes);
  out->partial_bytes = bytes - RK_WORKSPACE_HEADER - kCounterBytes;
  return RK_OK;
}

int pow2_at_least(int v, int lo) {
  int r = lo;
  while (r < v) r <<= 1;
  return r;
}

// ------------------------------------------------------------------ tile selection
struct Plan {
  int swap, bn, tiles_a, tiles_b, splits, stages, tmem_cols, smem_bytes;
};

// `tactic` only nudges the shape of the decomposition (it can never change integer results and
// only reorders fp32 partial sums): bit 0 forbids swap, bit 1 forbids split-K, bit 2 halves bn.
Plan make_plan(int kind, int64_t m, int64_t n, int kblocks, int tactic, size_t partial_bytes) {
  Plan pl{};
  const bool block_scaled = kind == KIND_MXF8 || kind == KIND_NVF4;
  // Weights on the 128-lane axis whenever the activation row count fits one or a few
  // B-role tiles; otherwise activations take the 128-lane axis and weights use wide tiles.
  // Block-scaled kinds address scale factors in 128-row blocks, so a B-role tile that is not the
  // only one must start on a multiple of 128 rows: they swap only when one tile covers m.
  pl.swap = (m <= (block_scaled ? 256 : 1024) && !(tactic & 1)) ? 1 : 0;
  if (pl.swap) {
    // smallest number of <=256-row chunks, rows per chunk rounded up to 16 (block-scaled: 32)
    const int chunks = static_cast<int>((m + 255) / 256);
    const int q = block_scaled ? 32 : 16;
    int bn = static_cast<int>(round_up((m + chunks - 1) / chunks, q));
    if ((tactic & 4) && bn >= 2 * q) bn = static_cast<int>(round_up(bn / 2, q));
    pl.bn = bn;
    pl.tiles_a = static_cast<int>((n + 127) / 128);
    pl.tiles_b = static_cast<int>((m + bn - 1) / bn);
  } else {
    pl.bn = (tactic & 4) ? 128 : 256;
    if (n < pl.bn) pl.bn = static_cast<int>(round_up(n, block_scaled ? 32 : 16));
    pl.tiles_a = static_cast<int>((m + 127) / 128);
    pl.tiles_b = static_cast<int>((n + pl.bn - 1) / pl.bn);
  }
  const int stage = gemm_stage_bytes(kind, pl.bn);
  pl.stages = kSmemBudget / stage;
  if (pl.stages > kMaxStages) pl.stages = kMaxStages;
  if (pl.stages > kblocks) pl.stages = kblocks < 2 ? 2 : kblocks;
  pl.smem_bytes = pl.stages * stage + 1024;
  pl.tmem_cols = block_scaled ? 512 : pow2_at_least(pl.bn, 32);
  // split-K: fill the machine when the output has few tiles; keep >= 2 K blocks per split
  pl.splits = 1;
  const long long tiles = static_cast<long long>(pl.tiles_a) * pl.tiles_b;
  if (!(tactic & 2) && tiles < kNumSms && tiles <= static_cast<long long>(kMaxCounters)) {
    int s = static_cast<int>((kNumSms + tiles - 1) / tiles);
    if (s > kblocks / 2) s = kblocks / 2;
    if (static_cast<size_t>(m) * n * 4 > partial_bytes) s = 1;
    if (s > 1) pl.splits = s;
  }
  return pl;
}

template <int KIND>
int launch_tc(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const GemmParams& p, const Plan& pl, cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_tc_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  const dim3 grid(pl.tiles_a, pl.tiles_b, pl.splits);
  rk_gemm_tc_kernel<KIND><<<grid, kGemmThreads, pl.smem_bytes, st>>>(tm_a, tm_b, p);
  return check_launch("rk_gemm_tc_kernel");
}

struct TcArgs {
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
  if (!a.act || !a.wgt || (!a.out && !a.acc_out)) return fail(RK_EINVAL, "%s: null pointer", a.who);
  if (a.m < 1 || a.n < 1 || a.k_bytes < 16) return fail(RK_EINVAL, "%s: empty problem", a.who);
  if (a.m > (1 << 24) || a.n > (1 << 24) || a.k_bytes > (1 << 24)) return fail(RK_EUNSUPPORTED, "%s: dimension too large", a.who);
  if (a.n % 8 != 0) return fail(RK_EINVAL, "%s: n must be a multiple of 8", a.who);
  Workspace ws;
  int rc = carve_workspace(a.workspace, a.workspace_bytes, &ws, a.who);
  if (rc != RK_OK) return rc;
  const int kblocks = static_cast<int>((a.k_bytes + kStageKBytes - 1) / kStageKBytes);
  const Plan pl = make_plan(a.kind, a.m, a.n, kblocks, a.tactic, ws.partial_bytes);

  CUtensorMap tm_act, tm_wgt;
  const uint32_t box_act = pl.swap ? pl.bn : kTileA;
  const uint32_t box_wgt = pl.swap ? kTileA : pl.bn;
  rc = make_map_2d(&tm_act, a.act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.k_bytes, a.m, a.k_bytes, kStageKBytes, box_act,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  rc = make_map_2d(&tm_wgt, a.wgt, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.k_bytes, a.n, a.k_bytes, kStageKBytes, box_wgt,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;

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
  p.ldo = a.n;
  p.scale_act = a.scale_act;
  p.scale_wgt = a.scale_wgt;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.acc_out = a.acc_out;
  p.sf_act = a.sf_act;
  p.sf_wgt = a.sf_wgt;
  p.sf_kt = a.sf_kt;
  p.status = ws.status;
  p.counters = ws.counters;
  p.partial = ws.partial;
  const CUtensorMap& tm_a = pl.swap ? tm_wgt : tm_act;
  const CUtensorMap& tm_b = pl.swap ? tm_act : tm_wgt;
  switch (a.kind) {
    case KIND_I8: return launch_tc<KIND_I8>(tm_a, tm_b, p, pl, a.stream);
    case KIND_F8: return launch_tc<KIND_F8>(tm_a, tm_b, p, pl, a.stream);
    case KIND_MXF8: return launch_tc<KIND_MXF8>(tm_a, tm_b, p, pl, a.stream);
    default: return launch_tc<KIND_NVF4>(tm_a, tm_b, p, pl, a.stream);
  }
}

template <int BN>
int launch_w4(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const W4Params& p, int tiles_n, int tiles_m, int smem,
              cudaStream_t st) {
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rk_gemm_w4a16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBudget + 1024);
    if (e != cudaSuccess) return fail(RK_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  rk_gemm_w4a16_kernel<BN><<<dim3(tiles_n, tiles_m), kW4Threads, smem, st>>>(tm_w, tm_x, p);
  return check_launch("rk_gemm_w4a16_kernel");
}

}  // namespace
}  // namespace rk

using namespace rk;

extern "C" size_t rk_workspace_bytes(int op, int64_t m, int64_t n, int64_t k) {
  (void)k;
  if (m < 1 || n < 1) return 0;
  size_t bytes = RK_WORKSPACE_HEADER + kCounterBytes;
  if (op != RK_OP_W4A16) bytes += static_cast<size_t>(m) * static_cast<size_t>(n) * 4;  // split-K partial sums
  return (bytes + 255) / 256 * 256;
}

extern "C" int rk_read_status(void* workspace, int* code, void* stream) {
  if (!workspace) return fail(RK_EWORKSPACE, "rk_read_status: null workspace");
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

static int gemm_int_common(const void* a, const float* sa, const void* b, const float* sb, const void* bias, void* out,
                           int32_t* acc, int64_t m, int64_t n, int64_t kpad, int bits, int tactic, void* workspace,
                           size_t workspace_bytes, void* stream, const char* who) {
  if (bits != 8) return fail(RK_EUNSUPPORTED, "%s: bits=%d has no kernel in this build", who, bits);
  if (kpad < 128 || kpad % 128 != 0) return fail(RK_EINVAL, "%s: kpad must be a positive multiple of 128", who);
  if (tactic < 0 || tactic > 7) return fail(RK_EINVAL, "%s: tactic must be 0..7", who);
  if (!acc && (!sa || !sb)) return fail(RK_EINVAL, "%s: null scale pointer", who);
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
  return run_tc(t);
}

extern "C" int rk_gemm_int(const void* a, const float* sa, const void* b, const float* sb, const void* bias, void* out,
                           int64_t m, int64_t n, int64_t kpad, int bits, int tactic, void* workspace,
                           size_t workspace_bytes, void* stream) {
  return gemm_int_common(a, sa, b, sb, bias, out, nullptr, m, n, kpad, bits, tactic, workspace, workspace_bytes, stream,
                         "rk_gemm_int");
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

extern "C" int rk_gemm_w4a16_g128(const void* x, const void* q, const void* scales, const void* bias, void* out,
                                  int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  const char* who = "rk_gemm_w4a16_g128";
  if (!x || !q || !scales || !out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (m < 1 || n < 1 || k < 128 || k % 128 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 128", who);
  if (n % 8 != 0) return fail(RK_EINVAL, "%s: n must be a multiple of 8", who);
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
  const int stage = kW4RawBytes + 2 * bn * 128;
  W4Params p{};
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.groups = static_cast<int>(k / 128);
  p.xf_stages = bn >= 128 ? 2 : 3;
  int stages = (kSmemBudget - p.xf_stages * kW4XfBytes) / stage;
  if (stages > kW4MaxStages) stages = kW4MaxStages;
  if (stages > p.groups) stages = p.groups < 2 ? 2 : p.groups;
  p.stages = stages;
  p.ldo = n;
  p.scales = static_cast<const __nv_bfloat16*>(scales);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = ws.status;
  const int smem = stages * stage + p.xf_stages * kW4XfBytes + 1024;
  CUtensorMap tm_w, tm_x;
  rc = make_map_2d(&tm_w, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k / 2, n, k / 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_64B);
  if (rc != RK_OK) return rc;
  rc = make_map_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, m, k * 2, 64, bn, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != RK_OK) return rc;
  cudaStream_t st = as_stream(stream);
  switch (bn) {
    case 16: return launch_w4<16>(tm_w, tm_x, p, tiles_n, tiles_m, smem, st);
    case 32: return launch_w4<32>(tm_w, tm_x, p, tiles_n, tiles_m, smem, st);
    case 64: return launch_w4<64>(tm_w, tm_x, p, tiles_n, tiles_m, smem, st);
    default: return launch_w4<128>(tm_w, tm_x, p, tiles_n, tiles_m, smem, st);
  }
}
