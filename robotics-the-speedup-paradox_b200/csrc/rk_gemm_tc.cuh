// Warp-specialised tcgen05 GEMM for operands that TMA can place directly in MMA layout:
// int8 x int8 -> s32 (W8A8), e4m3 x e4m3 -> f32 (per-tensor FP8), MXFP8 and NVFP4 block-scaled.
//
//   D[rowsA, rowsB] = A[rowsA, K] . B[rowsB, K]^T        (both operands K-major)
//
// A CTA computes 128 x bn accumulator tiles that live in TMEM.  The "A role" (128 rows on the MMA
// M axis, one TMEM lane per row) is taken by the weights when `swap` is set, so that a ragged,
// small activation row count lands on the MMA N axis (any multiple of 16 up to 256) instead of
// being padded to 128.
//
// Two schedules:
//   * persistent (splits == 1): grid = min(tiles, SMs); each CTA walks tiles t, t + grid, ...;
//     the accumulator is double-buffered in TMEM so the epilogue of one tile overlaps the MMAs
//     of the next; output goes through a shared-memory staging tile and a TMA store.
//   * split-K (splits > 1): a thread-block cluster of `splits` CTAs shares one output tile, each
//     CTA reducing a slice of K; partial accumulators are exchanged through distributed shared
//     memory (no global scratch, no atomics, fixed summation order) and each CTA finishes and
//     stores a slice of the tile's columns.  Used when the output has too few tiles to put
//     every SM to work streaming weights.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (warp w owns TMEM lanes 32*(w%4) .. +31).
//
// Three further kinds feed an operand that is NOT stored in the MMA's type: W4A4 (both operands
// packed int4, widened to int8: tcgen05 has no 4-bit integer kind), the FP8 "producer" GEMM (bf16
// activations converted to e4m3 with unit scale) and W4A8-MX (MXFP4 weights expanded to e4m3, which
// represents every e2m1 value exactly, against MXFP8 activations; used when K is not a multiple of
// 128 - otherwise TMA itself expands the packed rows into the padded 4-bit layout that
// kind::mxf8f6f4 reads and the plain MXFP8 kind runs).  For these, TMA lands the raw
// bytes in a staging part of the pipeline stage and eight more warps (6..13, 448 threads in all)
// rewrite them in shared memory into the 128-byte-swizzled K-major tile the MMA reads; the
// converted operand never exists in global memory.  These kinds run the persistent, non-swapped
// schedule with 128-row weight tiles.
#pragma once

#include <cuda.h>
#include <cuda_fp8.h>

#include "rk_common.cuh"

namespace rk {

enum GemmKind : int {
  KIND_I8 = 0, KIND_F8 = 1, KIND_MXF8 = 2, KIND_NVF4 = 3,
  KIND_I4 = 4,    // int4 x int4, both widened to int8 in shared memory, then as KIND_I8
  KIND_F8P = 5,   // bf16 activations converted to e4m3 in shared memory, e4m3 weights, then as KIND_F8
  KIND_MX48 = 6,  // MXFP8 activations x MXFP4 weights (expanded to e4m3 in shared memory), then as KIND_MXF8
};
// how a raw operand tile is rewritten into the MMA's type
enum XformOp : int { XF_NONE = 0, XF_INT4_TO_INT8 = 1, XF_BF16_TO_E4M3 = 2, XF_E2M1_TO_E4M3 = 3 };

constexpr int kGemmThreads = 192;
constexpr int kXformWarps = 8;           // rewriting is ALU-latency bound: two warps per scheduler
constexpr int kXformThreads = kXformWarps * 32;
constexpr int kGemmThreadsXform = kGemmThreads + kXformThreads;
constexpr int kTileA = 128;        // rows of the A-role tile (MMA M)
constexpr int kStageKBytes = 128;  // bytes of K per pipeline stage (one 128-byte swizzle atom)
constexpr int kMaxStages = 8;
constexpr int kOutBufBytes = 16 * 1024;    // one output staging buffer (one or two are carved)
constexpr int kVecBytes = 2 * 1024;        // per-tile B-role scale and bias vectors, 256 f32 entries each

struct GemmParams {
  int m;        // activation rows (output rows)
  int n;        // weight rows (output columns)
  int kblocks;  // number of 128-byte K blocks in the whole K extent
  int k_valid_mmas_last;  // MMAs (32 bytes of K each) to issue in the last K block (1..4)
  int bn;       // rows of the B-role tile (MMA N): multiple of 16, <= 256
  int swap;     // 1: A role = weights, B role = activations
  int splits;   // split-K factor == cluster size along z (1 = persistent schedule)
  int stages;   // pipeline depth
  int tmem_cols;
  int acc_stride;  // TMEM columns between the accumulator buffers
  int acc_bufs;    // 1 or 2 accumulator buffers in TMEM
  int out_bufs;    // 1 or 2 output staging buffers in shared memory
  int tiles_a, tiles_b;
  long long ldo;  // output row stride (elements)
  const float* scale_act;   // KIND_I8: [m] row scales.  other kinds: optional pointer to one scalar
  const float* scale_wgt;   // KIND_I8: [n] channel scales.  other kinds: optional pointer to one scalar
  const __nv_bfloat16* bias;  // [n] or null
  __nv_bfloat16* out;         // [m, ldo]
  int* acc_out;               // optional raw accumulators [m, n] (s32 or f32 bits), written instead of `out`
  const uint8_t* sf_act;      // block-scaled: swizzled scale-factor buffers
  const uint8_t* sf_wgt;
  int sf_kt;                  // 512-byte scale chunks per 128-row block along K
  int sfb_blocks;             // 128-row scale blocks fetched per B-role tile (1..3; a tile may straddle blocks)
  int sf_rows_b;              // rows of the B-role operand (its scale buffer holds ceil(rows / 128) blocks)
  int wait_limit;             // spin limit of every bounded wait (kWaitSpinMax unless a test shortens it)
  int debug_stall;            // test aid: the producer announces bytes that never arrive (first stage)
  int issue_block;            // issue a stage's tensor-core instructions as one straight-line block
  int fmt_a, fmt_b;           // KIND_MXF8: element formats of the A- and B-role operands (e4m3, or e2m1 for 4-bit
                              // weights that TMA expands to the 16-byte-padded layout of kind::mxf8f6f4)
  int tx_deficit;             // bytes per stage that the copies report short of the shared-memory bytes written
  // Column-parallel mode (peer_count > 0): this GPU computes one slab of columns of a wider output
  // that every GPU of the group holds in full.  A finished, staged chunk leaves either
  //  - through TMA stores into every rank's buffer (one descriptor per rank, kernel parameters: each
  //    describes this rank's slab inside that rank's buffer, this rank's own included), or
  //  - when peer_mc is set, through `multimem.st` to the multicast address of the buffers: ONE store
  //    leaves this GPU and the NVSwitch delivers it to every rank, so the bytes on this GPU's links
  //    do not grow with the number of ranks.
  // When the launch's last CTA has seen all stores complete it raises this rank's entry in every
  // rank's flag array.  Stores only: nothing is loaded from a peer.
  __nv_bfloat16* peer_mc;        // multicast address of the [m, peer_ld] output, or null
  long long peer_ld, peer_col0;  // row stride of the full output and first column of this slab (multicast form)
  int* peer_flags[8];            // every rank's flag array [ranks]
  int peer_count, peer_rank;
  // Gated residual update in the epilogue: out = bf16(residual + t), t = y or bf16(y * gate[row / tokens]),
  // y = the bf16 value the plain epilogue would have stored.  Rows are activation rows, columns channels.
  const __nv_bfloat16* residual;  // [m, n] or null
  const __nv_bfloat16* res_gate;  // [m / tokens, n] or null
  unsigned res_magic;             // 2^32 / tokens + 1 (row / tokens by one multiply; 0: tokens == 1)
  unsigned peer_mask;            // ranks whose buffer receives the TMA stores (all of them)
  int* peer_epoch;               // this rank's call counter (device memory): the launch that finishes call e writes e
  unsigned* peer_counter;        // device word counting the CTAs of this launch that have finished
  int* status;                // device status word
};

template <int KIND>
struct KindTraits;
struct NoXform {
  static constexpr int kXformA = XF_NONE, kXformB = XF_NONE;  // activations / weights (these kinds never swap)
  static constexpr int kRawA = 0, kRawB = 0;                  // raw bytes per row and pipeline stage
  static constexpr int kThreads = kGemmThreads;
};
template <>
struct KindTraits<KIND_I8> : NoXform {
  static constexpr int kBase = KIND_I8;
  static constexpr bool kBlockScaled = false;
  static constexpr int kSfChunksPerStage = 0;
};
template <>
struct KindTraits<KIND_F8> : NoXform {
  static constexpr int kBase = KIND_F8;
  static constexpr bool kBlockScaled = false;
  static constexpr int kSfChunksPerStage = 0;
};
template <>
struct KindTraits<KIND_MXF8> : NoXform {
  static constexpr int kBase = KIND_MXF8;
  static constexpr bool kBlockScaled = true;
  static constexpr int kSfChunksPerStage = 1;  // 128 elements of K = 4 scale factors per row = one 512 B chunk
};
template <>
struct KindTraits<KIND_NVF4> : NoXform {
  static constexpr int kBase = KIND_NVF4;
  static constexpr bool kBlockScaled = true;
  static constexpr int kSfChunksPerStage = 4;  // 256 elements of K = 16 scale factors per row
};
template <>
struct KindTraits<KIND_I4> {
  static constexpr int kBase = KIND_I8;
  static constexpr bool kBlockScaled = false;
  static constexpr int kSfChunksPerStage = 0;
  static constexpr int kXformA = XF_INT4_TO_INT8, kXformB = XF_INT4_TO_INT8;
  static constexpr int kRawA = 64, kRawB = 64;
  static constexpr int kThreads = kGemmThreadsXform;
};
template <>
struct KindTraits<KIND_F8P> {
  static constexpr int kBase = KIND_F8;
  static constexpr bool kBlockScaled = false;
  static constexpr int kSfChunksPerStage = 0;
  static constexpr int kXformA = XF_BF16_TO_E4M3, kXformB = XF_NONE;
  static constexpr int kRawA = 256, kRawB = 0;
  static constexpr int kThreads = kGemmThreadsXform;
};
template <>
struct KindTraits<KIND_MX48> {
  static constexpr int kBase = KIND_MXF8;
  static constexpr bool kBlockScaled = true;
  static constexpr int kSfChunksPerStage = 1;
  static constexpr int kXformA = XF_NONE, kXformB = XF_E2M1_TO_E4M3;
  static constexpr int kRawA = 0, kRawB = 64;
  static constexpr int kThreads = kGemmThreadsXform;
};

__host__ __device__ inline int gemm_raw_bytes_a(int kind) { return kind == KIND_I4 ? 64 : (kind == KIND_F8P ? 256 : 0); }
__host__ __device__ inline int gemm_raw_bytes_b(int kind) { return (kind == KIND_I4 || kind == KIND_MX48) ? 64 : 0; }

// One pipeline stage: [A-role tile][B-role tile][scale chunks][raw A rows][raw B rows]
__host__ __device__ inline int gemm_stage_sf_bytes(int kind, int sfb_blocks) {
  int chunks = (kind == KIND_MXF8 || kind == KIND_MX48) ? 1 : (kind == KIND_NVF4 ? 4 : 0);
  return chunks * 512 * (1 + sfb_blocks);
}
__host__ __device__ inline int gemm_stage_bytes(int kind, int bn, int sfb_blocks) {
  int data = kTileA * kStageKBytes + bn * kStageKBytes;
  int raw = kTileA * gemm_raw_bytes_a(kind) + bn * gemm_raw_bytes_b(kind);
  return (data + gemm_stage_sf_bytes(kind, sfb_blocks) + raw + 1023) / 1024 * 1024;
}

// ---- rewriting a raw operand tile into the MMA's type (warps 6..9, 128 threads) -----------------
// Destination: `rows` x 128 bytes, K-major, 128-byte swizzle (16-byte chunk c of row r at
// r * 128 + ((c ^ (r & 7)) << 4)), exactly what a SWIZZLE_128B TMA box would have written.
__device__ __forceinline__ uint32_t swz128(int row, int chunk) {
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}
// two's-complement nibbles (low nibble = even k) -> int8, eight per 32-bit word
__device__ __forceinline__ void widen_int4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t even = __vsub4((w & 0x0F0F0F0Fu) ^ 0x08080808u, 0x08080808u);
  const uint32_t odd = __vsub4(((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u, 0x08080808u);
  lo = __byte_perm(even, odd, 0x5140);  // k0 k1 k2 k3
  hi = __byte_perm(even, odd, 0x7362);  // k4 k5 k6 k7
}
// e2m1 codes (low nibble = even k) -> the e4m3 bytes of the same values: 0, .5, 1, 1.5, 2, 3, 4, 6
__device__ __forceinline__ uint32_t e2m1x4_to_e4m3(uint32_t h) {  // four nibbles in the low 16 bits
  // two byte permutes: the magnitude bits of every nibble select from the table of the eight e4m3
  // magnitudes, the sign bit selects 0x00 or 0x80
  const uint32_t mag = __byte_perm(0x3C383000u, 0x4C484440u, h & 0x7777u);
  const uint32_t sign = __byte_perm(0x00008000u, 0u, (h >> 3) & 0x1111u);
  return mag | sign;
}
// ROWS is a compile-time row count (a multiple of 32): the loops unroll completely, all shared-memory
// loads of a thread are issued first and the conversions of different chunks interleave.  The four
// rewriting warps are one warp per scheduler, so their stream is latency bound unless it carries
// this much instruction-level parallelism.
template <int OP, int ROWS>
__device__ __forceinline__ void xform_tile(const uint8_t* raw, uint8_t* dst, int t) {
  if constexpr (OP == XF_INT4_TO_INT8 || OP == XF_E2M1_TO_E4M3) {
    // raw row = 64 bytes; a thread takes 16 raw bytes (32 codes) = two destination chunks
    constexpr int kIter = ROWS * 4 / kXformThreads;
    static_assert(ROWS * 4 % kXformThreads == 0, "rows per tile must fill the rewriting threads");
    uint4 v[kIter];
#pragma unroll
    for (int it = 0; it < kIter; ++it) {
      const int i = it * kXformThreads + t;
      v[it] = *reinterpret_cast<const uint4*>(raw + (i >> 2) * 64 + (i & 3) * 16);
    }
#pragma unroll
    for (int it = 0; it < kIter; ++it) {
      const int i = it * kXformThreads + t;
      const int r = i >> 2, c = i & 3;
      const uint32_t w[4] = {v[it].x, v[it].y, v[it].z, v[it].w};
      uint32_t o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if constexpr (OP == XF_INT4_TO_INT8) {
          widen_int4(w[j], o[2 * j], o[2 * j + 1]);
        } else {
          o[2 * j] = e2m1x4_to_e4m3(w[j] & 0xFFFFu);
          o[2 * j + 1] = e2m1x4_to_e4m3(w[j] >> 16);
        }
      }
      *reinterpret_cast<uint4*>(dst + swz128(r, 2 * c)) = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4*>(dst + swz128(r, 2 * c + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
    }
  } else if constexpr (OP == XF_BF16_TO_E4M3) {
    // raw row = 256 bytes (128 bf16); a thread takes 32 raw bytes (16 values) = one destination chunk
    constexpr int kIter = ROWS * 8 / kXformThreads;
#pragma unroll
    for (int half = 0; half < 2; ++half) {  // two batches of kIter / 2 chunks keep the register count moderate
      uint4 a[kIter / 2], b[kIter / 2];
#pragma unroll
      for (int it = 0; it < kIter / 2; ++it) {
        const int i = (half * (kIter / 2) + it) * kXformThreads + t;
        a[it] = *reinterpret_cast<const uint4*>(raw + (i >> 3) * 256 + (i & 7) * 32);
        b[it] = *reinterpret_cast<const uint4*>(raw + (i >> 3) * 256 + (i & 7) * 32 + 16);
      }
#pragma unroll
      for (int it = 0; it < kIter / 2; ++it) {
        const int i = (half * (kIter / 2) + it) * kXformThreads + t;
        const int r = i >> 3, c = i & 7;
        const uint32_t w[8] = {a[it].x, a[it].y, a[it].z, a[it].w, b[it].x, b[it].y, b[it].z, b[it].w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t packed = 0;
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const uint32_t pair = w[2 * j + e];
            // e4m3 of the value clamped to +-448 (unit scale), the arithmetic of the per-tensor quantizer
            const float lo = fminf(448.0f, fmaxf(-448.0f, __uint_as_float(pair << 16)));
            const float hi = fminf(448.0f, fmaxf(-448.0f, __uint_as_float(pair & 0xFFFF0000u)));
            const uint32_t c2 = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
            packed |= c2 << (16 * e);
          }
          o[j] = packed;
        }
        *reinterpret_cast<uint4*>(dst + swz128(r, c)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}
// B-role tiles of the rewriting kinds are 128 rows, or 64 for a narrow weight matrix
template <int OP>
__device__ __forceinline__ void xform_tile_b(const uint8_t* raw, uint8_t* dst, int rows, int t) {
  if (rows == 128) xform_tile<OP, 128>(raw, dst, t);
  else xform_tile<OP, 64>(raw, dst, t);
}

// The final value written for output element (m, n) from its 32-bit accumulator.
template <int KIND>
__device__ __forceinline__ float finish_value(uint32_t acc_bits, float s_act, float s_wgt, bool has_bias,
                                              float bias) {
  if constexpr (KIND == KIND_I8) {
    // float(acc) * sa, then * sb, then + bias: three separately rounded fp32 operations.
    float t = __int2float_rn(static_cast<int>(acc_bits));
    t = __fmul_rn(t, s_act);
    t = __fmul_rn(t, s_wgt);
    if (has_bias) t = __fadd_rn(t, bias);
    return t;
  } else {
    float t = __fmul_rn(__uint_as_float(acc_bits), __fmul_rn(s_act, s_wgt));
    if (has_bias) t = __fadd_rn(t, bias);
    return t;
  }
}

// The gated residual update (see GemmParams::residual) on one finished value; row < m and col < n.
template <class Params>
__device__ __forceinline__ float with_residual(const Params& p, float v, int row, int col) {
  float y = __bfloat162float(__float2bfloat16_rn(v));
  if (p.res_gate != nullptr) {
    const unsigned batch = p.res_magic ? __umulhi(static_cast<unsigned>(row), p.res_magic) : static_cast<unsigned>(row);
    const float g = __bfloat162float(p.res_gate[static_cast<long long>(batch) * p.n + col]);
    y = __bfloat162float(__float2bfloat16_rn(__fmul_rn(y, g)));
  }
  return __fadd_rn(__bfloat162float(p.residual[static_cast<long long>(row) * p.n + col]), y);
}

// The same on sixteen values whose varying coordinate runs first .. first + 15 (activation rows when
// `rows_vary`, else channels) at one fixed other coordinate.  All loads are issued before the first
// use - from clamped, hence always valid, addresses through the read-only path - so that they
// overlap instead of paying one L2 round trip each (measured: +14 us per 400 x 1024 GEMM when every
// value waited for its own loads).  Values beyond `lim` or with `fixed_ok` false are left as they are.
template <class Params>
__device__ __forceinline__ void with_residual16(const Params& p, float (&v)[16], int first, int lim, int fixed, bool fixed_ok,
                                                bool rows_vary) {
  const unsigned short* const res = reinterpret_cast<const unsigned short*>(p.residual);
  const unsigned short* const gat = reinterpret_cast<const unsigned short*>(p.res_gate);
  const int fixed_c = min(fixed, (rows_vary ? p.n : p.m) - 1);
  unsigned short r16[16], g16[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int t = min(first + j, lim - 1);
    const int row = rows_vary ? t : fixed_c, col = rows_vary ? fixed_c : t;
    r16[j] = __ldg(res + static_cast<long long>(row) * p.n + col);
    g16[j] = 0;
    if (gat != nullptr) {
      const unsigned batch = p.res_magic ? __umulhi(static_cast<unsigned>(row), p.res_magic) : static_cast<unsigned>(row);
      g16[j] = __ldg(gat + static_cast<long long>(batch) * p.n + col);
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float y = __bfloat162float(__float2bfloat16_rn(v[j]));
    if (gat != nullptr)
      y = __bfloat162float(__float2bfloat16_rn(__fmul_rn(y, __uint_as_float(static_cast<uint32_t>(g16[j]) << 16))));
    const float updated = __fadd_rn(__uint_as_float(static_cast<uint32_t>(r16[j]) << 16), y);
    if (fixed_ok && first + j < lim) v[j] = updated;
  }
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dsmem_ld_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}

// one 16-byte store to a multicast address: the switch writes it into every bound GPU's memory
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Multicast form of the output stores, executed by all 128 epilogue threads on a staged region.
//   swap layout:     `rows` activation rows x 128 channels, row-major (256 bytes per row)
//   non-swap layout: 128 activation rows x 64 channels, rows of 128 bytes in the 128-byte swizzle
// (m0, n0) = first activation row / first channel (inside the slab) of the region.
__device__ __forceinline__ void multicast_store_region(const GemmParams& p, const uint8_t* stage, bool swap_layout, int rows,
                                                       int m0, int n0, int et) {
  const int per_row = swap_layout ? 16 : 8;
  const int shift = swap_layout ? 4 : 3;
  for (int pc = et; pc < rows * per_row; pc += 128) {
    const int rr = pc >> shift, ch = pc & (per_row - 1);
    const int gm = m0 + rr, gn = n0 + ch * 8;
    if (gm < p.m && gn < p.n) {  // the slab's width is a multiple of 8: a piece exists whole or not at all
      const uint8_t* src = swap_layout ? stage + rr * 256 + ch * 16 : stage + rr * 128 + ((ch ^ (rr & 7)) << 4);
      multimem_st_16(p.peer_mc + static_cast<long long>(gm) * p.peer_ld + p.peer_col0 + gn, *reinterpret_cast<const uint4*>(src));
    }
  }
}

// The kernel body.  The tensor maps are kernel parameters of the callers below (`peer_maps`: the
// store descriptors of the column-parallel mode, one per rank, or null).
// RESIDUAL: the epilogue applies GemmParams::residual (a separate instantiation: the 64 values it keeps
// in flight would otherwise cost every launch of the kind its registers).
template <int KIND, bool RESIDUAL = false>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_out,
                                             const CUtensorMap* peer_maps, const GemmParams& p) {
  using T = KindTraits<KIND>;
  constexpr int BK = T::kBase;  // the MMA kind and epilogue this kind runs on
  constexpr bool kXform = T::kXformA != XF_NONE || T::kXformB != XF_NONE;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_raw_full[kMaxStages];   // raw operand bytes have landed (rewriting kinds)
  __shared__ __align__(8) uint64_t bar_raw_empty[kMaxStages];  // the rewriting warps have read them
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int verdict_epi[2];
  __shared__ volatile int verdict_xf[2];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));  // generic pointer to smem_base
  const int stage_bytes = gemm_stage_bytes(KIND, p.bn, p.sfb_blocks);
  const int rb_b = p.sfb_blocks;  // 128-row scale blocks fetched per B tile
  const uint32_t spin_max = static_cast<uint32_t>(p.wait_limit);
  // offsets inside a stage: [A-role tile][B-role tile][scale chunks][raw A rows][raw B rows]
  const uint32_t raw_a_off = (kTileA + p.bn) * kStageKBytes + gemm_stage_sf_bytes(KIND, p.sfb_blocks);
  const uint32_t raw_b_off = raw_a_off + kTileA * T::kRawA;
  // shared memory map: [pipeline stages][output staging, 1 or 2 x 16 KB][B-role scale + bias vectors]
  const uint32_t out_stage_off = p.stages * stage_bytes;
  const uint32_t vec_off = out_stage_off + p.out_bufs * kOutBufBytes;

  const bool split_mode = p.splits > 1;
  const int num_tiles = p.tiles_a * p.tiles_b;
  const int tile_first = split_mode ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int tile_step = split_mode ? num_tiles : static_cast<int>(gridDim.x);  // split mode: exactly one tile
  const int split = split_mode ? static_cast<int>(blockIdx.z) : 0;
  const int kb_begin = static_cast<int>((static_cast<long long>(p.kblocks) * split) / p.splits);
  const int kb_end = static_cast<int>((static_cast<long long>(p.kblocks) * (split + 1)) / p.splits);
  const int nkb = kb_end - kb_begin;

  pdl_launch_dependents();
  if (threadIdx.x == 64) {  // first thing, by a thread that has no part in the set-up
    // The weight rows of this CTA's first tile start their way from DRAM to L2 during set-up, while
    // the preceding kernel drains (weights are parameters, never that kernel's output).
    if (tile_first < num_tiles) {
      const int row_a0 = (tile_first / p.tiles_b) * kTileA;
      const int row_b0 = (tile_first % p.tiles_b) * p.bn;
      const int ahead = min(nkb, p.stages);
      for (int i = 0; i < ahead; ++i) {
        if (p.swap) tma_prefetch_l2_2d(&tm_a, (kb_begin + i) * kStageKBytes, row_a0);
        else tma_prefetch_l2_2d(&tm_b, (kb_begin + i) * kStageKBytes, row_b0);
      }
    }
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), kXform ? 1 + kXformWarps : 1);  // the producer's announcement (+ the rewriting warps)
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_raw_full[s]), 1);
      mbar_init(smem_u32(&bar_raw_empty[s]), kXformWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), 128);
    }
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane < p.peer_count && peer_maps != nullptr) tma_prefetch_desc(peer_maps + lane);
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // from here on global memory is read and written
  const uint32_t tmem_base = tmem_base_slot;
  // TMEM columns: two accumulator buffers, then (block-scaled kinds) the scale factors.
  const uint32_t tmem_sfa = tmem_base + p.acc_bufs * p.acc_stride;
  const uint32_t tmem_sfb = tmem_sfa + 16;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // the whole warp walks the loop (uniform control flow); the copies are issued by one elected lane
    {
      const uint32_t on = elect_one();
      // Weights are read once: let them leave L2 first.  Activations are re-read by every tile.
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const uint64_t pol_a = p.swap ? pol_w : pol_x;
      const uint64_t pol_b = p.swap ? pol_x : pol_w;
      const uint8_t* sf_a = p.swap ? p.sf_wgt : p.sf_act;
      const uint8_t* sf_b = p.swap ? p.sf_act : p.sf_wgt;
      Ring ring{0, 0};
      bool alive = true;
      // a barrier probe costs a shared-memory round trip: the probe of the NEXT stage is issued before
      // this stage's copies and read one trip later, so a stage that is already free costs no wait
      uint32_t ready = 0;
      const uint32_t tx_data = (kTileA + p.bn) * kStageKBytes - p.tx_deficit;
      for (int tile = tile_first; tile < num_tiles && alive; tile += tile_step) {
        const int row_a0 = (tile / p.tiles_b) * kTileA;
        const int row_b0 = (tile % p.tiles_b) * p.bn;
        for (int i = 0; i < nkb; ++i) {
          const int s = ring.stage;
          const uint32_t ph = ring.phase;
          if constexpr (kXform) {
            // raw rows may be refilled as soon as the rewriting warps have read them, long before the
            // MMAs of the stage's previous use complete; only an operand that TMA writes straight into
            // the MMA's tile has to wait for those
            if (!mbar_wait_bounded(smem_u32(&bar_raw_empty[s]), ph ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_EMPTY, spin_max)) {
              alive = false;
              break;
            }
            if constexpr (T::kXformA == XF_NONE || T::kXformB == XF_NONE || T::kBlockScaled) {
              if (!mbar_wait_bounded(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_EMPTY, spin_max)) {
                alive = false;
                break;
              }
            }
            ring.advance(p.stages);
          } else {
            if (!ready && !mbar_wait_bounded(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_EMPTY, spin_max)) {
              alive = false;
              break;
            }
            ring.advance(p.stages);
            ready = mbar_test_wait(smem_u32(&bar_empty[ring.stage]), ring.phase ^ 1);
          }
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t sa = smem_base + s * stage_bytes;
          const uint32_t sb = sa + kTileA * kStageKBytes;
          const int kb = kb_begin + i;
          uint32_t tx = tx_data;
          // scale chunks present in this K block (the last block of a ragged K holds fewer)
          int cs = 0, nb = 0;
          const int blk_b0 = row_b0 >> 7;  // first 128-row scale block of the B tile
          if constexpr (T::kBlockScaled) {
            cs = min(T::kSfChunksPerStage, p.sf_kt - kb * T::kSfChunksPerStage);
            nb = min(rb_b, ((p.sf_rows_b + 127) >> 7) - blk_b0);  // blocks that exist in the buffer
            tx += cs * 512 * (1 + nb);
          }
          if (p.debug_stall && i == 0 && tile == tile_first) tx += 16;  // test aid: this phase never completes
          if constexpr (!kXform) {
            mbar_arrive_expect_tx(full, tx, on);
            tma_load_2d_hint(sa, &tm_a, kb * kStageKBytes, row_a0, full, pol_a, on);
            tma_load_2d_hint(sb, &tm_b, kb * kStageKBytes, row_b0, full, pol_b, on);
          } else {
            // operands stored in the MMA's type go straight to their tile; the others land as raw rows
            // (unswizzled boxes of kRaw bytes per row) for the rewriting warps
            const uint32_t raw_full = smem_u32(&bar_raw_full[s]);
            uint32_t tx_direct = tx - tx_data, tx_raw = 0;
            if constexpr (T::kXformA == XF_NONE) tx_direct += kTileA * kStageKBytes;
            else tx_raw += kTileA * T::kRawA;
            if constexpr (T::kXformB == XF_NONE) tx_direct += p.bn * kStageKBytes;
            else tx_raw += p.bn * T::kRawB;
            mbar_arrive_expect_tx(full, tx_direct, on);
            mbar_arrive_expect_tx(raw_full, tx_raw, on);
            if constexpr (T::kXformA == XF_NONE) tma_load_2d_hint(sa, &tm_a, kb * kStageKBytes, row_a0, full, pol_a, on);
            else tma_load_2d_hint(sa + raw_a_off, &tm_a, kb * T::kRawA, row_a0, raw_full, pol_a, on);
            if constexpr (T::kXformB == XF_NONE) tma_load_2d_hint(sb, &tm_b, kb * kStageKBytes, row_b0, full, pol_b, on);
            else tma_load_2d_hint(sa + raw_b_off, &tm_b, kb * T::kRawB, row_b0, raw_full, pol_b, on);
          }
          if constexpr (T::kBlockScaled) {
            // Scale factors: contiguous 512-byte chunks in the 128-row swizzled global layout.
            const uint32_t ssf = sb + p.bn * kStageKBytes;
            const int c = T::kSfChunksPerStage;
            const long long chunk0 = static_cast<long long>(kb) * c;
            const uint8_t* src_a = sf_a + (static_cast<long long>(row_a0 / 128) * p.sf_kt + chunk0) * 512;
            asm volatile(
                "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %4, 0;\n\t"
                "@q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t}"
                ::"r"(ssf), "l"(src_a), "r"(cs * 512), "r"(full), "r"(on) : "memory");
            for (int rb = 0; rb < nb; ++rb) {
              const uint8_t* src_b = sf_b + (static_cast<long long>(blk_b0 + rb) * p.sf_kt + chunk0) * 512;
              asm volatile(
                  "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %4, 0;\n\t"
                  "@q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t}"
                  ::"r"(ssf + (1 + rb) * c * 512), "l"(src_b), "r"(cs * 512), "r"(full), "r"(on) : "memory");
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (uniform control flow); the tcgen05 instructions execute in one
    // elected lane.  Every lane takes part in the barrier waits.
    {
      const uint32_t on = elect_one();
      Ring ring{0, 0}, racc{0, 0};
      bool alive = true;
      uint32_t ready = 0;  // answer of the early probe of the next stage's "full" barrier
      // instruction descriptor(s) and the descriptor of stage 0 are loop invariants
      uint32_t idesc = 0;
      if constexpr (BK == KIND_I8) idesc = umma_idesc(DFMT_S32, FMT_S8, FMT_S8, 128, p.bn);
      else if constexpr (BK == KIND_F8) idesc = umma_idesc(DFMT_F32, FMT_E4M3, FMT_E4M3, 128, p.bn);
      else if constexpr (BK == KIND_MXF8) idesc = umma_idesc_bs(p.fmt_a, p.fmt_b, 128, p.bn, 1, 0, 0);
      else idesc = umma_idesc_bs(FMT_E2M1_MXF4, FMT_E2M1_MXF4, 128, p.bn, 0, 0, 0);
      const uint64_t adesc0 = umma_desc_k128(smem_base);
      const uint64_t bdesc0 = umma_desc_k128(smem_base + kTileA * kStageKBytes);
      const uint32_t stage_step = static_cast<uint32_t>(stage_bytes) >> 4;
      for (int tile = tile_first; tile < num_tiles && alive; tile += tile_step, racc.advance(p.acc_bufs)) {
        const int ab = racc.stage;
        // the epilogue must have drained this accumulator buffer (its previous use)
        if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[ab]), racc.phase ^ 1, &abort_flag, p.status,
                               RK_DEV_TIMEOUT_ACC_FREE, spin_max)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * p.acc_stride;
        // a B tile that starts inside a 128-row scale block reads its factors from the matching
        // column of the block's four (one 32-bit column per 32 rows)
        const uint32_t sfb_col0 = static_cast<uint32_t>((((tile % p.tiles_b) * p.bn) & 127) >> 5);
        for (int i = 0; i < nkb; ++i) {
          const int s = ring.stage;
          const uint32_t ph = ring.phase;
          if (!ready && !mbar_wait_bounded(smem_u32(&bar_full[s]), ph, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL, spin_max)) {
            alive = false;
            break;
          }
          tc_fence_after();
          ring.advance(p.stages);  // probe the next stage now, read the answer after this stage's MMAs
          ready = mbar_test_wait(smem_u32(&bar_full[ring.stage]), ring.phase);
          const uint32_t sa = smem_base + s * stage_bytes;
          const uint32_t sb = sa + kTileA * kStageKBytes;
          const uint64_t adesc = adesc0 + static_cast<uint64_t>(s * stage_step);
          const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(s * stage_step);
          const int nmma = (kb_begin + i == p.kblocks - 1) ? p.k_valid_mmas_last : 4;
          if constexpr (T::kBlockScaled && !kXform) {
            // Whole K blocks of the block-scaled kinds: up to 17 tensor-core instructions per stage (scale
            // copies, MMAs, the commit).  The issuing thread's cost per instruction is what paces these
            // kinds, so the elected lane runs them as one straight-line block without per-instruction
            // predicates and with descriptors that differ from a per-stage base by constants (NVFP4
            // 816 x 16384 x 2048: 34.1 -> 25.9 us).  For the kinds without scale copies (five
            // instructions per stage) the same block measured slower than the predicated form below.
            if (p.issue_block && nmma == 4 && (kb_begin + i + 1) * T::kSfChunksPerStage <= p.sf_kt) {
              if (on) {
                constexpr int c = T::kSfChunksPerStage;
                const uint64_t sfdesc0 = umma_desc_noswizzle(sb + p.bn * kStageKBytes, 16, 128);
                const uint32_t accumulate0 = i > 0 ? 1u : 0u;
                if (rb_b == 1) {
#pragma unroll
                  for (int j = 0; j < c; ++j) {
                    tmem_cp_32x128b_warpx4_np(tmem_sfa + j * 4, sfdesc0 + static_cast<uint64_t>(j * 32));
                    tmem_cp_32x128b_warpx4_np(tmem_sfb + j * 4, sfdesc0 + static_cast<uint64_t>((c + j) * 32));
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < c; ++j) {
                    tmem_cp_32x128b_warpx4_np(tmem_sfa + j * 4, sfdesc0 + static_cast<uint64_t>(j * 32));
                    tmem_cp_32x128b_warpx4_np(tmem_sfb + j * 8, sfdesc0 + static_cast<uint64_t>((c + j) * 32));
                    tmem_cp_32x128b_warpx4_np(tmem_sfb + j * 8 + 4, sfdesc0 + static_cast<uint64_t>((2 * c + j) * 32));
                  }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint32_t accumulate = k > 0 ? 1u : accumulate0;
                  if constexpr (BK == KIND_MXF8)
                    mma_mxf8_np(d_tmem, adesc + k * 2, bdesc + k * 2,
                                idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29), tmem_sfa,
                                tmem_sfb + sfb_col0, accumulate);
                  else
                    mma_nvf4_np(d_tmem, adesc + k * 2, bdesc + k * 2, idesc, tmem_sfa + k * 4,
                                tmem_sfb + k * rb_b * 4 + sfb_col0, accumulate);
                }
                tc_commit_np(smem_u32(&bar_empty[s]));
              }
              __syncwarp();
              continue;
            }
          }
          if constexpr (T::kBlockScaled) {
            const uint32_t ssf = sb + p.bn * kStageKBytes;
            const int c = T::kSfChunksPerStage;
            // chunk (row block r, k chunk j) of the stage -> 4 TMEM columns
            const int cs = min(c, p.sf_kt - (kb_begin + i) * c);
            for (int j = 0; j < cs; ++j) {
              tmem_cp_32x128b_warpx4(tmem_sfa + j * 4, umma_desc_noswizzle(ssf + j * 512, 16, 128), on);
              for (int rb = 0; rb < rb_b; ++rb)
                tmem_cp_32x128b_warpx4(tmem_sfb + (j * rb_b + rb) * 4,
                                       umma_desc_noswizzle(ssf + ((1 + rb) * c + j) * 512, 16, 128), on);
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (k < nmma) {
              const uint32_t accumulate = (i > 0 || k > 0) ? 1u : 0u;
              // 32 bytes of K per MMA: advance the descriptor start address by 32 >> 4.
              const uint64_t ad = adesc + static_cast<uint64_t>(k * 2);
              const uint64_t bd = bdesc + static_cast<uint64_t>(k * 2);
              if constexpr (BK == KIND_I8) {
                mma_i8(d_tmem, ad, bd, idesc, accumulate, on);
              } else if constexpr (BK == KIND_F8) {
                mma_f8f6f4(d_tmem, ad, bd, idesc, accumulate, on);
              } else if constexpr (BK == KIND_MXF8) {
                // four MMAs share one set of scale columns; byte k of each 32-bit column is theirs
                // (scale-factor ids: bits [4,6) for B, [29,31) for A)
                mma_mxf8(d_tmem, ad, bd, idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29),
                         tmem_sfa, tmem_sfb + sfb_col0, accumulate, on);
              } else {
                mma_nvf4(d_tmem, ad, bd, idesc, tmem_sfa + k * 4, tmem_sfb + k * rb_b * 4 + sfb_col0, accumulate, on);
              }
            }
          }
          tc_commit(smem_u32(&bar_empty[s]), on);  // stage reusable once these MMAs have read it
        }
        if (alive) tc_commit(smem_u32(&bar_acc_full[ab]), on);  // accumulator complete
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ operand rewriting (warps 6..13, rewriting kinds only)
    if constexpr (kXform) {
      const int t = threadIdx.x - kGemmThreads;  // 0..kXformThreads-1
      Ring ring{0, 0};
      bool alive = true;
      uint32_t xf_iter = 0;
      for (int tile = tile_first; tile < num_tiles && alive; tile += tile_step) {
        for (int i = 0; i < nkb; ++i) {
          const int s = ring.stage;
          // the raw bytes are here, and the MMAs of the stage's previous use have read the tiles that
          // are about to be overwritten
          // (one thread waits on the barriers, parked by the hardware; a named barrier releases the rest)
          if (t == 0) {
            const bool got = mbar_wait_bounded(smem_u32(&bar_raw_full[s]), ring.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_RAW, spin_max) &&
                             mbar_wait_bounded(smem_u32(&bar_empty[s]), ring.phase ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_EMPTY, spin_max);
            verdict_xf[xf_iter & 1] = got ? 1 : 0;
          }
          asm volatile("bar.sync 2, %0;" ::"n"(kXformThreads) : "memory");
          if (verdict_xf[xf_iter++ & 1] == 0) {
            alive = false;
            break;
          }
          ring.advance(p.stages);
          uint8_t* const stage = smem_gen + s * stage_bytes;
          if constexpr (T::kXformA != XF_NONE) xform_tile<T::kXformA, kTileA>(stage + raw_a_off, stage, t);
          if constexpr (T::kXformB != XF_NONE)
            xform_tile_b<T::kXformB>(stage + raw_b_off, stage + kTileA * kStageKBytes, p.bn, t);
          fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(smem_u32(&bar_full[s]));       // first: a refill announcement must not overtake this arrival
            mbar_arrive(smem_u32(&bar_raw_empty[s]));
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    const int et = quad * 32 + lane;  // 0..127: TMEM lane == row of the A-role tile
    const int lim_a = p.swap ? p.n : p.m;
    const int lim_b = p.swap ? p.m : p.n;
    const bool has_bias = p.bias != nullptr && p.acc_out == nullptr;
    float* const vec_scale = reinterpret_cast<float*>(smem_gen + vec_off);  // [256] B-role scales
    float* const vec_bias = vec_scale + 256;                                // [256] B-role bias (non-swap)
    float s_act_scalar = 1.0f, s_wgt_scalar = 1.0f;
    if constexpr (BK != KIND_I8) {
      if (p.scale_act) s_act_scalar = *p.scale_act;
      if (p.scale_wgt) s_wgt_scalar = *p.scale_wgt;
    }
    Ring racc{0, 0};
    uint32_t epi_iter = 0;
    int pending_store = 0;  // epilogue thread 0: a TMA store may still be reading a staging buffer
    // one staged box to its destination: this GPU's output, or the slab's place in every rank's buffer
    auto store_box = [&](uint32_t src, int x, int y) {
      if (p.peer_count > 0) {
        for (int g = 0; g < p.peer_count; ++g)
          if ((p.peer_mask >> g) & 1u) tma_store_2d(peer_maps + g, src, x, y);
      } else {
        tma_store_2d(&tm_out, src, x, y);
      }
    };
    int obuf = 0;
    for (int tile = tile_first; tile < num_tiles; tile += tile_step, racc.advance(p.acc_bufs)) {
      const int ab = racc.stage;
      const int row_a0 = (tile / p.tiles_b) * kTileA;
      const int row_b0 = (tile % p.tiles_b) * p.bn;
      const int ra = row_a0 + et;
      const bool ra_ok = ra < lim_a;
      // per-thread constants of the A-role row, and the B-role vectors of this tile into shared memory
      float row_scale = 1.0f, row_bias = 0.0f;
      if (p.acc_out == nullptr) {
        if constexpr (BK == KIND_I8) {
          if (ra_ok) row_scale = p.swap ? p.scale_wgt[ra] : p.scale_act[ra];
        }
        if (p.swap && has_bias && ra_ok) row_bias = __bfloat162float(p.bias[ra]);
        epi_bar_sync();  // previous tile's readers of the vectors are done
        for (int j = et; j < p.bn; j += 128) {
          const int rb = row_b0 + j;
          float sv = 1.0f, bv = 0.0f;
          if (rb < lim_b) {
            if constexpr (BK == KIND_I8) sv = p.swap ? p.scale_act[rb] : p.scale_wgt[rb];
            if (!p.swap && has_bias) bv = __bfloat162float(p.bias[rb]);
          }
          vec_scale[j] = sv;
          vec_bias[j] = bv;
        }
        epi_bar_sync();
      }
      const bool ok = mbar_wait_group(smem_u32(&bar_acc_full[ab]), racc.phase, et == 0, 1, 128, &abort_flag, p.status,
                                      RK_DEV_TIMEOUT_ACC, verdict_epi, epi_iter++, spin_max);
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ab * p.acc_stride + (static_cast<uint32_t>(quad * 32) << 16);

      if (split_mode) {
        // ---- split-K: park the raw partial accumulators in shared memory, column-major [bn][128]
        uint32_t* const part = reinterpret_cast<uint32_t*>(smem_gen);
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld_16(t_acc + c0, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c0 + j) * 128 + et] = ok ? r[j] : 0u;
        }
        continue;  // reduction happens after the cluster barrier below
      }

      if (p.acc_out != nullptr) {
        // ---- raw accumulator dump (parity aid): plain stores
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld_16(t_acc + c0, r);
          tc_wait_ld();
          if (ra_ok && ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int rbj = row_b0 + c0 + j;
              if (rbj < lim_b) {
                const long long om = p.swap ? rbj : ra, on = p.swap ? ra : rbj;
                p.acc_out[om * p.n + on] = static_cast<int>(r[j]);
              }
            }
          }
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_acc_empty[ab]));
        continue;
      }

      // ---- swapped tiles that fit: stage the whole tile once, then issue all its TMA stores.  The
      // chunk-by-chunk path below costs two CTA-wide rendezvous per 32 columns; for a CTA that owns
      // a single tile nothing overlaps that tail, so it is taken in one pass whenever the tile
      // ([bn][128] bf16) fits the staging area.
      // A CTA that owns exactly one tile may also use its pipeline stages as staging memory: once the
      // accumulator is complete every copy into them has landed and every MMA has read them.
      const bool one_tile = num_tiles <= static_cast<int>(gridDim.x);
      const bool fits_out = p.bn * 256 <= p.out_bufs * kOutBufBytes;
      const bool fits_pipe = one_tile && p.bn * 256 <= p.stages * stage_bytes;
      if (p.swap && (fits_out || fits_pipe)) {
        uint8_t* const stage = fits_out ? smem_gen + out_stage_off : smem_gen;
        if (et == 0 && pending_store) tma_store_wait_read<0>();
        epi_bar_sync();
        __nv_bfloat16* const srow = reinterpret_cast<__nv_bfloat16*>(stage);
        for (int c0 = 0; c0 < p.bn; c0 += 32) {
          const bool two = c0 + 32 <= p.bn;  // warp-uniform
          uint32_t r0[16], r1[16];
          __syncwarp();
          tmem_ld_16(t_acc + c0, r0);
          if (two) {
            tmem_ld_16(t_acc + c0 + 16, r1);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) r1[j] = 0u;
          }
          tc_wait_ld();
          // the per-column scales are read into registers BEFORE the first store: a shared-memory load
          // placed between the stores would have to wait for each of them (the two may alias)
          float sv0[16], sv1[16];
          if constexpr (BK == KIND_I8) {
            const float4* const vs4 = reinterpret_cast<const float4*>(vec_scale + c0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 a = vs4[q];
              sv0[4 * q] = a.x, sv0[4 * q + 1] = a.y, sv0[4 * q + 2] = a.z, sv0[4 * q + 3] = a.w;
              const float4 b = two ? vs4[4 + q] : a;
              sv1[4 * q] = b.x, sv1[4 * q + 1] = b.y, sv1[4 * q + 2] = b.z, sv1[4 * q + 3] = b.w;
            }
          }
          float v0[16], v1[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if constexpr (BK == KIND_I8) {
              v0[j] = finish_value<BK>(r0[j], sv0[j], row_scale, has_bias, row_bias);
              v1[j] = finish_value<BK>(r1[j], sv1[j], row_scale, has_bias, row_bias);
            } else {
              v0[j] = finish_value<BK>(r0[j], s_act_scalar, s_wgt_scalar, has_bias, row_bias);
              v1[j] = finish_value<BK>(r1[j], s_act_scalar, s_wgt_scalar, has_bias, row_bias);
            }
          }
          if constexpr (RESIDUAL) {  // swapped tile: this thread's channel, columns are activation rows
            with_residual16(p, v0, row_b0 + c0, lim_b, ra, ra_ok, true);
            with_residual16(p, v1, row_b0 + c0 + 16, lim_b, ra, ra_ok, true);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) srow[(c0 + j) * 128 + et] = __float2bfloat16_rn(v0[j]);
          if (two) {
#pragma unroll
            for (int j = 0; j < 16; ++j) srow[(c0 + 16 + j) * 128 + et] = __float2bfloat16_rn(v1[j]);
          }
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_acc_empty[ab]));
        fence_proxy_async_smem();
        epi_bar_sync();
        if (p.peer_mc != nullptr) {
          if (ok) multicast_store_region(p, stage, true, p.bn, row_b0, row_a0, et);
        } else if (et == 0) {
          if (ok)
            for (int r0w = 0; r0w < p.bn; r0w += 32) store_box(smem_u32(stage + r0w * 256), row_a0, row_b0 + r0w);
          tma_store_commit();
          pending_store = 1;
        }
        continue;
      }

      // ---- finish values, stage them in shared memory, store with TMA (clipped at the matrix edge)
      // swap:     chunk = 32 activation rows x 128 channels, row-major [32][128] bf16 (8 KB)
      // non-swap: chunk = 128 activation rows x 64 channels, 128-byte-swizzled rows (16 KB)
      const int chunk_cols = p.swap ? 32 : 64;
      for (int cc = 0; cc < p.bn; cc += chunk_cols, obuf = (p.out_bufs == 2) ? (obuf ^ 1) : 0) {
        uint8_t* const stage = smem_gen + out_stage_off + obuf * kOutBufBytes;
        // the staging buffer was handed to TMA earlier: wait until that store has read it
        if (et == 0 && pending_store) {
          if (p.out_bufs == 2) tma_store_wait_read<1>();
          else tma_store_wait_read<0>();
        }
        epi_bar_sync();
        const int ncols = min(chunk_cols, p.bn - cc);
        for (int c0 = 0; c0 < ncols; c0 += 16) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld_16(t_acc + cc + c0, r);
          tc_wait_ld();
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float sv = vec_scale[cc + c0 + j];
            if constexpr (BK == KIND_I8) {
              v[j] = p.swap ? finish_value<BK>(r[j], sv, row_scale, has_bias, row_bias)
                            : finish_value<BK>(r[j], row_scale, sv, has_bias, vec_bias[cc + c0 + j]);
            } else {
              v[j] = finish_value<BK>(r[j], s_act_scalar, s_wgt_scalar, has_bias,
                                        p.swap ? row_bias : vec_bias[cc + c0 + j]);
            }
          }
          if constexpr (RESIDUAL) with_residual16(p, v, row_b0 + cc + c0, lim_b, ra, ra_ok, p.swap != 0);
          if (p.swap) {
            __nv_bfloat16* const srow = reinterpret_cast<__nv_bfloat16*>(stage);
#pragma unroll
            for (int j = 0; j < 16; ++j) srow[(c0 + j) * 128 + et] = __float2bfloat16_rn(v[j]);
          } else {
            // 16 values = two 16-byte chunks (index c0/8, c0/8+1) of this thread's 128-byte row
            uint4 lo = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                  pack_bf16x2(v[6], v[7]));
            uint4 hi = make_uint4(pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]), pack_bf16x2(v[12], v[13]),
                                  pack_bf16x2(v[14], v[15]));
            const int ch = c0 >> 3;
            *reinterpret_cast<uint4*>(stage + et * 128 + (((ch) ^ (et & 7)) << 4)) = lo;
            *reinterpret_cast<uint4*>(stage + et * 128 + (((ch + 1) ^ (et & 7)) << 4)) = hi;
          }
        }
        if (cc + chunk_cols >= p.bn) {
          // last TMEM read of this tile is done: hand the accumulator buffer back to the MMA warp
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_acc_empty[ab]));
        }
        fence_proxy_async_smem();
        epi_bar_sync();
        if (p.peer_mc != nullptr) {
          if (ok) {
            if (p.swap) multicast_store_region(p, stage, true, min(32, p.bn - cc), row_b0 + cc, row_a0, et);
            else multicast_store_region(p, stage, false, 128, row_a0, row_b0 + cc, et);
          }
        } else if (et == 0) {
          if (ok) {
            if (p.swap) store_box(smem_u32(stage), row_a0, row_b0 + cc);
            else store_box(smem_u32(stage), row_b0 + cc, row_a0);
          }
          tma_store_commit();
          pending_store = 1;
        }
      }
    }
    if (et == 0) tma_store_wait_read<0>();  // the staging memory has been read; the writes drain after the CTA has left
    if (p.peer_count > 0) {
      // Hand-off.  Each CTA waits until its own stores have completed and orders them - at GPU scope,
      // which is cheap - before it counts itself as finished; the launch's last CTA then issues the
      // ONE system-scope fence of the launch and tells every rank that the slab is there.  (A
      // system-scope fence costs ~3 us here; with one per CTA and one release store per flag the tail
      // of a 20 us kernel measured 8.5 us, with this arrangement the fence is paid once.)
      if (p.peer_mc != nullptr) {
        __threadfence();  // each thread's own multicast stores
        epi_bar_sync();
      }
      if (et == 0) {
        if (p.peer_mc == nullptr) {
          tma_store_wait_all();
          fence_proxy_async_all();
        }
        __threadfence();
        const unsigned done = atomicAdd(p.peer_counter, 1u);
        if (done == gridDim.x - 1) {
          *p.peer_counter = 0u;
          // the call counter lives in device memory, so a replayed CUDA graph announces a fresh value
          const int epoch = *p.peer_epoch + 1;
          *p.peer_epoch = epoch;
          __threadfence_system();  // everything this thread has observed - all CTAs' stores - before the flags
          if (!abort_flag)
            for (int g = 0; g < p.peer_count; ++g)
              asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[g] + p.peer_rank), "r"(epoch) : "memory");
        }
      }
    }
  }

  // ---------------------------------------------------------------- split-K: reduce across the cluster
  if (split_mode) {
    __syncthreads();
    cluster_sync_all();  // every CTA's partial tile is in its shared memory
    if (warp >= 2 && warp < 6) {
      const int quad = warp & 3;
      const int et = quad * 32 + lane;
      const int tile = tile_first;
      const int row_a0 = (tile / p.tiles_b) * kTileA;
      const int row_b0 = (tile % p.tiles_b) * p.bn;
      const int lim_a = p.swap ? p.n : p.m;
      const int lim_b = p.swap ? p.m : p.n;
      const int ra = row_a0 + et;
      const bool has_bias = p.bias != nullptr && p.acc_out == nullptr;
      float s_act_scalar = 1.0f, s_wgt_scalar = 1.0f;
      if constexpr (BK != KIND_I8) {
        if (p.scale_act) s_act_scalar = *p.scale_act;
        if (p.scale_wgt) s_wgt_scalar = *p.scale_wgt;
      }
      // this CTA finishes columns [c_lo, c_hi) of the tile
      const int per = (p.bn + p.splits - 1) / p.splits;
      const int c_lo = static_cast<int>(cluster_ctarank()) * per;
      const int c_hi = min(p.bn, c_lo + per);
      float row_scale = 1.0f, row_bias = 0.0f;
      if (ra < lim_a && p.acc_out == nullptr) {
        if constexpr (BK == KIND_I8) row_scale = p.swap ? p.scale_wgt[ra] : p.scale_act[ra];
        if (p.swap && has_bias) row_bias = __bfloat162float(p.bias[ra]);
      }
      const float* const vec_scale_r = reinterpret_cast<const float*>(smem_gen + vec_off);
      const float* const vec_bias_r = vec_scale_r + 256;
      // shared::cluster base address of every peer's partial tile
      uint32_t peer[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        peer[q] = 0;
        if (q < p.splits)
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[q]) : "r"(smem_base), "r"(q));
      }
      for (int c4 = c_lo; c4 < c_hi; c4 += 4) {
        // issue the loads of four columns from every peer back to back, then add in rank order
        uint32_t v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            v[u][q] = 0u;
            if (q < p.splits && c4 + u < c_hi)
              asm volatile("ld.shared::cluster.u32 %0, [%1];"
                           : "=r"(v[u][q])
                           : "r"(peer[q] + static_cast<uint32_t>((c4 + u) * 128 + et) * 4u)
                           : "memory");
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c4 + u;
          if (c >= c_hi) continue;
          uint32_t total = 0;
          float ftotal = 0.0f;
#pragma unroll
          for (int q = 0; q < 8; ++q) {  // fixed order: rank 0, 1, ... (absent ranks contribute zero)
            if constexpr (BK == KIND_I8) total += v[u][q];
            else ftotal += __uint_as_float(v[u][q]);
          }
          if constexpr (BK != KIND_I8) total = __float_as_uint(ftotal);
          const int rbj = row_b0 + c;
          if (ra >= lim_a || rbj >= lim_b || abort_flag) continue;
          const long long om = p.swap ? rbj : ra, on = p.swap ? ra : rbj;
          if (p.acc_out != nullptr) {
            p.acc_out[om * p.n + on] = static_cast<int>(total);
            continue;
          }
          float val;
          // B-role scale and bias of this column were staged in shared memory by the epilogue prologue
          const float bias_v = p.swap ? row_bias : vec_bias_r[c];
          if constexpr (BK == KIND_I8) {
            const float other = vec_scale_r[c];
            val = p.swap ? finish_value<BK>(total, other, row_scale, has_bias, bias_v)
                         : finish_value<BK>(total, row_scale, other, has_bias, bias_v);
          } else {
            val = finish_value<BK>(total, s_act_scalar, s_wgt_scalar, has_bias, bias_v);
          }
          if constexpr (RESIDUAL) val = with_residual(p, val, static_cast<int>(om), static_cast<int>(on));
          p.out[om * p.ldo + on] = __float2bfloat16_rn(val);
        }
      }
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

template <int KIND, bool RESIDUAL = false>
__global__ void __launch_bounds__(KindTraits<KIND>::kThreads, 1)
rk_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_out, const GemmParams p) {
  gemm_tc_body<KIND, RESIDUAL>(tm_a, tm_b, tm_out, nullptr, p);
}

// The per-tensor FP8 GEMM in column-parallel mode: one store descriptor per rank instead of one output map.
struct PeerMaps {
  CUtensorMap m[8];
};
__global__ void __launch_bounds__(kGemmThreads, 1)
rk_gemm_tc_peer_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                       const __grid_constant__ PeerMaps maps, const GemmParams p) {
  gemm_tc_body<KIND_F8>(tm_a, tm_b, tm_a, maps.m, p);
}

}  // namespace rk
