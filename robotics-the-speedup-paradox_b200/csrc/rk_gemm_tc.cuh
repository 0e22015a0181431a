// Warp-specialised tcgen05 GEMM for operands that TMA can place directly in MMA layout:
// int8 x int8 -> s32 (W8A8), e4m3 x e4m3 -> f32 (per-tensor FP8), MXFP8 and NVFP4 block-scaled.
//
//   D[rowsA, rowsB] = A[rowsA, K] . B[rowsB, K]^T        (both operands K-major)
//
// One CTA computes one 128 x bn accumulator tile that lives in TMEM.  The "A role" (128 rows on
// the MMA M axis, one TMEM lane per row) is taken by the weights when `swap` is set, so that a
// ragged, small activation row count lands on the MMA N axis (any multiple of 16 up to 256)
// instead of being padded to 128.  Split-K (grid.z) spreads weight streaming over all SMs for
// small outputs; partial sums are combined in a zero-initialised scratch buffer by the CTA that
// arrives last on a per-tile counter (no spinning), which also restores the scratch to zero.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (warp w owns TMEM lanes 32*(w%4) .. +31).
#pragma once

#include <cuda.h>

#include "rk_common.cuh"

namespace rk {

enum GemmKind : int { KIND_I8 = 0, KIND_F8 = 1, KIND_MXF8 = 2, KIND_NVF4 = 3 };

constexpr int kGemmThreads = 192;
constexpr int kTileA = 128;        // rows of the A-role tile (MMA M)
constexpr int kStageKBytes = 128;  // bytes of K per pipeline stage (one 128-byte swizzle atom)
constexpr int kMaxStages = 8;

struct GemmParams {
  int m;        // activation rows (output rows)
  int n;        // weight rows (output columns)
  int kblocks;  // number of 128-byte K blocks in the whole K extent
  int k_valid_mmas_last;  // MMAs (32 bytes of K each) to issue in the last K block (1..4)
  int bn;       // rows of the B-role tile (MMA N): multiple of 16, <= 256
  int swap;     // 1: A role = weights, B role = activations
  int splits;   // split-K factor (grid.z)
  int stages;   // pipeline depth
  int tmem_cols;
  long long ldo;  // output row stride (elements)
  const float* scale_act;   // KIND_I8: [m] row scales.  KIND_F8: pointer to one scalar.  block-scaled: optional scalar
  const float* scale_wgt;   // KIND_I8: [n] channel scales.  KIND_F8: pointer to one scalar.  block-scaled: optional scalar
  const __nv_bfloat16* bias;  // [n] or null
  __nv_bfloat16* out;         // [m, ldo]
  int* acc_out;               // optional raw accumulators [m, n] (s32 or f32 bits), written instead of `out`
  const uint8_t* sf_act;      // block-scaled: swizzled scale-factor buffers
  const uint8_t* sf_wgt;
  int sf_kt;                  // 512-byte scale chunks per 128-row block along K
  int* status;                // device status word
  unsigned* counters;         // split-K: one arrival counter per output tile (zero between calls)
  int* partial;               // split-K: [m, n] 32-bit partial sums (zero between calls)
};

template <int KIND>
struct KindTraits;
template <>
struct KindTraits<KIND_I8> {
  static constexpr bool kBlockScaled = false;
  static constexpr int kSfChunksPerStage = 0;
};
template <>
struct KindTraits<KIND_F8> {
  static constexpr bool kBlockScaled = false;
  static constexpr int kSfChunksPerStage = 0;
};
template <>
struct KindTraits<KIND_MXF8> {
  static constexpr bool kBlockScaled = true;
  static constexpr int kSfChunksPerStage = 1;  // 128 elements of K = 4 scale factors per row = one 512 B chunk
};
template <>
struct KindTraits<KIND_NVF4> {
  static constexpr bool kBlockScaled = true;
  static constexpr int kSfChunksPerStage = 4;  // 256 elements of K = 16 scale factors per row
};

__host__ __device__ inline int gemm_stage_bytes(int kind, int bn) {
  int data = kTileA * kStageKBytes + bn * kStageKBytes;
  int chunks = kind == KIND_MXF8 ? 1 : (kind == KIND_NVF4 ? 4 : 0);
  int rb = (bn + 127) / 128;
  int sf = chunks * 512 * (1 + rb);
  return (data + sf + 1023) / 1024 * 1024;
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

template <int KIND>
__global__ void __launch_bounds__(kGemmThreads, 1)
rk_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const GemmParams p) {
  using T = KindTraits<KIND>;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_acc;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int is_last_cta;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int stage_bytes = gemm_stage_bytes(KIND, p.bn);
  const int rb_b = (p.bn + 127) / 128;  // 128-row scale blocks in the B tile

  const int tile_a = blockIdx.x;  // 128-row tile index along the A role
  const int tile_b = blockIdx.y;  // bn-row tile index along the B role
  const int split = blockIdx.z;
  const int kb_begin = static_cast<int>((static_cast<long long>(p.kblocks) * split) / p.splits);
  const int kb_end = static_cast<int>((static_cast<long long>(p.kblocks) * (split + 1)) / p.splits);
  const int nkb = kb_end - kb_begin;
  const int row_a0 = tile_a * kTileA;
  const int row_b0 = tile_b * p.bn;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_acc), 1);
    abort_flag = 0;
    is_last_cta = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // TMEM columns: [0, bn) accumulator; block-scaled kinds keep scale factors after it.
  const uint32_t tmem_sfa = tmem_base + 256;
  const uint32_t tmem_sfb = tmem_base + 256 + 16;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // Weights are read once: let them leave L2 first.  Activations are re-read by every tile.
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const uint64_t pol_a = p.swap ? pol_w : pol_x;
      const uint64_t pol_b = p.swap ? pol_x : pol_w;
      const uint8_t* sf_a = p.swap ? p.sf_wgt : p.sf_act;
      const uint8_t* sf_b = p.swap ? p.sf_act : p.sf_wgt;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (i / p.stages) & 1;
        if (!mbar_wait_bounded(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_EMPTY)) break;
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t sa = smem_base + s * stage_bytes;
        const uint32_t sb = sa + kTileA * kStageKBytes;
        const int kb = kb_begin + i;
        uint32_t tx = (kTileA + p.bn) * kStageKBytes;
        // scale chunks present in this K block (the last block of a ragged K holds fewer)
        int cs = 0;
        if constexpr (T::kBlockScaled) {
          cs = min(T::kSfChunksPerStage, p.sf_kt - kb * T::kSfChunksPerStage);
          tx += cs * 512 * (1 + rb_b);
        }
        mbar_arrive_expect_tx(full, tx);
        tma_load_2d_hint(sa, &tm_a, kb * kStageKBytes, row_a0, full, pol_a);
        tma_load_2d_hint(sb, &tm_b, kb * kStageKBytes, row_b0, full, pol_b);
        if constexpr (T::kBlockScaled) {
          // Scale factors: contiguous 512-byte chunks in the 128-row swizzled global layout.
          const uint32_t ssf = sb + p.bn * kStageKBytes;
          const int c = T::kSfChunksPerStage;
          const long long chunk0 = static_cast<long long>(kb) * c;
          const uint8_t* src_a = sf_a + (static_cast<long long>(row_a0 / 128) * p.sf_kt + chunk0) * 512;
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
              ::"r"(ssf), "l"(src_a), "r"(cs * 512), "r"(full) : "memory");
          for (int rb = 0; rb < rb_b; ++rb) {
            const uint8_t* src_b = sf_b + (static_cast<long long>(row_b0 / 128 + rb) * p.sf_kt + chunk0) * 512;
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                ::"r"(ssf + (1 + rb) * c * 512), "l"(src_b), "r"(cs * 512), "r"(full) : "memory");
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (i / p.stages) & 1;
        if (!mbar_wait_bounded(smem_u32(&bar_full[s]), ph, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL)) break;
        tc_fence_after();
        const uint32_t sa = smem_base + s * stage_bytes;
        const uint32_t sb = sa + kTileA * kStageKBytes;
        const uint64_t adesc = umma_desc_k128(sa);
        const uint64_t bdesc = umma_desc_k128(sb);
        const int nmma = (kb_begin + i == p.kblocks - 1) ? p.k_valid_mmas_last : 4;
        if constexpr (T::kBlockScaled) {
          const uint32_t ssf = sb + p.bn * kStageKBytes;
          const int c = T::kSfChunksPerStage;
          // chunk (row block r, k chunk j) of the stage -> 4 TMEM columns
          const int cs = min(c, p.sf_kt - (kb_begin + i) * c);
          for (int j = 0; j < cs; ++j) {
            tmem_cp_32x128b_warpx4(tmem_sfa + j * 4, umma_desc_noswizzle(ssf + j * 512, 16, 128));
            for (int rb = 0; rb < rb_b; ++rb)
              tmem_cp_32x128b_warpx4(tmem_sfb + (j * rb_b + rb) * 4,
                                     umma_desc_noswizzle(ssf + ((1 + rb) * c + j) * 512, 16, 128));
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (k < nmma) {
            const uint32_t accumulate = (i > 0 || k > 0) ? 1u : 0u;
            // 32 bytes of K per MMA: advance the descriptor start address by 32 >> 4.
            const uint64_t ad = adesc + static_cast<uint64_t>(k * 2);
            const uint64_t bd = bdesc + static_cast<uint64_t>(k * 2);
            if constexpr (KIND == KIND_I8) {
              mma_i8(tmem_base, ad, bd, umma_idesc(DFMT_S32, FMT_S8, FMT_S8, 128, p.bn), accumulate);
            } else if constexpr (KIND == KIND_F8) {
              mma_f8f6f4(tmem_base, ad, bd, umma_idesc(DFMT_F32, FMT_E4M3, FMT_E4M3, 128, p.bn), accumulate);
            } else if constexpr (KIND == KIND_MXF8) {
              // four MMAs share one set of scale columns; byte k of each 32-bit column is theirs
              mma_mxf8(tmem_base, ad, bd, umma_idesc_bs(FMT_E4M3, FMT_E4M3, 128, p.bn, 1, k, k), tmem_sfa,
                       tmem_sfb, accumulate);
            } else {
              mma_nvf4(tmem_base, ad, bd, umma_idesc_bs(FMT_E2M1_MXF4, FMT_E2M1_MXF4, 128, p.bn, 0, 0, 0),
                       tmem_sfa + k * 4, tmem_sfb + k * rb_b * 4, accumulate);
            }
          }
        }
        tc_commit(smem_u32(&bar_empty[s]));  // stage reusable once these MMAs have read it
      }
      tc_commit(smem_u32(&bar_acc));  // accumulator complete
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    const bool ok = mbar_wait_bounded(smem_u32(&bar_acc), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_ACC);
    tc_fence_after();
    const int ra = row_a0 + quad * 32 + lane;  // this thread's row along the A role
    const int lim_a = p.swap ? p.n : p.m;
    const int lim_b = p.swap ? p.m : p.n;
    const bool ra_ok = ok && ra < lim_a;
    const bool direct = (p.splits == 1);
    // per-thread constants of the A-role row
    float row_scale = 1.0f, row_bias = 0.0f;
    const bool has_bias = p.bias != nullptr;
    // (the raw-accumulator variant passes no scales at all)
    if constexpr (KIND == KIND_I8) {
      if (ra_ok && p.acc_out == nullptr) row_scale = p.swap ? p.scale_wgt[ra] : p.scale_act[ra];
    }
    if (p.swap && has_bias && ra_ok && p.acc_out == nullptr) row_bias = __bfloat162float(p.bias[ra]);
    float s_act_scalar = 1.0f, s_wgt_scalar = 1.0f;
    if constexpr (KIND != KIND_I8) {
      if (p.scale_act) s_act_scalar = *p.scale_act;
      if (p.scale_wgt) s_wgt_scalar = *p.scale_wgt;
    }
    for (int c0 = 0; c0 < p.bn; c0 += 16) {
      uint32_t r[16];
      __syncwarp();  // the collective TMEM load needs the whole warp, whatever the lanes skipped above
      tmem_ld_16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c0, r);
      tc_wait_ld();
      if (!ra_ok) continue;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int rbj = row_b0 + c0 + j;  // row along the B role
        if (rbj >= lim_b) continue;
        const int om = p.swap ? rbj : ra;
        const int on = p.swap ? ra : rbj;
        if (!direct) {
          int* dst = p.partial + static_cast<long long>(om) * p.n + on;
          if constexpr (KIND == KIND_I8) {
            atomicAdd(dst, static_cast<int>(r[j]));
          } else {
            atomicAdd(reinterpret_cast<float*>(dst), __uint_as_float(r[j]));
          }
          continue;
        }
        if (p.acc_out) {
          p.acc_out[static_cast<long long>(om) * p.n + on] = static_cast<int>(r[j]);
          continue;
        }
        float sa_v, sw_v, bias_v;
        if constexpr (KIND == KIND_I8) {
          sa_v = p.swap ? p.scale_act[om] : row_scale;
          sw_v = p.swap ? row_scale : p.scale_wgt[on];
        } else {
          sa_v = s_act_scalar;
          sw_v = s_wgt_scalar;
        }
        bias_v = p.swap ? row_bias : (has_bias ? __bfloat162float(p.bias[on]) : 0.0f);
        const float v = finish_value<KIND>(r[j], sa_v, sw_v, has_bias, bias_v);
        p.out[static_cast<long long>(om) * p.ldo + on] = __float2bfloat16_rn(v);
      }
    }
  }

  // ---------------------------------------------------------------- split-K fix-up (last arriver)
  if (p.splits > 1) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned tile_id = blockIdx.y * gridDim.x + blockIdx.x;
      const unsigned prev = atomicAdd(&p.counters[tile_id], 1u);
      is_last_cta = (prev == static_cast<unsigned>(p.splits - 1)) ? 1 : 0;
      if (is_last_cta) p.counters[tile_id] = 0;  // restore for the next call
    }
    __syncthreads();
    if (is_last_cta && !abort_flag) {
      __threadfence();
      const int lim_a = p.swap ? p.n : p.m;
      const int lim_b = p.swap ? p.m : p.n;
      const bool has_bias = p.bias != nullptr;
      float s_act_scalar = 1.0f, s_wgt_scalar = 1.0f;
      if constexpr (KIND != KIND_I8) {
        if (p.scale_act) s_act_scalar = *p.scale_act;
        if (p.scale_wgt) s_wgt_scalar = *p.scale_wgt;
      }
      // Walk the tile so that consecutive threads touch consecutive output columns.
      const int span_n = p.swap ? kTileA : p.bn;   // tile extent along output columns
      const int span_m = p.swap ? p.bn : kTileA;   // tile extent along output rows
      const int m0 = p.swap ? row_b0 : row_a0;
      const int n0 = p.swap ? row_a0 : row_b0;
      const int lim_m = p.swap ? lim_b : lim_a;
      const int lim_n = p.swap ? lim_a : lim_b;
      for (int idx = threadIdx.x; idx < span_n * span_m; idx += kGemmThreads) {
        const int om = m0 + idx / span_n;
        const int on = n0 + idx % span_n;
        if (om >= lim_m || on >= lim_n) continue;
        int* src = p.partial + static_cast<long long>(om) * p.n + on;
        const uint32_t bits = static_cast<uint32_t>(__ldcg(src));
        *src = 0;  // restore for the next call
        if (p.acc_out) {
          p.acc_out[static_cast<long long>(om) * p.n + on] = static_cast<int>(bits);
          continue;
        }
        float sa_v = s_act_scalar, sw_v = s_wgt_scalar;
        if constexpr (KIND == KIND_I8) {
          sa_v = p.scale_act[om];
          sw_v = p.scale_wgt[on];
        }
        const float bias_v = has_bias ? __bfloat162float(p.bias[on]) : 0.0f;
        const float v = finish_value<KIND>(bits, sa_v, sw_v, has_bias, bias_v);
        p.out[static_cast<long long>(om) * p.ldo + on] = __float2bfloat16_rn(v);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

}  // namespace rk
