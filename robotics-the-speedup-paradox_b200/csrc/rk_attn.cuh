// Attention of a short block of fresh query tokens over a long cached key / value prefix: the
// action expert's 50 chunk tokens x 8 heads against 816 + 50 keys of one shared KV head
// (models/pi05/modeling_gemma.py:247-274, eager_attention_forward).  Non-causal, no mask.
//
// Arithmetic follows the reference's eager path step by step:
//   s = bf16(q . k) * scaling          (matmul output rounded to bf16, then the bf16 scale)
//   p = bf16( softmax_fp32(s) )        (fp32 max / exp / sum over ALL keys, probabilities to bf16)
//   o = bf16( sum_j p_j v_j )          (fp32 accumulation)
//
// Work decomposition.  The query rows of `G` heads that share a KV head form one 128-lane tile
// (row = token * G + head_in_tile, G * tokens <= 128).  The keys are cut into KS equal slices and a
// thread-block cluster of KS CTAs shares one tile, one slice each, so that 8 x 4 tiles become
// 128 CTAs.  Per CTA:
//   1. S = Q K^T for its slice with tcgen05 kind::f16 MMAs (Q and the K slice staged by TMA in the
//      128-byte swizzle), fp32 accumulators in TMEM;
//   2. softmax threads (one per row) find the slice's maximum, the KS CTAs exchange the maxima
//      through distributed shared memory, exp(score - max) is taken once per score and summed, the
//      sums are exchanged: every CTA knows the exact global max and sum;
//   3. p is written back to TMEM as packed bf16 (over the scores it replaces) and is the TMEM
//      A operand of the second MMA, O_slice = P V, against V^T tiles (keys contiguous) from TMA;
//   4. the partial outputs are parked in shared memory and summed across the cluster in rank
//      order; each CTA finishes 256 / KS of the head's columns and stores bf16 rows.
// No global scratch, no atomics, fixed summation order.  Every wait is bounded.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..9 =
// softmax / epilogue: warp w works on TMEM lanes 32 * (w % 4) .. + 31 (one thread per query row) and
// two warps share each row, taking alternate 32-column chunks.  The softmax stream is latency
// bound (long dependent chains per row), so two warps per scheduler nearly halve it.
#pragma once

#include <cuda.h>

#include "rk_gemm_tc.cuh"

namespace rk {

constexpr int kAttnThreads = 320;
constexpr int kAttnSoftmaxThreads = 256;
constexpr int kAttnDim = 256;                 // head dimension this kernel is built for
constexpr int kAttnQBytes = 128 * 128;        // one 64-element column block of the query tile
constexpr int kAttnSlotBytes = 256 * 128;     // ring slot: a K block (keys x 128 B) or a V^T block (256 x 128 B)
constexpr int kAttnSlots = 4;
constexpr int kAttnSmem = 4 * kAttnQBytes + kAttnSlots * kAttnSlotBytes + 1024;

struct AttnParams {
  int tokens, heads, kv_heads, group;  // group = query heads per tile (share one KV head)
  int kv_len;        // valid keys
  int keys;          // keys per slice (multiple of 32, <= 256)
  int splits;        // slices == cluster size
  float scaling;     // applied to the bf16-rounded scores
  __nv_bfloat16* out;  // [batch, tokens, heads, 256]
  int* status;
};

__device__ __forceinline__ float attn_round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// score as the reference's bf16 tensor ops leave it: the matmul output rounded to bf16, times the scale, rounded again
__device__ __forceinline__ float attn_score(uint32_t acc_bits, float scaling) {
  return attn_round_bf16(attn_round_bf16(__uint_as_float(acc_bits)) * scaling);
}

__device__ __forceinline__ float attn_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st_16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ float dsmem_ld_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(kAttnThreads, 1)
rk_attn_prefix_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_vt, const AttnParams p) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_q;                    // the query tile has landed
  __shared__ __align__(8) uint64_t bar_full[kAttnSlots];   // K blocks complete phase 0 of slots 0..3, V^T blocks phase 1
  __shared__ __align__(8) uint64_t bar_empty[kAttnSlots];
  __shared__ __align__(8) uint64_t bar_s_full, bar_p_full, bar_o_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int verdict[2];
  __shared__ float row_max[2][128], row_sum[2][128];  // this slice's softmax statistics per warp of a row pair, read by the peers

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const uint32_t ring_base = smem_base + 4 * kAttnQBytes;
  const int split = static_cast<int>(cluster_ctarank());
  const int tile = blockIdx.y;                      // head group
  const int b = blockIdx.z;
  const int head0 = tile * p.group;
  const int kv_head = head0 / (p.heads / p.kv_heads);
  const int key0 = split * p.keys;
  const int rows_valid = p.group * p.tokens;
  const int kblocks_v = (p.keys + 63) >> 6;         // V^T blocks of 64 keys

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_q), 1);
    for (int s = 0; s < kAttnSlots; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_s_full), 1);
    mbar_init(smem_u32(&bar_p_full), kAttnSoftmaxThreads);
    mbar_init(smem_u32(&bar_o_full), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_vt);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), 512u);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tmem_s = tmem_base;         // scores (fp32, `keys` columns), later the packed probabilities
  const uint32_t tmem_o = tmem_base + 256;   // output accumulator, 256 columns

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    const uint32_t on = elect_one();
    const uint64_t pol_keep = l2_policy_evict_last();  // Q is read by KS CTAs, K / V by every tile of the batch row
    mbar_arrive_expect_tx(smem_u32(&bar_q), static_cast<uint32_t>(4 * rows_valid * 128), on);
    for (int kb = 0; kb < 4; ++kb)
      asm volatile(
          "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %7, 0;\n\t"
          "@q cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
          " [%0], [%1, {%3, %4, %5}], [%2], %6;\n\t}"
          ::"r"(smem_base + kb * kAttnQBytes), "l"(reinterpret_cast<uint64_t>(&tm_q)), "r"(smem_u32(&bar_q)), "r"(kb * 64),
            "r"(head0), "r"(b * p.tokens), "l"(pol_keep), "r"(on)
          : "memory");
    // four K blocks (64 of the 256 dimensions each), then the V^T blocks (64 keys each) as the slots free up
    for (int i = 0; i < 4 + kblocks_v; ++i) {
      const int s = i & (kAttnSlots - 1);
      if (i >= kAttnSlots &&
          !mbar_wait_bounded(smem_u32(&bar_empty[s]), ((i / kAttnSlots) & 1) ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_EMPTY))
        break;
      const uint32_t full = smem_u32(&bar_full[s]);
      const uint32_t dst = ring_base + s * kAttnSlotBytes;
      if (i < 4) {
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(p.keys * 128), on);
        asm volatile(
            "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %7, 0;\n\t"
            "@q cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5}], [%2], %6;\n\t}"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(&tm_k)), "r"(full), "r"(i * 64), "r"(key0),
              "r"(b * p.kv_heads + kv_head), "l"(pol_keep), "r"(on)
            : "memory");
      } else {
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(kAttnSlotBytes), on);
        asm volatile(
            "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %7, 0;\n\t"
            "@q cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5}], [%2], %6;\n\t}"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(&tm_vt)), "r"(full), "r"(key0 + (i - 4) * 64), "r"(0),
              "r"(b * p.kv_heads + kv_head), "l"(pol_keep), "r"(on)
            : "memory");
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t on = elect_one();
    bool alive = mbar_wait_bounded(smem_u32(&bar_q), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL);
    tc_fence_after();
    const uint32_t idesc_s = umma_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 128, static_cast<uint32_t>(p.keys));
    const uint32_t idesc_o = umma_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 128, 256);
    // S = Q K^T: four column blocks of 64 dimensions, four MMAs (16 dimensions) each
    for (int kb = 0; kb < 4 && alive; ++kb) {
      if (!mbar_wait_bounded(smem_u32(&bar_full[kb]), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL)) {
        alive = false;
        break;
      }
      tc_fence_after();
      const uint64_t ad = umma_desc_k128(smem_base + kb * kAttnQBytes);
      const uint64_t bd = umma_desc_k128(ring_base + kb * kAttnSlotBytes);
#pragma unroll
      for (int k = 0; k < 4; ++k) mma_f16(tmem_s, ad + k * 2, bd + k * 2, idesc_s, (kb > 0 || k > 0) ? 1u : 0u, on);
      tc_commit(smem_u32(&bar_empty[kb]), on);  // the slot may take a V^T block
    }
    if (alive) tc_commit(smem_u32(&bar_s_full), on);
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");  // #1
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");  // #1b
    // O = P V: the probabilities are the TMEM A operand (two bf16 per column), V^T blocks of 64 keys
    alive = alive && mbar_wait_bounded(smem_u32(&bar_p_full), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM);
    tc_fence_after();
    const int mmas = p.keys >> 4;  // 16 keys per MMA
    for (int j = 0; j < kblocks_v && alive; ++j) {
      const int i = 4 + j, s = i & (kAttnSlots - 1);
      if (!mbar_wait_bounded(smem_u32(&bar_full[s]), (i / kAttnSlots) & 1, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL)) {
        alive = false;
        break;
      }
      tc_fence_after();
      const uint64_t bd = umma_desc_k128(ring_base + s * kAttnSlotBytes);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int kk = j * 4 + k;
        if (kk < mmas) mma_f16_ts(tmem_o, tmem_s + kk * 8, bd + k * 2, idesc_o, kk > 0 ? 1u : 0u, on);
      }
      tc_commit(smem_u32(&bar_empty[s]), on);
    }
    if (alive) tc_commit(smem_u32(&bar_o_full), on);
  } else {
    // ------------------------------------------------------------ softmax / epilogue: two threads per query row
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // which of the row's two threads: chunks half, half + 2, ...
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float log2e = 1.4426950408889634f;
    const int valid = min(p.keys, p.kv_len - key0);  // keys of this slice that exist (may be <= 0 for a trailing slice)
    bool ok = mbar_wait_group(smem_u32(&bar_s_full), 0, threadIdx.x == 64, 1, kAttnSoftmaxThreads, &abort_flag, p.status,
                              RK_DEV_TIMEOUT_ACC, verdict, 0);
    tc_fence_after();
    // pass 1: the maximum of this thread's chunks.  Rounding to bf16 and the positive scale are
    // monotonic, so the maximum of the scores is the score of the largest raw accumulator.
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for (int c0 = half * 32; c0 < p.keys; c0 += 64) {
      uint32_t a[32];
      __syncwarp();
      tmem_ld_32(tmem_s + lane_addr + c0, a);
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c0 + j < valid) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(a[j]));
    }
    const float m_raw = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
    row_max[half][r] = m_raw > -INFINITY ? attn_score(__float_as_uint(m_raw), p.scaling) : -INFINITY;
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");  // #1
    // the exact global maximum: every thread reads the 2 * KS partial maxima of its row
    float m_glob = -INFINITY;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q < p.splits) {
        uint32_t am;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(am) : "r"(smem_u32(&row_max[0][r])), "r"(q));
        m_glob = fmaxf(m_glob, fmaxf(dsmem_ld_f32(am), dsmem_ld_f32(am + 128u * 4u)));
      }
    }
    // pass 2: e = exp(score - max) once per score, summed, and written back over the score (fp32)
    const float mneg = -m_glob * log2e;
    float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int c0 = half * 32; c0 < p.keys; c0 += 64) {
      uint32_t a[32];
      __syncwarp();
      tmem_ld_32(tmem_s + lane_addr + c0, a);
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float e = 0.0f;
        if (c0 + j < valid) e = attn_ex2(fmaf(attn_score(a[j], p.scaling), log2e, mneg));
        ls[j & 3] += e;
        a[j] = __float_as_uint(e);
      }
      __syncwarp();
      tmem_st_32(tmem_s + lane_addr + c0, a);
    }
    tc_wait_st();
    row_sum[half][r] = (ls[0] + ls[1]) + (ls[2] + ls[3]);
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");  // #1b
    float l_glob = 0.0f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {  // fixed order: slice 0 (even chunks, odd chunks), slice 1, ...
      if (q < p.splits) {
        uint32_t al;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(al) : "r"(smem_u32(&row_sum[0][r])), "r"(q));
        l_glob += dsmem_ld_f32(al);
        l_glob += dsmem_ld_f32(al + 128u * 4u);
      }
    }
    const float inv_l = l_glob > 0.0f ? __fdiv_rn(1.0f, l_glob) : 0.0f;
    // pass 3: probabilities as packed bf16 over the values they replace.  Packed column j covers the
    // fp32 columns 2j, 2j + 1; chunk c lands in the first (c even) or second (c odd) half of chunk
    // c / 2, which one of the row's two threads read in this step or an earlier one: a barrier of
    // the row's two warps between the reads and the writes of a step keeps every read before the
    // write that replaces it.
    for (int c0 = half * 32; c0 < ((p.keys + 63) & ~63); c0 += 64) {
      uint32_t a[32];
      uint32_t w[16];
      const bool mine = c0 < p.keys;  // the last step may hold a chunk for one of the two warps only
      if (mine) {
        __syncwarp();
        tmem_ld_32(tmem_s + lane_addr + c0, a);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          w[j] = pack_bf16x2(__uint_as_float(a[2 * j]) * inv_l, __uint_as_float(a[2 * j + 1]) * inv_l);
      }
      tc_fence_before();
      asm volatile("bar.sync %0, 64;" ::"r"(2 + quad) : "memory");
      tc_fence_after();
      if (mine) {
        __syncwarp();
        tmem_st_16(tmem_s + lane_addr + (c0 >> 1), w);
      }
    }
    tc_wait_st();
    tc_fence_before();
    mbar_arrive(smem_u32(&bar_p_full));
    ok = mbar_wait_group(smem_u32(&bar_o_full), 0, threadIdx.x == 64, 1, kAttnSoftmaxThreads, &abort_flag, p.status,
                         RK_DEV_TIMEOUT_ACC, verdict, 1) && ok;
    tc_fence_after();
    // park this slice's partial output, column-major [256][128] fp32, over the operand buffers
    // (every MMA that read them has completed); each of the row's two threads takes 128 columns
    float* const part = reinterpret_cast<float*>(smem_gen);
    for (int c0 = half * 128; c0 < half * 128 + 128; c0 += 32) {
      uint32_t a[32];
      __syncwarp();
      tmem_ld_32(tmem_o + lane_addr + c0, a);
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) part[(c0 + j) * 128 + r] = ok ? __uint_as_float(a[j]) : 0.0f;
    }
  }
  if (warp == 0) {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");  // #1
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");  // #1b
  }

  // ---------------------------------------------------------------- sum the slices across the cluster
  __syncthreads();
  cluster_sync_all();  // #2: every CTA's partial output is in its shared memory
  if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const int per = 128 / p.splits;  // columns this thread finishes: the CTA takes 256 / splits, each of the row's two threads half
    const int c_lo = split * 2 * per + ((warp - 2) >> 2) * per;
    uint32_t peer[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      peer[q] = 0;
      if (q < p.splits) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[q]) : "r"(smem_base), "r"(q));
    }
    const int token = r / p.group, head = head0 + r % p.group;
    __nv_bfloat16* const dst =
        p.out + ((static_cast<long long>(b) * p.tokens + token) * p.heads + head) * kAttnDim + c_lo;
    for (int c8 = 0; c8 < per; c8 += 8) {
      // all loads of eight columns from every slice first (up to 64 in flight), then the sums in slice order
      float x[8][8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          x[q][u] = 0.0f;
          if (q < p.splits) x[q][u] = dsmem_ld_f32(peer[q] + static_cast<uint32_t>((c_lo + c8 + u) * 128 + r) * 4u);
        }
      }
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float t = x[0][u];
#pragma unroll
        for (int q = 1; q < 8; ++q)
          if (q < p.splits) t += x[q][u];
        v[u] = t;
      }
      if (r < rows_valid && !abort_flag)
        *reinterpret_cast<uint4*>(dst + c8) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                          pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    }
  }
  cluster_sync_all();  // #3: nobody leaves while a peer may still read its shared memory

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512u);
  }
}

}  // namespace rk
