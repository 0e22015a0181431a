// Two-CTA tcgen05 GEMM for large activation row counts: int8 x int8 -> s32 (W8A8), e4m3 x e4m3 -> f32
// (per-tensor FP8), and the block-scaled MXFP8 / NVFP4 kinds.
//
// A pair of CTAs (a cluster of two SMs) computes one 256 x bn output tile with
// `tcgen05.mma.cta_group::2`: each CTA holds 128 of the 256 activation rows (its half of the
// accumulator lives in its own TMEM) and loads only bn/2 of the bn weight rows; the tensor cores
// of both SMs read both halves of the weight tile through the pair's shared memory.  Compared
// with two independent 128 x bn tiles this halves the weight traffic from L2 per SM and makes a
// pipeline stage 32 KB instead of 48 KB, so more stages are in flight.
//
// Every TMA load is issued by the CTA that owns the destination shared memory (no multicast);
// the loads of both CTAs signal the leader CTA's "full" barrier, the leader issues the MMAs, and
// `tcgen05.commit ... multicast::cluster` releases the stage in both CTAs.
//
// Block-scaled kinds: the scale-factor buffers are read through their own tensor maps ([chunks, 128]
// 32-bit words: one row is one 512-byte chunk of 128 rows x 4 factors), so that their copies can be
// counted on the leader's barrier like the operand tiles.  Each CTA fetches the chunks of its own 128
// activation rows and of ALL bn weight rows (every CTA's half of the accumulator spans all columns);
// the leader's `tcgen05.cp.cta_group::2` then moves each CTA's chunks into that CTA's tensor memory.
// What bounds these kinds on one CTA is the rate at which an SM takes operand bytes from L2 (about
// 64 bytes per clock): a pair halves the weight bytes per SM and MMA, which is where the speed-up
// over the one-CTA kernel comes from.
//
// Warp roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocation (+ MMA issue
// in the leader), warps 2..5 = epilogue.
#pragma once

#include <cuda.h>

#include "rk_blockscale.cuh"
#include "rk_gemm_tc.cuh"

namespace rk {

// The SwiGLU-requantising epilogue is ALU heavy and latency bound (an exponential, two IEEE
// reciprocals and five bf16 roundings per activation, in one dependent chain): it runs on sixteen
// epilogue warps (four per TMEM lane quadrant, one 16-element block of every group each) instead of
// four.  816 x 32768 x 2048: 131.7 us with four warps, 82.5 with eight.
constexpr int kGemm2SwigluSets = 4;
constexpr int kGemm2ThreadsSwiglu = 64 + 128 * kGemm2SwigluSets;

struct Gemm2Params {
  int m, n, kblocks;
  int k_valid_mmas_last;
  int bn;        // weight rows per pair tile (128, 192 or 256); each CTA loads bn / 2
  int stages;
  int out_bufs;
  int acc_bufs;  // accumulator buffers in tensor memory (2, or 1 when bn = 256 shares it with scale columns)
  int sf_kt;     // block-scaled: 512-byte scale chunks per 128-row block along K
  int sfb_blocks;  // 128-row scale blocks a weight tile touches (1 or 2)
  int issue_block; // issue a stage's tensor-core instructions as one straight-line block
  int fmt_a, fmt_b;  // KIND_MXF8: element formats (e4m3, or e2m1 for 4-bit weights expanded by TMA)
  int tx_deficit;    // bytes per stage and CTA that the copies report short of the shared-memory bytes written
  // SwiGLU-requantising epilogue (NVFP4 gate/up projection with the 64-column interleaved weight
  // layout: of every 128 output columns the first 64 are `up`, the next 64 their `gate`): when sw_q
  // is set the tile never leaves as bf16 - the epilogue forms silu(gate) * up and packs it to NVFP4.
  uint8_t* sw_q;     // [m, n / 4] bytes: two e2m1 codes per byte of the [m, n / 2] activation
  uint8_t* sw_sf;    // its UE4M3 scale factors in the swizzled 128 x 4 layout
  int sw_kt;         // 512-byte scale chunks per 128-row block of that buffer = (n / 2) / 64 (NVFP4), (n / 2) / 128 (MXFP8)
  // sw_table set: MXFP8 output instead - bf16(table[gate] * up) with the 65536-entry SiLU table, blocks of 32
  // channels, e4m3 codes [m, n / 2] bytes and UE8M0 scale bytes (the `silu_mul_pack` producer fused behind the GEMM)
  const __nv_bfloat16* sw_table;
  // sw_mode 0: NVFP4 pack of SwiGLU in bf16 steps; 1: MXFP8 pack of bf16(table[gate] * up); 2: the bf16 product
  // bf16(table[gate] * up) itself, [m, n / 2] at sw_q, and the maximum of its finite magnitudes into the word
  // sw_sf points at (atomicMax on float bits; null: not collected) - what a per-tensor-scaled packer needs next
  int sw_mode;
  int tiles_m, tiles_n;  // pair tiles: 256 x bn
  long long ldo;
  const float* scale_act;
  const float* scale_wgt;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int* status;
};

__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// load into this CTA's shared memory, completion counted on a barrier of the pair (cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, int x, int y, uint32_t bar_cluster,
                                                 uint64_t policy, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %6, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;\n\t}"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster), "r"(x), "r"(y), "l"(policy), "r"(on)
      : "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint32_t bar, uint32_t on = 1u) {
  // arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}"
      ::"r"(bar), "h"(static_cast<uint16_t>(3)), "r"(on)
      : "memory");
}
#define RK_DEFINE_MMA2(NAME, KIND)                                                                          \
  __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,     \
                                       uint32_t accumulate, uint32_t on = 1u) {                             \
    asm volatile(                                                                                           \
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"                        \
        "@q tcgen05.mma.cta_group::2.kind::" KIND " [%0], %1, %2, %3, p;\n\t}"                              \
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(on)                         \
        : "memory");                                                                                        \
  }
RK_DEFINE_MMA2(mma2_i8, "i8")
RK_DEFINE_MMA2(mma2_f8f6f4, "f8f6f4")
#undef RK_DEFINE_MMA2
__device__ __forceinline__ void mma2_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %6, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate), "r"(on)
      : "memory");
}
__device__ __forceinline__ void mma2_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %6, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate), "r"(on)
      : "memory");
}
// every CTA of the pair: 32 lanes x 128 bits of its own shared memory into its own tensor memory
__device__ __forceinline__ void tmem_cp2_32x128b_warpx4(uint32_t taddr, uint64_t sdesc, uint32_t on = 1u) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;\n\t}" ::"r"(taddr), "l"(sdesc), "r"(on) : "memory");
}

// Unpredicated forms for the straight-line issue block of the leader's elected lane.
#define RK_DEFINE_MMA2_NP(NAME, KIND)                                                                       \
  __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,     \
                                       uint32_t accumulate) {                                               \
    asm volatile(                                                                                           \
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                                  \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], %1, %2, %3, p;\n\t}"                                 \
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)                                  \
        : "memory");                                                                                        \
  }
RK_DEFINE_MMA2_NP(mma2_i8_np, "i8")
RK_DEFINE_MMA2_NP(mma2_f8f6f4_np, "f8f6f4")
#undef RK_DEFINE_MMA2_NP
__device__ __forceinline__ void mma2_mxf8_np(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma2_nvf4_np(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_cp2_32x128b_warpx4_np(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc2_commit_both_np(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

__host__ __device__ inline int gemm2_stage_bytes(int kind, int bn, int sfb_blocks) {
  const int chunks = kind == KIND_MXF8 ? 1 : (kind == KIND_NVF4 ? 4 : 0);
  return ((kTileA + bn / 2) * kStageKBytes + chunks * 512 * (1 + sfb_blocks) + 1023) / 1024 * 1024;
}

template <int KIND>
__global__ void __launch_bounds__(kGemm2ThreadsSwiglu, 1)
rk_gemm_tc2_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_sfa,
                   const __grid_constant__ CUtensorMap tm_sfb, const Gemm2Params p) {
  using T = KindTraits<KIND>;
  constexpr int kC = T::kSfChunksPerStage;  // scale chunks per stage and 128-row block
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];    // used in the leader: both CTAs' loads land
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];   // per CTA: the MMAs have read this stage
  __shared__ __align__(8) uint64_t bar_acc_full[2];         // per CTA: accumulator buffer complete
  __shared__ __align__(8) uint64_t bar_acc_empty[2];        // used in the leader: both epilogues drained it
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int verdict_epi[2];
  __shared__ unsigned sw_amax_bits;  // sw_mode 2: this CTA's maximum so far

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const int half_bn = p.bn / 2;
  const int stage_bytes = gemm2_stage_bytes(KIND, p.bn, p.sfb_blocks);
  const uint32_t sf_off = (kTileA + half_bn) * kStageKBytes;  // scale chunks of a stage: [A: kC][B: blocks x kC]
  const uint32_t out_stage_off = p.stages * stage_bytes;
  const uint32_t vec_off = out_stage_off + p.out_bufs * kOutBufBytes;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int tile_first = static_cast<int>(blockIdx.x >> 1);
  const int tile_step = static_cast<int>(gridDim.x >> 1);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), p.sw_q != nullptr ? 8 * kGemm2SwigluSets : 8);  // the epilogue warps of both CTAs of the pair
    }
    abort_flag = 0;
    sw_amax_bits = 0u;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_out);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything may signal them
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_base_slot;
  // tensor memory: accumulator buffers 256 columns apart, then the scale-factor columns
  const uint32_t tmem_sfa = tmem_base + (p.acc_bufs == 2 ? 256 + p.bn : p.bn);
  const uint32_t tmem_sfb = tmem_sfa + 16;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    // the whole warp walks the loop (uniform control flow); the copies are issued by one elected lane
    {
      const uint32_t on = elect_one();
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      Ring ring{0, 0};
      bool alive = true;
      // a barrier probe costs a shared-memory round trip: the probe of the NEXT stage is issued before
      // this stage's copies and read one trip later, so a stage that is already free costs no wait
      uint32_t ready = 0;
      for (int tile = tile_first; tile < num_tiles && alive; tile += tile_step) {
        const int row_a0 = (tile / p.tiles_n) * 256 + static_cast<int>(rank) * kTileA;
        const int row_b0 = (tile % p.tiles_n) * p.bn + static_cast<int>(rank) * half_bn;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          const int s = ring.stage;
          if (!ready && !mbar_wait_bounded(smem_u32(&bar_empty[s]), ring.phase ^ 1, &abort_flag, p.status,
                                           RK_DEV_TIMEOUT_EMPTY)) {
            alive = false;
            break;
          }
          ring.advance(p.stages);
          ready = mbar_test_wait(smem_u32(&bar_empty[ring.stage]), ring.phase ^ 1);
          // both CTAs' bytes are counted on the leader's barrier; the leader announces the total
          const uint32_t full_leader = mapa_u32(smem_u32(&bar_full[s]), 0);
          const uint32_t tx = sf_off + kC * 512 * (1 + p.sfb_blocks) - p.tx_deficit;  // per CTA; boxes count in full even when clipped
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bar_full[s]), 2u * tx, on);
          const uint32_t sa = smem_base + s * stage_bytes;
          tma_load_2d_pair(sa, &tm_a, kb * kStageKBytes, row_a0, full_leader, pol_x, on);
          tma_load_2d_pair(sa + kTileA * kStageKBytes, &tm_b, kb * kStageKBytes, row_b0, full_leader, pol_w, on);
          if constexpr (T::kBlockScaled) {
            // chunk rows of the scale maps: (128-row block) * sf_kt + (K chunk)
            const int blk_a = row_a0 >> 7;
            const int blk_b = ((tile % p.tiles_n) * p.bn) >> 7;
            tma_load_2d_pair(sa + sf_off, &tm_sfa, 0, blk_a * p.sf_kt + kb * kC, full_leader, pol_x, on);
            for (int bb = 0; bb < p.sfb_blocks; ++bb)
              tma_load_2d_pair(sa + sf_off + (1 + bb) * kC * 512, &tm_sfb, 0, (blk_b + bb) * p.sf_kt + kb * kC,
                               full_leader, pol_w, on);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    // the whole warp of the leader walks the loop; the tcgen05 instructions execute in one elected lane
    if (rank == 0) {
      const uint32_t on = elect_one();
      Ring ring{0, 0}, racc{0, 0};
      bool alive = true;
      uint32_t ready = 0;
      uint32_t idesc;
      if constexpr (KIND == KIND_I8) idesc = umma_idesc(DFMT_S32, FMT_S8, FMT_S8, 256, p.bn);
      else if constexpr (KIND == KIND_F8) idesc = umma_idesc(DFMT_F32, FMT_E4M3, FMT_E4M3, 256, p.bn);
      else if constexpr (KIND == KIND_MXF8) idesc = umma_idesc_bs(p.fmt_a, p.fmt_b, 256, p.bn, 1, 0, 0);
      else idesc = umma_idesc_bs(FMT_E2M1_MXF4, FMT_E2M1_MXF4, 256, p.bn, 0, 0, 0);
      const uint64_t adesc0 = umma_desc_k128(smem_base);
      const uint64_t bdesc0 = umma_desc_k128(smem_base + kTileA * kStageKBytes);
      const uint32_t stage_step = static_cast<uint32_t>(stage_bytes) >> 4;
      for (int tile = tile_first; tile < num_tiles && alive; tile += tile_step, racc.advance(p.acc_bufs)) {
        const int ab = racc.stage;
        if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[ab]), racc.phase ^ 1, &abort_flag, p.status,
                               RK_DEV_TIMEOUT_ACC_FREE)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * 256;
        // a weight tile that starts inside a 128-row scale block: even column offset (tiles start on multiples of 64 rows)
        const uint32_t sfb_col0 = static_cast<uint32_t>((((tile % p.tiles_n) * p.bn) & 127) >> 5);
        for (int kb = 0; kb < p.kblocks; ++kb) {
          const int s = ring.stage;
          if (!ready && !mbar_wait_bounded(smem_u32(&bar_full[s]), ring.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL)) {
            alive = false;
            break;
          }
          tc_fence_after();
          ring.advance(p.stages);  // probe the next stage now, read the answer after this stage's MMAs
          ready = mbar_test_wait(smem_u32(&bar_full[ring.stage]), ring.phase);
          const uint64_t adesc = adesc0 + static_cast<uint64_t>(s * stage_step);
          const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(s * stage_step);
          const int nmma = (kb == p.kblocks - 1) ? p.k_valid_mmas_last : 4;
          if (T::kBlockScaled && p.issue_block && nmma == 4) {
            // whole K blocks of the block-scaled kinds: the stage's up to 17 tensor-core instructions as one
            // straight-line block of the elected lane (the issuing thread's cost per instruction paces
            // these kinds; one instruction here drives both SMs, which is what makes the pair faster);
            // the kinds without scale copies measured faster in the predicated form below
            if (on) {
              const uint32_t accumulate0 = kb > 0 ? 1u : 0u;
              if constexpr (T::kBlockScaled) {
                const uint64_t sfdesc0 = umma_desc_noswizzle(smem_base + s * stage_bytes + sf_off, 16, 128);
                if (p.sfb_blocks == 1) {
#pragma unroll
                  for (int j = 0; j < kC; ++j) {
                    tmem_cp2_32x128b_warpx4_np(tmem_sfa + j * 4, sfdesc0 + static_cast<uint64_t>(j * 32));
                    tmem_cp2_32x128b_warpx4_np(tmem_sfb + j * 4, sfdesc0 + static_cast<uint64_t>((kC + j) * 32));
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < kC; ++j) {
                    tmem_cp2_32x128b_warpx4_np(tmem_sfa + j * 4, sfdesc0 + static_cast<uint64_t>(j * 32));
                    tmem_cp2_32x128b_warpx4_np(tmem_sfb + j * 8, sfdesc0 + static_cast<uint64_t>((kC + j) * 32));
                    tmem_cp2_32x128b_warpx4_np(tmem_sfb + j * 8 + 4, sfdesc0 + static_cast<uint64_t>((2 * kC + j) * 32));
                  }
                }
              }
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t accumulate = k > 0 ? 1u : accumulate0;
                if constexpr (KIND == KIND_I8) {
                  mma2_i8_np(d_tmem, adesc + k * 2, bdesc + k * 2, idesc, accumulate);
                } else if constexpr (KIND == KIND_F8) {
                  mma2_f8f6f4_np(d_tmem, adesc + k * 2, bdesc + k * 2, idesc, accumulate);
                } else if constexpr (KIND == KIND_MXF8) {
                  mma2_mxf8_np(d_tmem, adesc + k * 2, bdesc + k * 2,
                               idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29), tmem_sfa,
                               tmem_sfb + sfb_col0, accumulate);
                } else {
                  mma2_nvf4_np(d_tmem, adesc + k * 2, bdesc + k * 2, idesc, tmem_sfa + k * 4,
                               tmem_sfb + k * p.sfb_blocks * 4 + sfb_col0, accumulate);
                }
              }
              tc2_commit_both_np(smem_u32(&bar_empty[s]));
            }
            __syncwarp();
            continue;
          }
          if constexpr (T::kBlockScaled) {
            const uint32_t ssf = smem_base + s * stage_bytes + sf_off;
            const int nb = p.sfb_blocks;
            for (int j = 0; j < kC; ++j) {
              tmem_cp2_32x128b_warpx4(tmem_sfa + j * 4, umma_desc_noswizzle(ssf + j * 512, 16, 128), on);
              for (int bb = 0; bb < nb; ++bb)
                tmem_cp2_32x128b_warpx4(tmem_sfb + (j * nb + bb) * 4,
                                        umma_desc_noswizzle(ssf + ((1 + bb) * kC + j) * 512, 16, 128), on);
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (k < nmma) {
              const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
              if constexpr (KIND == KIND_I8) {
                mma2_i8(d_tmem, adesc + k * 2, bdesc + k * 2, idesc, accumulate, on);
              } else if constexpr (KIND == KIND_F8) {
                mma2_f8f6f4(d_tmem, adesc + k * 2, bdesc + k * 2, idesc, accumulate, on);
              } else if constexpr (KIND == KIND_MXF8) {
                mma2_mxf8(d_tmem, adesc + k * 2, bdesc + k * 2,
                          idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29), tmem_sfa,
                          tmem_sfb + sfb_col0, accumulate, on);
              } else {
                mma2_nvf4(d_tmem, adesc + k * 2, bdesc + k * 2, idesc, tmem_sfa + k * 4,
                          tmem_sfb + k * p.sfb_blocks * 4 + sfb_col0, accumulate, on);
              }
            }
          }
          tc2_commit_both(smem_u32(&bar_empty[s]), on);
        }
        if (alive) tc2_commit_both(smem_u32(&bar_acc_full[ab]), on);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quad = warp & 3;
    const int et = quad * 32 + lane;
    const bool has_bias = p.bias != nullptr;
    float* const vec_scale = reinterpret_cast<float*>(smem_gen + vec_off);
    float* const vec_bias = vec_scale + 256;
    float s_act_scalar = 1.0f, s_wgt_scalar = 1.0f;
    if constexpr (KIND != KIND_I8) {
      if (p.scale_act) s_act_scalar = *p.scale_act;
      if (p.scale_wgt) s_wgt_scalar = *p.scale_wgt;
    }
    const int epi_threads = static_cast<int>(blockDim.x) - 64;  // 128, or 512 with the re-packing epilogue
    const int set = (warp - 2) >> 2;                              // which of a lane quadrant's warps (re-packing epilogue)
    auto epi_sync = [](int n) { asm volatile("bar.sync 1, %0;" ::"r"(n) : "memory"); };
    const uint32_t acc_empty_leader0 = mapa_u32(smem_u32(&bar_acc_empty[0]), 0);
    const uint32_t acc_empty_leader1 = mapa_u32(smem_u32(&bar_acc_empty[1]), 0);
    Ring racc{0, 0};
    uint32_t epi_iter = 0;
    int pending_store = 0, obuf = 0;
    for (int tile = tile_first; tile < num_tiles; tile += tile_step, racc.advance(p.acc_bufs)) {
      const int ab = racc.stage;
      const int row_a0 = (tile / p.tiles_n) * 256 + static_cast<int>(rank) * kTileA;  // this CTA's 128 rows
      const int row_b0 = (tile % p.tiles_n) * p.bn;                                    // all bn columns
      const int ra = row_a0 + et;
      float row_scale = 1.0f;
      if constexpr (KIND == KIND_I8) {
        if (ra < p.m) row_scale = p.scale_act[ra];
      }
      epi_sync(epi_threads);
      for (int j = et; j < p.bn; j += 128) {
        const int rb = row_b0 + j;
        float sv = 1.0f, bv = 0.0f;
        if (rb < p.n) {
          if constexpr (KIND == KIND_I8) sv = p.scale_wgt[rb];
          if (has_bias) bv = __bfloat162float(p.bias[rb]);
        }
        vec_scale[j] = sv;
        vec_bias[j] = bv;
      }
      epi_sync(epi_threads);
      const bool ok = mbar_wait_group(smem_u32(&bar_acc_full[ab]), racc.phase, threadIdx.x == 64, 1, epi_threads, &abort_flag, p.status,
                                      RK_DEV_TIMEOUT_ACC, verdict_epi, epi_iter++);
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ab * 256 + (static_cast<uint32_t>(quad * 32) << 16);
      if (p.sw_q != nullptr) {
        // ---- SwiGLU + NVFP4 re-pack: this thread owns one activation row of the tile.  Per 128 output
        // columns: 64 `up` then 64 `gate` values -> 64 activations = four 16-element blocks = 32 code
        // bytes and 4 scale bytes (one aligned word of the swizzled layout).  The arithmetic is the
        // two-launch path's, step for step: bf16(alpha * acc), SwiGLU in bf16 steps, block pack.  Four warps
        // share a row: each takes one of the group's four blocks.
        const float alpha = s_act_scalar * s_wgt_scalar;
        const int rows_sf = (p.m + 127) & ~127;  // the scale buffer covers whole 128-row blocks; padding rows get zeros
        if (p.sw_mode == 2) {
          // ---- the activation itself as bf16 (the arithmetic of the table mode of the row quantizers) + its maximum
          __nv_bfloat16* const prod = reinterpret_cast<__nv_bfloat16*>(p.sw_q);
          float amax = 0.0f;
          for (int cc = 0; cc < p.bn; cc += 128) {
            const int col0 = row_b0 + cc;
            const int ch0 = col0 >> 1;
            const int c0 = set * 16;
            uint32_t ru[16], rg[16];
            __syncwarp();
            tmem_ld_16(t_acc + cc + c0, ru);
            tmem_ld_16(t_acc + cc + 64 + c0, rg);
            tc_wait_ld();
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              float v2[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const float up = round_bf16(__fmul_rn(alpha, __uint_as_float(ru[j + u])));
                const float gate = round_bf16(__fmul_rn(alpha, __uint_as_float(rg[j + u])));
                v2[u] = round_bf16(__fmul_rn(__bfloat162float(p.sw_table[__float_as_uint(gate) >> 16]), up));
                const float a = fabsf(v2[u]);
                if (a <= 3.4028234664e38f && ra < p.m && col0 < p.n) amax = fmaxf(amax, a);
              }
              w[j >> 1] = (__float_as_uint(v2[0]) >> 16) | (__float_as_uint(v2[1]) & 0xFFFF0000u);
            }
            if (ok && col0 < p.n && ra < p.m) {
              uint4* const dst = reinterpret_cast<uint4*>(prod + static_cast<long long>(ra) * (p.n >> 1) + ch0 + c0);
              dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
              dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(ab == 0 ? acc_empty_leader0 : acc_empty_leader1);
          if (p.sw_sf != nullptr) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0 && ok && amax > 0.0f) atomicMax(&sw_amax_bits, __float_as_uint(amax));
          }
          continue;
        }
        if (p.sw_mode == 1) {
          // ---- MXFP8 output: blocks of 32 channels = two warp sets; the sets of a pair exchange their 16 channels'
          // maximum (and whether a value was not finite) through shared memory, then each converts its own half
          float* const part_max = reinterpret_cast<float*>(smem_gen + out_stage_off);  // [4 sets][128 rows]
          uint32_t* const part_bad = reinterpret_cast<uint32_t*>(part_max + 4 * 128);    // [4 sets][128 rows]
          for (int cc = 0; cc < p.bn; cc += 128) {
            const int col0 = row_b0 + cc;
            const int ch0 = col0 >> 1;
            const int c0 = set * 16;
            uint32_t ru[16], rg[16];
            __syncwarp();
            tmem_ld_16(t_acc + cc + c0, ru);
            tmem_ld_16(t_acc + cc + 64 + c0, rg);
            tc_wait_ld();
            float v[16];
            float amax = 0.0f;
            uint32_t bad = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float up = round_bf16(__fmul_rn(alpha, __uint_as_float(ru[j])));
              const float gate = round_bf16(__fmul_rn(alpha, __uint_as_float(rg[j])));
              v[j] = round_bf16(__fmul_rn(__bfloat162float(p.sw_table[__float_as_uint(gate) >> 16]), up));
              amax = fmaxf(amax, fabsf(v[j]));
              bad |= !(fabsf(v[j]) <= 3.4028234664e38f);
            }
            part_max[set * 128 + et] = amax;
            part_bad[set * 128 + et] = bad;
            epi_sync(epi_threads);
            amax = fmaxf(amax, part_max[(set ^ 1) * 128 + et]);
            bad |= part_bad[(set ^ 1) * 128 + et];
            const uint32_t e = mxfp8_block_scale(amax, bad != 0);
            const float inverse = mxfp8_inverse_scale(e);
            uint32_t w[4];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              w[q4] = 0;
#pragma unroll
              for (int i = 0; i < 4; ++i)
                w[q4] |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fmul_rn(v[4 * q4 + i], inverse), __NV_SATFINITE, __NV_E4M3))
                         << (8 * i);
            }
            if (ok && col0 < p.n) {
              if (ra < p.m)
                *reinterpret_cast<uint4*>(p.sw_q + static_cast<long long>(ra) * (p.n >> 1) + ch0 + c0) = make_uint4(w[0], w[1], w[2], w[3]);
              if ((set & 1) == 0 && ra < rows_sf)
                p.sw_sf[sf_offset(ra, (ch0 >> 5) + (set >> 1), p.sw_kt)] = ra < p.m ? static_cast<uint8_t>(e) : static_cast<uint8_t>(0);
            }
            epi_sync(epi_threads);  // the exchange words are free again
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(ab == 0 ? acc_empty_leader0 : acc_empty_leader1);
          continue;
        }
        for (int cc = 0; cc < p.bn; cc += 128) {
          const int col0 = row_b0 + cc;       // first output column of this 128-column group
          const int ch0 = col0 >> 1;          // first activation channel of the group
          // warp set s packs block s of the group (channels 16 s .. 16 s + 15)
          const int c0 = set * 16;
          uint32_t ru[16], rg[16];
          __syncwarp();
          tmem_ld_16(t_acc + cc + c0, ru);
          tmem_ld_16(t_acc + cc + 64 + c0, rg);
          tc_wait_ld();
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float up = round_bf16(__fmul_rn(alpha, __uint_as_float(ru[j])));
            const float gate = round_bf16(__fmul_rn(alpha, __uint_as_float(rg[j])));
            v[j] = swiglu_bf16_steps(gate, up);
          }
          uint8_t code;
          const unsigned long long packed = nvfp4_block(v, &code);
          if (ok && col0 < p.n) {
            if (ra < p.m)
              *reinterpret_cast<unsigned long long*>(p.sw_q + static_cast<long long>(ra) * (p.n >> 2) + (ch0 >> 1) + set * 8) = packed;
            if (ra < rows_sf) p.sw_sf[sf_offset(ra, (ch0 >> 4) + set, p.sw_kt)] = ra < p.m ? code : static_cast<uint8_t>(0);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(ab == 0 ? acc_empty_leader0 : acc_empty_leader1);
        continue;
      }
      for (int cc = 0; cc < p.bn; cc += 64, obuf = (p.out_bufs == 2) ? (obuf ^ 1) : 0) {
        uint8_t* const stage = smem_gen + out_stage_off + obuf * kOutBufBytes;
        if (et == 0 && pending_store) {
          if (p.out_bufs == 2) tma_store_wait_read<1>();
          else tma_store_wait_read<0>();
        }
        epi_bar_sync();
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld_16(t_acc + cc + c0, r);
          tc_wait_ld();
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if constexpr (KIND == KIND_I8)
              v[j] = finish_value<KIND>(r[j], row_scale, vec_scale[cc + c0 + j], has_bias, vec_bias[cc + c0 + j]);
            else
              v[j] = finish_value<KIND>(r[j], s_act_scalar, s_wgt_scalar, has_bias, vec_bias[cc + c0 + j]);
          }
          const uint4 lo = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                      pack_bf16x2(v[6], v[7]));
          const uint4 hi = make_uint4(pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]), pack_bf16x2(v[12], v[13]),
                                      pack_bf16x2(v[14], v[15]));
          const int ch = c0 >> 3;
          *reinterpret_cast<uint4*>(stage + et * 128 + ((ch ^ (et & 7)) << 4)) = lo;
          *reinterpret_cast<uint4*>(stage + et * 128 + (((ch + 1) ^ (et & 7)) << 4)) = hi;
        }
        if (cc + 64 >= p.bn) {
          // accumulator drained: tell the leader's MMA thread (its barrier counts both CTAs' warps)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(ab == 0 ? acc_empty_leader0 : acc_empty_leader1);
        }
        fence_proxy_async_smem();
        epi_bar_sync();
        if (et == 0) {
          if (ok) tma_store_2d(&tm_out, smem_u32(stage), row_b0 + cc, row_a0);
          tma_store_commit();
          pending_store = 1;
        }
      }
    }
    if (et == 0) tma_store_wait_read<0>();  // the staging memory has been read; the writes drain after the CTA has left
    if (p.sw_mode == 2 && p.sw_sf != nullptr) {
      epi_sync(epi_threads);  // every warp has added its maximum
      if (threadIdx.x == 64 && sw_amax_bits != 0u) atomicMax(reinterpret_cast<unsigned*>(p.sw_sf), sw_amax_bits);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still be reading this CTA's shared memory through its MMAs
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace rk
