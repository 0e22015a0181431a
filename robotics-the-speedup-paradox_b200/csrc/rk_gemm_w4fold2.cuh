// W4A16 group-wise int4 GEMM, scale folded into the expanded weights, for 256 activation rows per
// tile on a PAIR of CTAs (a cluster of two SMs, `tcgen05.mma.cta_group::2`).
//
// The one-CTA kernel (rk_gemm_w4fold.cuh) streams the [256 rows x 64 K] activation tile of every
// pipeline step through its shared memory: 32 KB written by TMA and 32 KB read by the tensor core per
// step, next to the raw and expanded weights.  That is about 80 KB of shared-memory traffic for the
// 512 cycles the tensor pipe needs, and the shared-memory port (128 bytes per cycle), not the tensor
// pipe, sets the pace.  Here two CTAs share one activation tile: each loads 128 of the 256 rows
// (16 KB per step) and the MMA reads both halves across the pair, so each SM's port carries about
// 48 KB per step and the tensor pipe becomes the limit.  Each CTA still expands its own 128 output
// channels into its own tensor memory (the A operand, M = 256 across the pair) and owns the matching
// half of the accumulator rows, so the epilogue is unchanged.
//
// Protocol (all waits bounded): the raw-weight ring is private to each CTA.  A slot is "full" when
// the unpack warps of BOTH CTAs have written their expanded weights and both halves of the
// activation tile have landed; all of that is counted on the LEADER's slot_full barrier (remote
// arrivals from the peer, TMA completions of both CTAs).  The leader issues the MMAs, and
// `tcgen05.commit ... multicast::cluster` arrives on slot_empty (and at the end on acc_full) in both
// CTAs.  Every TMA load is issued by the CTA that owns the destination shared memory (no multicast).
//
// Warp roles per CTA: 0 = TMA producer, 1 = TMEM owner (+ MMA issuer in the leader), 2..9 = unpack,
// 10..13 = epilogue.
#pragma once

#include <cuda.h>

#include "rk_common.cuh"
#include "rk_gemm_tc2.cuh"
#include "rk_gemm_w4fold.cuh"

namespace rk {

constexpr int kW4f2Slots = 8;             // 8 x 32 TMEM columns of expanded weights below the accumulator
constexpr int kW4f2XBytes = 128 * 128;    // this CTA's half of a step's activation tile

// D[tmem, both CTAs] (+)= A[tmem of each CTA] * B[shared memory of both CTAs]^T
__device__ __forceinline__ void mma2_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(on)
      : "memory");
}

__global__ void __launch_bounds__(kW4fThreads, 1)
rk_gemm_w4a16_fold2_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                           const __grid_constant__ CUtensorMap tm_s, const __grid_constant__ CUtensorMap tm_o,
                           const W4Params p) {
  constexpr int UW = kW4fUnpackWarps;
  constexpr int BN = 256;  // activation rows per pair tile
  constexpr int kSlots = kW4f2Slots;
  constexpr uint32_t kTmemCols = 512;
  constexpr int kEpiWarp0 = 2 + UW;
  static_assert(kSlots * kW4fStepCols <= kW4fAccCol, "expanded-weight ring overlaps the accumulator");

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_w_full[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_w_empty[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_slot_full[kW4f2Slots];   // used in the leader only
  __shared__ __align__(8) uint64_t bar_slot_empty[kW4f2Slots];  // per CTA: the MMAs have read this slot
  __shared__ __align__(8) uint64_t bar_acc_full;                // per CTA
  __shared__ __align__(8) uint64_t bar_scales;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int epi_dead;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  // shared memory map: [this CTA's halves of the activation tiles][raw ring][group scales]
  const uint32_t x_off = 0;
  const uint32_t w_off = x_off + kSlots * kW4f2XBytes;
  const uint32_t scales_off = w_off + p.w_stages * kW4PairBytes;
  const int n0 = blockIdx.x * 128;  // this CTA's output channels
  const int m0 = blockIdx.y * BN;
  const int G = p.groups;
  const int S = 2 * G;
  // K is walked from a different start in every pair (see the one-CTA kernel); both CTAs of a pair
  // must be on the same step, so the rotation is a function of the pair index
  const int P = (G + 1) >> 1;
  const int rot_copies = (G & 1) ? 0 : static_cast<int>((blockIdx.x >> 1) % P);
  const int rot_steps = rot_copies * 4;

  pdl_launch_dependents();
  if (threadIdx.x == 64) {
    // first thing, by a thread that has no part in the set-up: the first raw copies and the scales
    // start their way from DRAM to L2 while the CTA sets up and the preceding kernel drains
    tma_prefetch_l2_2d(&tm_s, n0, 0);
    const int ahead = min(P, kW4MaxW);
    for (int i = 0, kw = rot_copies; i < ahead; ++i) {
      tma_prefetch_l2_2d(&tm_w, kw * 128, n0);
      if (++kw == P) kw = 0;
    }
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.w_stages; ++s) {
      mbar_init(smem_u32(&bar_w_full[s]), 1);
      mbar_init(smem_u32(&bar_w_empty[s]), UW);
    }
    for (int t = 0; t < kSlots; ++t) {
      // four unpack warps of the step in each CTA + the leader's announcement of the copy bytes
      mbar_init(smem_u32(&bar_slot_full[t]), UW + 1);
      mbar_init(smem_u32(&bar_slot_empty[t]), 1);  // MMA commit (multicast to both CTAs)
    }
    mbar_init(smem_u32(&bar_acc_full), 1);
    mbar_init(smem_u32(&bar_scales), 1);
    abort_flag = 0;
    epi_dead = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_s);
    tma_prefetch_desc(&tm_o);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything may signal them
  tc_fence_after();
  pdl_wait();  // from here on global memory is read and written
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      mbar_arrive_expect_tx(smem_u32(&bar_scales), static_cast<uint32_t>(G) * 256u);
      tma_load_2d_hint(smem_base + scales_off, &tm_s, n0, 0, smem_u32(&bar_scales), pol_w);
      int gw = 0, sx = 0;
      int kw = rot_copies, kx = rot_steps;
      Ring rw{0, 0}, rx{0, 0};
      uint32_t idle = 0;
      while ((gw < P || sx < S) && !*reinterpret_cast<volatile int*>(&abort_flag)) {
        bool progressed = false;
        if (gw < P) {
          const int s = rw.stage;
          if (mbar_test_wait(smem_u32(&bar_w_empty[s]), rw.phase ^ 1)) {
            const uint32_t full = smem_u32(&bar_w_full[s]);
            mbar_arrive_expect_tx(full, kW4PairBytes);
            tma_load_2d_hint(smem_base + w_off + s * kW4PairBytes, &tm_w, kw * 128, n0, full, pol_w);
            if (++kw == P) kw = 0;
            ++gw;
            rw.advance(p.w_stages);
            progressed = true;
          }
        }
        if (sx < S) {
          const int t = rx.stage;
          if (mbar_test_wait(smem_u32(&bar_slot_empty[t]), rx.phase ^ 1)) {
            // both CTAs' halves are counted on the leader's barrier; the leader announces the total
            const uint32_t full_leader = mapa_u32(smem_u32(&bar_slot_full[t]), 0);
            if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bar_slot_full[t]), 2u * kW4f2XBytes);
            tma_load_2d_pair(smem_base + x_off + t * kW4f2XBytes, &tm_x, kx * 64, m0 + static_cast<int>(rank) * 128,
                             full_leader, pol_x);
            if (++kx == S) kx = 0;
            ++sx;
            rx.advance(kSlots);
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (gw == P && sx < S) {
          // only activation copies remain: park on the slot's barrier instead of spinning
          if (!mbar_wait_bounded(smem_u32(&bar_slot_empty[rx.stage]), rx.phase ^ 1, &abort_flag, p.status,
                                 RK_DEV_TIMEOUT_EMPTY)) break;
        } else if (++idle > kWaitSpinMax) {
          abort_flag = 1;
          atomicCAS(p.status, 0, RK_DEV_TIMEOUT_EMPTY);
        } else {
          __nanosleep(idle > kWaitSpinFast ? 256 : 128);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only): four MMAs of K = 16 per step
    // the whole warp walks the loop (uniform control flow); the tcgen05 instructions execute in one elected lane
    if (rank == 0) {
      const uint32_t on = elect_one();
      const uint32_t idesc = umma_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 256, BN);
      const uint64_t desc_x0 = umma_desc_k128(smem_base + x_off);
      const uint32_t d_tmem = tmem_base + kW4fAccCol;
      Ring rt{0, 0};
      bool alive = true;
      uint32_t ready = 0;  // probe of the NEXT slot, issued before this step's MMAs and read one trip later
      for (int s = 0; s < S; ++s) {
        const int t = rt.stage;
        if (!ready && !mbar_wait_bounded(smem_u32(&bar_slot_full[t]), rt.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM)) {
          alive = false;
          break;
        }
        tc_fence_after();
        rt.advance(kSlots);
        ready = (s + 1 < S) ? mbar_test_wait(smem_u32(&bar_slot_full[rt.stage]), rt.phase) : 0u;
        const uint64_t bd0 = desc_x0 + static_cast<uint64_t>((t * kW4f2XBytes) >> 4);
        const uint32_t a_tmem = tmem_base + t * kW4fStepCols;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma2_f16_ts(d_tmem, a_tmem + k * 8, bd0 + static_cast<uint64_t>((k * 32) >> 4), idesc, (s | k) ? 1u : 0u, on);
        tc2_commit_both(smem_u32(&bar_slot_empty[t]), on);  // frees the slot in both CTAs
      }
      if (alive) tc2_commit_both(smem_u32(&bar_acc_full), on);
    }
  } else {
    if (warp < kEpiWarp0) {
      // ------------------------------------------------------------ unpack: int4 -> bf16(q * scale) into this CTA's TMEM
      // as in the one-CTA kernel; the "slot written" arrival goes to the leader's barrier
      const int uw = warp - 2;
      const int quad = warp & 3;
      const int r = quad * 32 + lane;
      const int h = uw >> 2;
      bool alive = mbar_poll_warp(smem_u32(&bar_scales), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL);
      const __nv_bfloat16* my_scales = reinterpret_cast<const __nv_bfloat16*>(smem_gen + scales_off) + r;
      Ring rw{0, 0};
      Ring rt{h % kSlots, 0};
      int kg = rot_copies * 2;
      uint32_t ready = 0;
      for (int g = 0; g < G && alive; ++g) {
        const int sw = rw.stage;
        const int t = rt.stage;
        const int odd = g & 1;
        if (!__all_sync(0xffffffffu, ready != 0)) {
          bool ok = true;
          if (!odd) ok = mbar_poll_lane(smem_u32(&bar_w_full[sw]), rw.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_RAW);
          ok = ok && mbar_poll_lane(smem_u32(&bar_slot_empty[t]), rt.phase ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM);
          if (!__all_sync(0xffffffffu, ok)) break;
        }
        const uint8_t* raw = smem_gen + w_off + sw * kW4PairBytes + r * 128;
        const int c = odd * 4 + h * 2;
        const uint4 pk0 = *reinterpret_cast<const uint4*>(raw + ((c ^ (r & 7)) << 4));
        const uint4 pk1 = *reinterpret_cast<const uint4*>(raw + (((c + 1) ^ (r & 7)) << 4));
        const __nv_bfloat162 ss = __bfloat162bfloat162(my_scales[kg * 128]);
        if (++kg == G) kg = 0;
        const bool raw_done = odd || g == G - 1;
        Ring rt2 = rt, rw2 = rw;
        rt2.stage += 2;
        if (rt2.stage >= kSlots) {
          rt2.stage -= kSlots;
          rt2.phase ^= 1u;
        }
        if (raw_done) rw2.advance(p.w_stages);
        ready = 0;
        if (g + 1 < G) {
          ready = mbar_test_wait(smem_u32(&bar_slot_empty[rt2.stage]), rt2.phase ^ 1);
          if (odd) ready &= mbar_test_wait(smem_u32(&bar_w_full[rw2.stage]), rw2.phase);
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + t * kW4fStepCols;
        const uint32_t words[8] = {pk0.x, pk0.y, pk0.z, pk0.w, pk1.x, pk1.y, pk1.z, pk1.w};
  #pragma unroll
        for (int w = 0; w < 8; w += 2) {
          uint4 u0 = w4_unpack8(words[w]);
          uint4 u1 = w4_unpack8(words[w + 1]);
          uint32_t* v0 = reinterpret_cast<uint32_t*>(&u0);
          uint32_t* v1 = reinterpret_cast<uint32_t*>(&u1);
  #pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 a = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v0[j]), ss);
            __nv_bfloat162 b = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v1[j]), ss);
            v0[j] = *reinterpret_cast<uint32_t*>(&a);
            v1[j] = *reinterpret_cast<uint32_t*>(&b);
          }
          tmem_st_8(taddr + w * 4, u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) mbar_arrive(smem_u32(&bar_slot_full[t]));
          else mbar_arrive_cluster(mapa_u32(smem_u32(&bar_slot_full[t]), 0));
          if (raw_done) mbar_arrive(smem_u32(&bar_w_empty[sw]));
        }
        rt = rt2;
        rw = rw2;
      }
    }
    // ------------------------------------------------------------ epilogue: all twelve unpack and epilogue warps
    // accumulator column j is activation row m0 + j (columns 0..127 came from the leader's half of
    // the activation tile, 128..255 from the peer's); transposed through shared memory as
    // [m][128 n] rows (the activation slots are free by now) and stored by TMA, 32 rows per store
    // The unpack warps have nothing left to do once their last group is written, and a warp may read
    // any TMEM column of its own lane quadrant: the 16-column chunks of the accumulator are dealt
    // round-robin to the three warps of each quadrant.
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // 0, 1: unpack warps; 2: epilogue warps
    const int nl = quad * 32 + lane;
    const int n = n0 + nl;
    const bool alive = mbar_poll_warp(smem_u32(&bar_acc_full), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_ACC);
    tc_fence_after();
    if (!alive) *reinterpret_cast<volatile int*>(&epi_dead) = 1;
    asm volatile("bar.sync 1, 384;" ::: "memory");
    if (*reinterpret_cast<volatile int*>(&epi_dead) == 0) {
      const float bias = (p.bias && n < p.n) ? __bfloat162float(p.bias[n]) : 0.0f;
      const int rows = p.m - m0 < BN ? p.m - m0 : BN;
      __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem_gen + x_off);
      for (int c0 = part * 16; c0 < rows; c0 += 48) {  // warp-uniform bound: tcgen05.ld is a warp-wide instruction
        uint32_t v[16];
        tmem_ld_16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kW4fAccCol + c0, v);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) stage[(c0 + j) * 128 + nl] = __float2bfloat16_rn(__uint_as_float(v[j]) + bias);
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 384;" ::: "memory");
      if (warp == kEpiWarp0 && lane == 0) {
        for (int r0 = 0; r0 < rows; r0 += 32)
          tma_store_2d(&tm_o, smem_u32(stage + r0 * 128), n0, m0 + r0);
        tma_store_commit();
        tma_store_wait_read<0>();  // the staging memory has been read; the writes drain after the CTA has left
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // no remote arrival or MMA read may target a CTA that has left
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace rk
