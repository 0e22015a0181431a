// W4A16 group-wise int4 GEMM for activation batches above 64 rows: the group scale is folded into
// the weights while they are expanded, so that ONE accumulator serves all of K.
//
// rk_gemm_w4.cuh keeps every K group's partial sum apart and applies the group scale in fp32; that
// costs a TMEM accumulator and an epilogue pass per group, which stops paying once the activation
// tile is wide (the accumulators alone would fill tensor memory, and the weight tile would have to
// be expanded once per 128 activation rows).  Here an unpack thread multiplies each expanded weight
// by its group scale in bf16 - bf16(q * s), one rounding of at most 2^-9 relative, the same
// "dequantize to bf16, then multiply" the reference's mixed-input GEMM performs
// (blackwell/csrc/fp4_mixed_cutlass_linear.cu:190-260) - so a CTA expands each weight tile ONCE for
// up to 256 activation rows (MMA N = 256) and the tensor pipe, not the expansion, bounds the loop.
//
// Pipeline step = 64 elements of K (half a scale group).  A ring of slots holds, per step, the
// activation tile [BN rows x 128 bytes] in shared memory and the expanded weights (128 lanes x 32
// TMEM columns).  Raw packed weights arrive through their own ring, 256 elements of K (four steps)
// of 128 channels per copy.  slot_full: unpack warps + activation copy -> MMA thread; slot_empty:
// MMA commit -> unpack warps and producer.  All multi-warp waits poll with the non-blocking probe.
//
// Warp roles: 0 = TMA producer, 1 = TMEM owner + MMA issuer, 2..9 = unpack, 10..13 = epilogue.
#pragma once

#include <cuda.h>

#include "rk_common.cuh"
#include "rk_gemm_w4.cuh"

namespace rk {

constexpr int kW4fUnpackWarps = 8;
constexpr int kW4fThreads = 32 * (2 + kW4fUnpackWarps + 4);
constexpr int kW4fStepCols = 32;  // TMEM columns of one expanded step: 64 bf16 of K per lane
constexpr int kW4fAccCol = 256;   // the accumulator occupies TMEM columns [256, 256 + BN)
constexpr int kW4fMaxSlots = 8;

__host__ __device__ constexpr int w4f_slots(int bn) { return bn > 128 ? 5 : 8; }

template <int BN>
__global__ void __launch_bounds__(kW4fThreads, 1)
rk_gemm_w4a16_fold_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                          const __grid_constant__ CUtensorMap tm_s, const __grid_constant__ CUtensorMap tm_o,
                          const W4Params p) {
  static_assert(BN == 128 || BN == 256, "activation tile of 128 or 256 rows");
  constexpr int UW = kW4fUnpackWarps;
  constexpr int kXBytes = BN * 128;  // one 64-element column block of BN rows
  constexpr int kSlots = w4f_slots(BN);
  constexpr uint32_t kTmemCols = 512;
  constexpr int kEpiWarp0 = 2 + UW;
  static_assert(kSlots * kW4fStepCols <= kW4fAccCol, "expanded-weight ring overlaps the accumulator");

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_w_full[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_w_empty[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_slot_full[kW4fMaxSlots];
  __shared__ __align__(8) uint64_t bar_slot_empty[kW4fMaxSlots];
  __shared__ __align__(8) uint64_t bar_acc_full;
  __shared__ __align__(8) uint64_t bar_scales;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int epi_dead;  // set by a warp that gave up on the accumulator, so that all skip the store together

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  // shared memory map: [activation tiles of the slots][raw ring][group scales]
  const uint32_t x_off = 0;
  const uint32_t w_off = x_off + kSlots * kXBytes;
  const uint32_t scales_off = w_off + p.w_stages * kW4PairBytes;
  const int n0 = blockIdx.x * 128;
  const int m0 = blockIdx.y * BN;
  const int G = p.groups;
  const int S = 2 * G;  // steps of 64 K elements
  // Every CTA of a launch reads the SAME activation tiles.  Walking K from a different start in
  // each CTA (a rotation by whole raw copies) spreads those reads over different L2 lines at any
  // moment instead of having all CTAs hit one tile together.  Summation order then differs between
  // CTAs but is fixed for a given CTA, so results stay deterministic.
  const int P = (G + 1) >> 1;  // raw copies of two groups; an odd last one reads zeros beyond K
  const int rot_copies = (G & 1) ? 0 : static_cast<int>(blockIdx.x % P);
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
      mbar_init(smem_u32(&bar_slot_full[t]), UW / 2 + 1);  // the four unpack warps of the step + the activation copy
      mbar_init(smem_u32(&bar_slot_empty[t]), 1);      // MMA commit
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
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // from here on global memory is read and written
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      mbar_arrive_expect_tx(smem_u32(&bar_scales), static_cast<uint32_t>(G) * 256u);
      tma_load_2d_hint(smem_base + scales_off, &tm_s, n0, 0, smem_u32(&bar_scales), pol_w);
      int gw = 0, sx = 0;
      int kw = rot_copies, kx = rot_steps;  // rotated positions along K
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
            const uint32_t full = smem_u32(&bar_slot_full[t]);
            mbar_arrive_expect_tx(full, kXBytes);
            tma_load_2d_hint(smem_base + x_off + t * kXBytes, &tm_x, kx * 64, m0, full, pol_x);
            if (++kx == S) kx = 0;
            ++sx;
            rx.advance(kSlots);
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (gw == P && sx < S) {
          // only activation copies remain: park on the slot's barrier instead of spinning, so that
          // this thread stops taking issue slots from the unpack warps of its scheduler
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
    // ------------------------------------------------------------ MMA issuer: four MMAs of K = 16 per step
    // the whole warp walks the loop (uniform control flow); the tcgen05 instructions execute in one elected lane
    {
      const uint32_t on = elect_one();
      const uint32_t idesc = umma_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 128, BN);
      const uint64_t desc_x0 = umma_desc_k128(smem_base + x_off);
      const uint32_t d_tmem = tmem_base + kW4fAccCol;
      Ring rt{0, 0};
      bool alive = true;
      // The thread's own instructions, not the tensor pipe, set the pace of this loop unless it stays
      // under the 4 x 128 cycles the pipe needs per step: the probe of the NEXT slot is issued before
      // this step's MMAs and read one trip later, so a slot that is already full costs no wait.
      uint32_t ready = 0;
      for (int s = 0; s < S; ++s) {
        const int t = rt.stage;
        if (!ready && !mbar_wait_bounded(smem_u32(&bar_slot_full[t]), rt.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM)) {
          alive = false;
          break;
        }
        tc_fence_after();
        rt.advance(kSlots);
        ready = (s + 1 < S) ? mbar_test_wait(smem_u32(&bar_slot_full[rt.stage]), rt.phase) : 0u;
        const uint64_t bd0 = desc_x0 + static_cast<uint64_t>((t * kXBytes) >> 4);
        const uint32_t a_tmem = tmem_base + t * kW4fStepCols;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_f16_ts(d_tmem, a_tmem + k * 8, bd0 + static_cast<uint64_t>((k * 32) >> 4), idesc, (s | k) ? 1u : 0u, on);
        tc_commit(smem_u32(&bar_slot_empty[t]), on);  // frees the expanded weights and the activation tile
      }
      if (alive) tc_commit(smem_u32(&bar_acc_full), on);
    }
  } else {
    if (warp < kEpiWarp0) {
      // ------------------------------------------------------------ unpack: int4 -> bf16(q * scale) into TMEM
      // row = 32 * (warp % 4) + lane (a warp writes only the TMEM lanes of its quadrant).  One loop
      // trip covers a scale group, i.e. two steps: warps 0..3 expand the group's first step, warps
      // 4..7 its second, each into its own slot - 64 weights per thread and one barrier probe, one
      // arrival and one scale fetch per trip.
      const int uw = warp - 2;
      const int quad = warp & 3;
      const int r = quad * 32 + lane;
      const int h = uw >> 2;
      bool alive = mbar_poll_warp(smem_u32(&bar_scales), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL);
      const __nv_bfloat16* my_scales = reinterpret_cast<const __nv_bfloat16*>(smem_gen + scales_off) + r;
      Ring rw{0, 0};
      Ring rt{h % kSlots, 0};  // slot of step 2 g + h
      int kg = rot_copies * 2;  // rotated group index along K
      // the barrier probes for the next trip are issued right after this trip's loads and consumed one
      // trip later (their latency hides behind the conversion); a warp stops to poll only on "not yet"
      uint32_t ready = 0;
      for (int g = 0; g < G && alive; ++g) {
        const int sw = rw.stage;
        const int t = rt.stage;
        const int odd = g & 1;  // second group of the raw copy
        if (!__all_sync(0xffffffffu, ready != 0)) {
          bool ok = true;
          if (!odd) ok = mbar_poll_lane(smem_u32(&bar_w_full[sw]), rw.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_RAW);
          ok = ok && mbar_poll_lane(smem_u32(&bar_slot_empty[t]), rt.phase ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM);
          if (!__all_sync(0xffffffffu, ok)) break;
        }
        // 128-byte swizzle of the raw copy: 16-byte chunk c of row r sits at c ^ (r & 7); the step of
        // this warp owns chunks 4 * odd + 2 * h and the next one
        const uint8_t* raw = smem_gen + w_off + sw * kW4PairBytes + r * 128;
        const int c = odd * 4 + h * 2;
        const uint4 pk0 = *reinterpret_cast<const uint4*>(raw + ((c ^ (r & 7)) << 4));
        const uint4 pk1 = *reinterpret_cast<const uint4*>(raw + (((c + 1) ^ (r & 7)) << 4));
        const __nv_bfloat162 ss = __bfloat162bfloat162(my_scales[kg * 128]);
        if (++kg == G) kg = 0;
        const bool raw_done = odd || g == G - 1;
        // next trip: this warp's slot two steps on, and - when it opens a new raw copy - that copy
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
          mbar_arrive(smem_u32(&bar_slot_full[t]));
          if (raw_done) mbar_arrive(smem_u32(&bar_w_empty[sw]));
        }
        rt = rt2;
        rw = rw2;
      }
    }
    // ------------------------------------------------------------ epilogue: all twelve unpack and epilogue warps
    // The accumulator holds one output channel per lane; the output is [m][n] with n contiguous.
    // Storing it straight from registers would be one 2-byte store per element.  Instead the tile
    // is transposed through shared memory (the activation slots are free by now) as [m][128 n]
    // rows and leaves by TMA stores of 32 rows each, which also clip the ragged edges.
    // The unpack warps have nothing left to do once their last group is written, and a warp may read
    // any TMEM column of its own lane quadrant: the 16-column chunks of the accumulator are dealt
    // round-robin to the three warps of each quadrant.
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // 0, 1: unpack warps; 2: epilogue warps
    const int nl = quad * 32 + lane;
    const int n = n0 + nl;
    const bool alive = mbar_poll_warp(smem_u32(&bar_acc_full), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_ACC);
    tc_fence_after();
    // every one of the twelve warps reaches this rendezvous, whether it saw the accumulator complete or gave up
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
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace rk
