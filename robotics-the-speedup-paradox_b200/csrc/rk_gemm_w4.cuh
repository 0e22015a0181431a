// W4A16 group-wise int4 GEMM: bf16 activations x signed-int4 weights (group 128 along K,
// bf16 group scales), fp32 accumulation, bf16 output.
//
// Packed weights stream from HBM by TMA as raw bytes through a deep ring, two K groups (128 bytes
// of every row) per copy; the weight stream is what must saturate HBM.  Everything else moves
// through ONE ring of "slots".  A slot holds what one K group needs on chip: the activation tile
// of the group in shared memory (one 3-D TMA copy, it comes from L2), the group's 128 x 128
// weight tile expanded to bf16 in TENSOR MEMORY, and a TMEM accumulator for the group's partial
// sum.  "Unpack" warps expand the raw tile to bf16 integers (exact) and store them straight into
// tensor memory with tcgen05.st (one output channel per TMEM lane, two bf16 per 32-bit column) -
// writing the four-times-larger bf16 tile to shared memory instead costs more shared-memory store
// bandwidth than the whole kernel may spend.  One thread issues tcgen05 kind::f16 MMAs whose A
// operand is that TMEM tile and whose B operand is the activation tile; the group's *unscaled*
// partial sum lands in the slot's accumulator; four epilogue warps drain it, multiply by the
// group's scale in fp32 and keep the running total in registers, then hand the whole slot back.
// The weights sit on the MMA M axis (one TMEM lane per output channel) so the group scale is a
// per-thread scalar; the group scales of the CTA's 128 channels are fetched once into shared memory.
//
// Barriers per slot: `slot_full` (unpack warps + the activation copy -> MMA thread), `acc_full`
// (MMA commit -> epilogue), `slot_empty` (epilogue -> unpack warps and producer).  The MMA thread
// is a single thread sharing its scheduler with busy unpack warps, so every instruction it issues
// is slow; it therefore waits on exactly one barrier and commits exactly once per group.
//
// Warp roles: 0 = TMA producer, 1 = TMEM owner + MMA issuer (even groups), 2 .. 2+UW-1 = unpack,
// next four = epilogue, last = MMA issuer (odd groups).
#pragma once

#include <cuda.h>

#include "rk_common.cuh"

namespace rk {

constexpr int kW4Group = 128;                // K elements per scale group == K elements per pipeline step
constexpr int kW4PairBytes = 128 * 128;      // packed weights of two K groups: 128 rows x 128 bytes
constexpr int kW4ACols = 64;                 // TMEM columns of one unpacked 128 x 128 bf16 tile (2 per column)
constexpr int kW4MaxW = 8;                   // raw-weight ring depth limit (group pairs)
constexpr int kW4MaxSlots = 6;               // slot ring depth limit

struct W4Params {
  int m, n, groups;  // activation rows, weight rows, K / 128
  int w_stages;      // raw-weight ring depth, in group pairs
  long long ldo;
  const __nv_bfloat16* bias;    // [n] or null
  __nv_bfloat16* out;           // [m, ldo]
  int* status;
};

__host__ __device__ constexpr int w4_threads(int unpack_warps) { return 32 * (2 + unpack_warps + 4 + 1); }
// TMEM budget (512 columns): every slot takes 64 columns of unpacked weights and `bn` accumulator columns.
__host__ __device__ constexpr int w4_slots(int bn) {
  return 512 / (kW4ACols + bn) < kW4MaxSlots ? 512 / (kW4ACols + bn) : kW4MaxSlots;
}

// One packed word = eight two's-complement nibbles; byte b holds weight k_b (low nibble) and
// k_{b+4} (high nibble).  Two logic ops isolate the low and the high nibbles as offset-binary bytes
// (n + 8, 0..15); one byte permute per output register then interleaves two of those bytes with
// the constant 0x43 (0x4300 | u is the bf16 value 128 + u exactly), and a packed subtract of 136
// gives the signed values.  Output register j holds the bf16 pair (k_2j, k_2j+1).
__device__ __forceinline__ uint4 w4_unpack8(uint32_t w) {
  const uint32_t lo = (w ^ 0x88888888u) & 0x0F0F0F0Fu;         // bytes: k0 k1 k2 k3 (+8)
  const uint32_t hi = ((w >> 4) ^ 0x08080808u) & 0x0F0F0F0Fu;  // bytes: k4 k5 k6 k7 (+8)
  const uint32_t c43 = 0x43434343u;
  const uint32_t c136 = 0x43084308u;  // bf16 136.0 twice
  uint32_t v[4] = {__byte_perm(lo, c43, 0x4140u), __byte_perm(lo, c43, 0x4342u), __byte_perm(hi, c43, 0x4140u),
                   __byte_perm(hi, c43, 0x4342u)};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v[j]),
                               *reinterpret_cast<const __nv_bfloat162*>(&c136));
    o[j] = *reinterpret_cast<uint32_t*>(&d);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int BN, int UW>
__global__ void __launch_bounds__(w4_threads(UW), 1)
rk_gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                     const __grid_constant__ CUtensorMap tm_s, const __grid_constant__ CUtensorMap tm_o,
                     const W4Params p) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 128, "activation tile must be 16..128 rows");
  static_assert(UW == 4 || UW == 8 || UW == 16, "four, eight or sixteen unpack warps");
  static_assert(UW / 4 <= w4_slots(BN), "every concurrently expanded group needs its own slot");
  constexpr int kXBytes = 2 * BN * 128;  // two 64-element column blocks of BN rows
  constexpr int kSlots = w4_slots(BN);
  constexpr uint32_t kTmemCols = 512;      // [0, kSlots*64): unpacked weights; then kSlots accumulators of BN columns
  constexpr uint32_t kAccBase = kSlots * kW4ACols;
  constexpr int kEpiWarp0 = 2 + UW;
  constexpr int kMmaWarpB = kEpiWarp0 + 4;  // second MMA-issuing warp

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_w_full[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_w_empty[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_slot_full[kW4MaxSlots];
  __shared__ __align__(8) uint64_t bar_slot_empty[kW4MaxSlots];
  __shared__ __align__(8) uint64_t bar_acc_full[kW4MaxSlots];
  __shared__ __align__(8) uint64_t bar_scales;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int verdict_epi[2];
  __shared__ int epi_dead;  // set by an epilogue warp that gave up, so that all four skip the store together

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

  pdl_launch_dependents();
  if (threadIdx.x == 64) {
    // first thing, by a thread that has no part in the set-up: the first raw copies and the scales
    // start their way from DRAM to L2 while the CTA sets up and the preceding kernel drains
    tma_prefetch_l2_2d(&tm_s, n0, 0);
    const int ahead = min((G + 1) >> 1, kW4MaxW);
    for (int i = 0; i < ahead; ++i) tma_prefetch_l2_2d(&tm_w, i * 128, n0);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.w_stages; ++s) {
      mbar_init(smem_u32(&bar_w_full[s]), 1);
      mbar_init(smem_u32(&bar_w_empty[s]), UW < 8 ? UW : 8);  // the warps that read a raw pair: at most two sets of four
    }
    for (int t = 0; t < kSlots; ++t) {
      mbar_init(smem_u32(&bar_slot_full[t]), 4 + 1);   // the four unpack warps of the group + the activation copy
      mbar_init(smem_u32(&bar_slot_empty[t]), 4);      // epilogue warps
      mbar_init(smem_u32(&bar_acc_full[t]), 1);
    }
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
    // ------------------------------------------------------------ TMA producer: weights run ahead of the slots
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      mbar_arrive_expect_tx(smem_u32(&bar_scales), static_cast<uint32_t>(G) * 256u);
      tma_load_2d_hint(smem_base + scales_off, &tm_s, n0, 0, smem_u32(&bar_scales), pol_w);
      const int P = (G + 1) >> 1;  // group pairs; an odd last pair reads zeros beyond K
      int gw = 0, gx = 0;
      Ring rw{0, 0}, rx{0, 0};
      uint32_t idle = 0;
      while ((gw < P || gx < G) && !*reinterpret_cast<volatile int*>(&abort_flag)) {
        bool progressed = false;
        if (gw < P) {
          const int s = rw.stage;
          if (mbar_test_wait(smem_u32(&bar_w_empty[s]), rw.phase ^ 1)) {
            const uint32_t full = smem_u32(&bar_w_full[s]);
            mbar_arrive_expect_tx(full, kW4PairBytes);
            tma_load_2d_hint(smem_base + w_off + s * kW4PairBytes, &tm_w, gw * 128, n0, full, pol_w);
            ++gw;
            rw.advance(p.w_stages);
            progressed = true;
          }
        }
        if (gx < G) {
          const int t = rx.stage;
          // nobody parks on this barrier: unpack warps and producer all probe it
          if (mbar_test_wait(smem_u32(&bar_slot_empty[t]), rx.phase ^ 1)) {
            const uint32_t full = smem_u32(&bar_slot_full[t]);
            mbar_arrive_expect_tx(full, kXBytes);
            // one copy brings both 64-element column blocks of the group: box {64, BN, 2}
            tma_load_3d_hint(smem_base + x_off + t * kXBytes, &tm_x, 0, m0, gx * 2, full, pol_x);
            ++gx;
            rx.advance(kSlots);
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (gw == P && gx < G) {
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
  } else if (warp == 1 || warp == kMmaWarpB) {
    // ------------------------------------------------------------ MMA issuers: one wait, eight MMAs, one commit per group
    // Two single threads in different warps share the issue work: one takes the even groups, the
    // other the odd ones.  Every group has its own accumulator, so their MMAs are independent; the
    // tensor pipe runs them back to back while each thread's waits, commits and loop overhead
    // (several hundred cycles per group for a lone thread) overlap with the other thread's MMAs.
    // Each issuing warp walks its loop as a whole (uniform control flow); the tcgen05 instructions
    // execute in one elected lane and every lane takes part in the barrier waits.
    {
      const uint32_t on = elect_one();
      const int parity = warp == 1 ? 0 : 1;
      const uint32_t idesc = umma_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 128, BN);
      const uint64_t desc_x0 = umma_desc_k128(smem_base + x_off);
      Ring rt{parity % kSlots, static_cast<uint32_t>(parity / kSlots)};
      // the probe of this thread's NEXT slot is issued before the group's MMAs and read one trip
      // later, so a slot that is already full costs no wait
      uint32_t ready = 0;
      for (int g = parity; g < G; g += 2) {
        const int t = rt.stage;
        if (!ready && !mbar_wait_bounded(smem_u32(&bar_slot_full[t]), rt.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM)) break;
        tc_fence_after();
        rt.stage += 2;
        while (rt.stage >= kSlots) {
          rt.stage -= kSlots;
          rt.phase ^= 1u;
        }
        ready = (g + 2 < G) ? mbar_test_wait(smem_u32(&bar_slot_full[rt.stage]), rt.phase) : 0u;
        // descriptors of the slot: the start-address field advances by bytes >> 4
        const uint64_t bd0 = desc_x0 + static_cast<uint64_t>((t * kXBytes) >> 4);
        const uint32_t a_tmem = tmem_base + t * kW4ACols;
        const uint32_t d_tmem = tmem_base + kAccBase + t * BN;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // 16 bf16 of K per MMA: 8 TMEM columns of A, 32 bytes of the activation column block
          const uint64_t bd = bd0 + static_cast<uint64_t>(((k >> 2) * (BN * 128) + (k & 3) * 32) >> 4);
          mma_f16_ts(d_tmem, a_tmem + k * 8, bd, idesc, k > 0 ? 1u : 0u, on);
        }
        tc_commit(smem_u32(&bar_acc_full[t]), on);
      }
    }
  } else if (warp < kEpiWarp0) {
    // ------------------------------------------------------------ unpack int4 -> bf16 into TMEM
    // A warp can only write the TMEM lanes of its quadrant (warp % 4), so the thread <-> row map
    // follows it: row = 32 * (warp % 4) + lane, and a thread expands its whole row of a group (64
    // raw bytes -> 64 columns).  UW == 4: every warp takes every group.  UW == 8: warps w and w + 4
    // share a quadrant and take the even and the odd group of each raw pair, so that one barrier
    // probe, one arrival and one loop trip cover 128 weights per thread.  UW == 16: four warps per
    // quadrant take groups g = 0, 1, 2, 3 (mod 4), i.e. every second raw pair each; the expansion
    // is a chain of short dependent integer operations, and four warps per scheduler instead of
    // two keep the pipes busy while a warp waits on its own results.
    constexpr int kStride = UW / 4;  // groups between two trips of one warp
    const int uw = warp - 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int h = uw >> 2;  // 0 for UW == 4
    const bool leader = (uw == 0 && lane == 0);
    // raw pair of this warp's first group, and how many pairs it moves on per trip
    constexpr int kPairStep = kStride >= 2 ? kStride / 2 : 1;
    Ring rw{(h >> 1) % p.w_stages, static_cast<uint32_t>(((h >> 1) / p.w_stages) & 1)};
    Ring rt{h, 0};  // slot of group g = h
    // Barrier probes cost a shared-memory round trip each.  The probes for the next trip are issued
    // right after this trip's loads and consumed one trip later, so their latency hides behind the
    // conversion work; only when such an early probe says "not yet" does the warp stop to poll.
    uint32_t ready = 0;
    for (int g = h; g < G; g += kStride) {
      const int sw = rw.stage;
      const int t = rt.stage;
      const int odd = g & 1;
      const bool new_pair = (kStride >= 2) || !odd;                 // this trip reads a raw pair for the first time
      const bool pair_done = (kStride >= 2) || odd || g == G - 1;   // ... and for the last time
      if (!__all_sync(0xffffffffu, ready != 0)) {
        bool ok = true;
        if (new_pair) ok = mbar_poll_lane(smem_u32(&bar_w_full[sw]), rw.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_RAW);
        ok = ok && mbar_poll_lane(smem_u32(&bar_slot_empty[t]), rt.phase ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM);
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      // The raw pair was written with the 128-byte swizzle: 16-byte chunk c of row r sits at c ^ (r & 7);
      // chunks 0..3 belong to the even group of the pair, 4..7 to the odd one.
      const uint8_t* raw = smem_gen + w_off + sw * kW4PairBytes + r * 128;
      uint4 pk[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pk[i] = *reinterpret_cast<const uint4*>(raw + (((odd * 4 + i) ^ (r & 7)) << 4));
      // next trip of this warp: its slot, and - when that trip opens a new raw pair - the pair
      Ring rt2 = rt, rw2 = rw;
      rt2.stage += kStride;
      if (rt2.stage >= kSlots) {
        rt2.stage -= kSlots;
        rt2.phase ^= 1u;
      }
      if (pair_done) {
        rw2.stage += kPairStep;
        while (rw2.stage >= p.w_stages) {
          rw2.stage -= p.w_stages;
          rw2.phase ^= 1u;
        }
      }
      ready = 0;
      if (g + kStride < G) {
        ready = mbar_test_wait(smem_u32(&bar_slot_empty[rt2.stage]), rt2.phase ^ 1);
        if (pair_done) ready &= mbar_test_wait(smem_u32(&bar_w_full[rw2.stage]), rw2.phase);
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + t * kW4ACols;
      // Convert the whole row first, then store: with the stores (ordered, volatile) out of the way
      // the compiler interleaves the sixteen independent word conversions, which hides the
      // latency of each word's short dependent chain (the warp was stalling on exactly that).
      uint32_t o[64];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t words[4] = {pk[i].x, pk[i].y, pk[i].z, pk[i].w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint4 u = w4_unpack8(words[w]);
          o[(i * 4 + w) * 4 + 0] = u.x;
          o[(i * 4 + w) * 4 + 1] = u.y;
          o[(i * 4 + w) * 4 + 2] = u.z;
          o[(i * 4 + w) * 4 + 3] = u.w;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        tmem_st_8(taddr + j * 8, o[j * 8 + 0], o[j * 8 + 1], o[j * 8 + 2], o[j * 8 + 3], o[j * 8 + 4], o[j * 8 + 5],
                  o[j * 8 + 6], o[j * 8 + 7]);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bar_slot_full[t]));                    // unpacked tile ready for the MMA thread
        if (pair_done) mbar_arrive(smem_u32(&bar_w_empty[sw]));      // raw slot reusable
      }
      rt = rt2;
      rw = rw2;
    }
  } else if (warp < kMmaWarpB) {
    // ------------------------------------------------------------ epilogue: scale each group, accumulate, store
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    const bool n_ok = n < p.n;
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.0f;
    const bool epi_leader = (warp == kEpiWarp0 && lane == 0);
    bool alive = mbar_poll_warp(smem_u32(&bar_scales), 0, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL);
    const __nv_bfloat16* my_scales = reinterpret_cast<const __nv_bfloat16*>(smem_gen + scales_off) + quad * 32 + lane;
    Ring rt{0, 0};
    for (int g = 0; g < G && alive; ++g, rt.advance(kSlots)) {
      const int t = rt.stage;
      const float sc = __bfloat162float(my_scales[g * 128]);
      // one thread parks on the barrier, the other 127 wait at a hardware barrier: a waiting epilogue
      // costs no issue slots (polling here took a third of all instructions the SM executed)
      alive = mbar_wait_group(smem_u32(&bar_acc_full[t]), rt.phase, epi_leader, 1, 128, &abort_flag, p.status,
                              RK_DEV_TIMEOUT_ACC, verdict_epi, static_cast<uint32_t>(g));
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld_16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kAccBase + t * BN + c0, r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c0 + j] = fmaf(__uint_as_float(r[j]), sc, acc[c0 + j]);
      }
      tc_fence_before();
      __syncwarp();
      // the MMAs of the group have completed (their commit was observed), so the slot's weight tile,
      // activation tile and - now drained - accumulator are all free
      if (lane == 0) mbar_arrive(smem_u32(&bar_slot_empty[t]));
    }
    // every epilogue warp reaches this rendezvous, whether it completed or gave up
    if (!alive) *reinterpret_cast<volatile int*>(&epi_dead) = 1;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*reinterpret_cast<volatile int*>(&epi_dead) == 0) {
      // The running totals hold one output channel per lane while the output is [m][n] with n
      // contiguous: transpose through shared memory (the activation tiles are free once the last
      // group's MMAs have completed) and let TMA stores write the rows, clipping ragged edges.
      const float bias = (p.bias && n_ok) ? __bfloat162float(p.bias[n]) : 0.0f;
      __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem_gen + x_off);
      const int nl = quad * 32 + lane;
#pragma unroll
      for (int j = 0; j < BN; ++j) stage[j * 128 + nl] = __float2bfloat16_rn(acc[j] + bias);
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == kEpiWarp0 && lane == 0) {
        constexpr int kBoxRows = BN < 32 ? BN : 32;
        const int rows = p.m - m0 < BN ? p.m - m0 : BN;
        for (int r0 = 0; r0 < rows; r0 += kBoxRows) tma_store_2d(&tm_o, smem_u32(stage + r0 * 128), n0, m0 + r0);
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
