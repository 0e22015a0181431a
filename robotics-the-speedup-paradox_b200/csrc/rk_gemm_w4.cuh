// W4A16 group-wise int4 GEMM: bf16 activations x signed-int4 weights (group 128 along K,
// bf16 group scales), fp32 accumulation, bf16 output.
//
// Packed weights stream from HBM by TMA as raw bytes through a deep ring (the weight stream is
// what must saturate HBM); the small activation tile of each K group rides a second, shallow ring
// (it comes from L2).  "Unpack" warps expand each 128 x 128 group tile to bf16 integers (exact) and
// store them straight into TENSOR MEMORY with tcgen05.st (one output channel per TMEM lane, two
// bf16 per 32-bit column) - writing the four-times-larger bf16 tile to shared memory instead costs
// more shared-memory store bandwidth than the whole kernel may spend.  One thread issues tcgen05
// kind::f16 MMAs whose A operand is that TMEM tile and whose B operand is the activation tile in
// shared memory; each K group's *unscaled* partial sum lands in a ring of TMEM accumulators; four
// epilogue warps drain each group's partial sum, multiply by that group's scale in fp32 and keep
// the running total in registers.  The weights sit on the MMA M axis (one TMEM lane per output
// channel) so the group scale is a per-thread scalar; the group scales of the CTA's 128 channels
// are fetched once into shared memory.
//
// Warp roles: 0 = TMA producer, 1 = TMEM owner + MMA issuer, 2 .. 2+UW-1 = unpack,
// last four = epilogue.
#pragma once

#include <cuda.h>

#include "rk_common.cuh"

namespace rk {

// Developer aid, compiled out unless RK_TRACE is defined: CTA (0,0) records SM-clock timestamps of
// each role's progress per K group into a device array that rk_trace_read() copies back.
#ifdef RK_TRACE
__device__ long long rk_trace_buf[16 * 64];
#define RK_TRACE_REC(slot, g)                                                        \
  do {                                                                               \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (g) < 64) rk_trace_buf[(slot) * 64 + (g)] = clock64(); \
  } while (0)
#else
#define RK_TRACE_REC(slot, g) do { } while (0)
#endif

constexpr int kW4Group = 128;                // K elements per scale group == K elements per pipeline step
constexpr int kW4RawBytes = 128 * 64;        // packed 128 x 128 int4 tile
constexpr int kW4ACols = 64;                 // TMEM columns of one unpacked 128 x 128 bf16 tile (2 per column)
constexpr int kW4MaxW = 16;                  // raw-weight ring depth limit
constexpr int kW4MaxX = 4;                   // activation ring depth limit
constexpr int kW4MaxXf = 4;                  // unpacked-weight ring depth limit
constexpr int kW4MaxAcc = 8;                 // TMEM accumulator ring depth limit

struct W4Params {
  int m, n, groups;  // activation rows, weight rows, K / 128
  int w_stages;      // raw-weight ring depth
  int x_stages;      // activation ring depth
  int xf_stages;     // unpacked-weight (TMEM) ring depth == activation ring depth
  long long ldo;
  const __nv_bfloat16* bias;    // [n] or null
  __nv_bfloat16* out;           // [m, ldo]
  int* status;
};

__host__ __device__ constexpr int w4_threads(int unpack_warps) { return 32 * (2 + unpack_warps + 4); }
// TMEM budget (512 columns): `xf` unpacked-weight tiles of 64 columns, the rest accumulators.
__host__ __device__ constexpr int w4_xf_depth(int bn) { return bn == 128 ? 2 : 4; }
__host__ __device__ constexpr int w4_acc_depth(int bn) {
  return (512 - w4_xf_depth(bn) * kW4ACols) / bn < kW4MaxAcc ? (512 - w4_xf_depth(bn) * kW4ACols) / bn : kW4MaxAcc;
}

// Eight two's-complement nibbles (k ascending from the low nibble) -> eight bf16 integers.
// Per pair of weights: one byte permute puts byte j of `w` (even k) in byte 0 and byte j of
// `w >> 4` (odd k) in byte 2, one logic op keeps the low nibbles and ORs in the bf16 pattern of
// 128 (0x4300 | u == 128 + u exactly), one packed subtract of 136 gives the signed value.
__device__ __forceinline__ uint4 w4_unpack8(uint32_t w) {
  w ^= 0x88888888u;  // n -> n + 8 (offset binary, 0..15)
  const uint32_t wh = w >> 4;
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t x = __byte_perm(w, wh, 0x0400u + j * 0x0101u);  // bytes: w[j], w[0], wh[j], w[0]
    const uint32_t v = (x & 0x000F000Fu) | 0x43004300u;
    const uint32_t c = 0x43084308u;  // bf16 136.0 twice
    __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v),
                               *reinterpret_cast<const __nv_bfloat162*>(&c));
    o[j] = *reinterpret_cast<uint32_t*>(&d);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int BN, int UW>
__global__ void __launch_bounds__(w4_threads(UW), 1)
rk_gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                     const __grid_constant__ CUtensorMap tm_s, const W4Params p) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 128, "activation tile must be 16..128 rows");
  static_assert(UW == 4 || UW == 8, "four or eight unpack warps");
  constexpr int kXBytes = 2 * BN * 128;  // two 64-element atoms of BN rows
  constexpr int kAcc = w4_acc_depth(BN);
  constexpr int kXf = w4_xf_depth(BN);
  constexpr int kAccCols = BN;             // TMEM columns of one accumulator slot
  constexpr uint32_t kTmemCols = 512;      // [0, kXf*64): unpacked weights; then kAcc accumulator slots
  constexpr uint32_t kAccBase = kXf * kW4ACols;
  constexpr int kEpiWarp0 = 2 + UW;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_w_full[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_w_empty[kW4MaxW];
  __shared__ __align__(8) uint64_t bar_x_full[kW4MaxX];
  __shared__ __align__(8) uint64_t bar_xf_full[kW4MaxXf];
  __shared__ __align__(8) uint64_t bar_xf_empty[kW4MaxXf];
  __shared__ __align__(8) uint64_t bar_acc_full[kW4MaxAcc];
  __shared__ __align__(8) uint64_t bar_acc_empty[kW4MaxAcc];
  __shared__ __align__(8) uint64_t bar_scales;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int verdict_unpack[2], verdict_epi[2];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  // shared memory map: [activation ring][raw ring][group scales]
  const uint32_t x_off = 0;
  const uint32_t w_off = x_off + p.x_stages * kXBytes;
  const uint32_t scales_off = w_off + p.w_stages * kW4RawBytes;
  const int n0 = blockIdx.x * 128;
  const int m0 = blockIdx.y * BN;
  const int G = p.groups;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.w_stages; ++s) {
      mbar_init(smem_u32(&bar_w_full[s]), 1);
      mbar_init(smem_u32(&bar_w_empty[s]), UW);
    }
    for (int s = 0; s < p.x_stages; ++s) {
      mbar_init(smem_u32(&bar_x_full[s]), 1);
    }
    for (int s = 0; s < p.xf_stages; ++s) {
      mbar_init(smem_u32(&bar_xf_full[s]), UW);
      mbar_init(smem_u32(&bar_xf_empty[s]), 1);
    }
    for (int b = 0; b < kAcc; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), 4);
    }
    mbar_init(smem_u32(&bar_scales), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_s);
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
  if (threadIdx.x == 0) RK_TRACE_REC(9, 0);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: two rings, weights run ahead
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      mbar_arrive_expect_tx(smem_u32(&bar_scales), static_cast<uint32_t>(G) * 256u);
      tma_load_2d_hint(smem_base + scales_off, &tm_s, n0, 0, smem_u32(&bar_scales), pol_w);
      int gw = 0, gx = 0;
      Ring rw{0, 0}, rx{0, 0};
      uint32_t idle = 0;
      while ((gw < G || gx < G) && !*reinterpret_cast<volatile int*>(&abort_flag)) {
        bool progressed = false;
        if (gw < G) {
          const int s = rw.stage;
          if (mbar_test_wait(smem_u32(&bar_w_empty[s]), rw.phase ^ 1)) {
            const uint32_t full = smem_u32(&bar_w_full[s]);
            RK_TRACE_REC(14, gw);
            mbar_arrive_expect_tx(full, kW4RawBytes);
            RK_TRACE_REC(15, gw);
            tma_load_2d_hint(smem_base + w_off + s * kW4RawBytes, &tm_w, gw * 64, n0, full, pol_w);
            RK_TRACE_REC(0, gw);
            ++gw;
            rw.advance(p.w_stages);
            progressed = true;
          }
        }
        if (gx < G) {
          const int s = rx.stage;
          // the activation ring is as deep as the unpacked ring and is released by the same commit;
          // the unpack leader parks on that barrier, so the producer only probes it
          if (mbar_test_wait(smem_u32(&bar_xf_empty[s]), rx.phase ^ 1)) {
            const uint32_t full = smem_u32(&bar_x_full[s]);
            const uint32_t xs = smem_base + x_off + s * kXBytes;
            mbar_arrive_expect_tx(full, kXBytes);
            tma_load_2d_hint(xs, &tm_x, gx * 128, m0, full, pol_x);                  // k 0..63 of the group
            tma_load_2d_hint(xs + BN * 128, &tm_x, gx * 128 + 64, m0, full, pol_x);  // k 64..127
            RK_TRACE_REC(1, gx);
            ++gx;
            rx.advance(p.x_stages);
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > kWaitSpinMax) {
          abort_flag = 1;
          atomicCAS(p.status, 0, RK_DEV_TIMEOUT_EMPTY);
        } else if (idle > 2) {
          __nanosleep(idle > kWaitSpinFast ? 256 : 32);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 128, BN);
      const uint64_t desc_x0 = umma_desc_k128(smem_base + x_off);
      Ring rx{0, 0}, rt{0, 0}, rb{0, 0};
      for (int g = 0; g < G; ++g, rx.advance(p.x_stages), rt.advance(p.xf_stages), rb.advance(kAcc)) {
        const int sx = rx.stage;
        const int t = rt.stage;
        const int b = rb.stage;
        if (!mbar_wait_bounded(smem_u32(&bar_x_full[sx]), rx.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_FULL)) break;
        if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[b]), rb.phase ^ 1, &abort_flag, p.status,
                               RK_DEV_TIMEOUT_ACC_FREE)) break;
        if (!mbar_wait_bounded(smem_u32(&bar_xf_full[t]), rt.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM)) break;
        tc_fence_after();
        RK_TRACE_REC(5, g);
        // descriptors of the stage: the start-address field advances by bytes >> 4
        const uint64_t bd0 = desc_x0 + static_cast<uint64_t>((sx * kXBytes) >> 4);
        const uint32_t a_tmem = tmem_base + t * kW4ACols;
        const uint32_t d_tmem = tmem_base + kAccBase + b * kAccCols;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // 16 bf16 of K per MMA: 8 TMEM columns of A, 32 bytes of the activation atom
          const uint64_t bd = bd0 + static_cast<uint64_t>(((k >> 2) * (BN * 128) + (k & 3) * 32) >> 4);
          mma_f16_ts(d_tmem, a_tmem + k * 8, bd, idesc, k > 0 ? 1u : 0u);
          if (k == 0) RK_TRACE_REC(10, g);
          if (k == 3) RK_TRACE_REC(11, g);
        }
        RK_TRACE_REC(12, g);
        RK_TRACE_REC(13, g);
        tc_commit(smem_u32(&bar_xf_empty[t]));  // frees the unpacked tile and the activation tile
        tc_commit(smem_u32(&bar_acc_full[b]));
        RK_TRACE_REC(6, g);
      }
    }
  } else if (warp < kEpiWarp0) {
    // ------------------------------------------------------------ unpack int4 -> bf16 into TMEM
    // A warp can only write the TMEM lanes of its quadrant (warp % 4), so the thread <-> row map
    // follows it: row = 32 * (warp % 4) + lane.  UW == 4: a thread converts its whole row of the
    // group (64 raw bytes -> 64 columns).  UW == 8: warps w and w + 4 share a quadrant and take
    // the two halves of K (32 raw bytes -> 32 columns each).
    constexpr int kHalves = UW / 4;          // threads per row
    constexpr int kRawChunks = 4 / kHalves;  // 16-byte raw chunks per thread
    const int uw = warp - 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int h = (kHalves == 2) ? (uw >> 2) : 0;
    Ring rw{0, 0}, rt{0, 0};
    for (int g = 0; g < G; ++g, rw.advance(p.w_stages), rt.advance(p.xf_stages)) {
      const int sw = rw.stage;
      const int t = rt.stage;
      // one rendezvous per group: the leader waits for the raw tile AND for the TMEM slot
      const bool leader = (uw == 0 && lane == 0);
      if (leader)
        verdict_unpack[g & 1] =
            (mbar_wait_bounded(smem_u32(&bar_w_full[sw]), rw.phase, &abort_flag, p.status, RK_DEV_TIMEOUT_RAW) &&
             mbar_wait_bounded(smem_u32(&bar_xf_empty[t]), rt.phase ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_XFORM))
                ? 1 : 0;
      asm volatile("bar.sync 2, %0;" ::"r"(UW * 32) : "memory");
      if (*reinterpret_cast<volatile int*>(&verdict_unpack[g & 1]) == 0) break;
      if (uw == 0 && lane == 0) RK_TRACE_REC(2, g);
      const uint8_t* raw = smem_gen + w_off + sw * kW4RawBytes;
      uint4 pk[kRawChunks];
#pragma unroll
      for (int i = 0; i < kRawChunks; ++i) {
        const int c4 = h * kRawChunks + i;
        // The raw tile was written with the 64-byte swizzle: 16-byte chunk c of row r sits at c ^ ((r >> 1) & 3).
        pk[i] = *reinterpret_cast<const uint4*>(raw + r * 64 + ((c4 ^ ((r >> 1) & 3)) << 4));
      }
      if (uw == 0 && lane == 0) RK_TRACE_REC(3, g);
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + t * kW4ACols + h * 32;
#pragma unroll
      for (int i = 0; i < kRawChunks; ++i) {
        // one raw chunk = 4 words = 32 weights = 16 columns, stored as two 8-column pieces as soon
        // as they are converted so that the TMEM stores overlap the remaining conversions
        const uint32_t words[4] = {pk[i].x, pk[i].y, pk[i].z, pk[i].w};
#pragma unroll
        for (int w = 0; w < 4; w += 2) {
          const uint4 u0 = w4_unpack8(words[w]);
          const uint4 u1 = w4_unpack8(words[w + 1]);
          tmem_st_8(taddr + i * 16 + w * 4, u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bar_w_empty[sw]));  // raw slot reusable
        mbar_arrive(smem_u32(&bar_xf_full[t]));   // unpacked tile ready for the MMA thread
      }
      if (uw == 0 && lane == 0) RK_TRACE_REC(4, g);
    }
  } else {
    // ------------------------------------------------------------ epilogue: scale each group, accumulate, store
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    const bool n_ok = n < p.n;
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.0f;
    const bool epi_leader = (warp == kEpiWarp0 && lane == 0);
    bool alive = mbar_wait_group(smem_u32(&bar_scales), 0, epi_leader, 1, 128, &abort_flag, p.status,
                                 RK_DEV_TIMEOUT_FULL, verdict_epi, 1u);
    const __nv_bfloat16* my_scales = reinterpret_cast<const __nv_bfloat16*>(smem_gen + scales_off) + quad * 32 + lane;
    Ring rb{0, 0};
    for (int g = 0; g < G && alive; ++g, rb.advance(kAcc)) {
      const int b = rb.stage;
      const float sc = __bfloat162float(my_scales[g * 128]);
      alive = mbar_wait_group(smem_u32(&bar_acc_full[b]), rb.phase, epi_leader, 1, 128, &abort_flag, p.status,
                              RK_DEV_TIMEOUT_ACC, verdict_epi, static_cast<uint32_t>(g));
      tc_fence_after();
      if (quad == 0 && lane == 0) RK_TRACE_REC(7, g);
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld_16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kAccBase + b * kAccCols + c0, r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c0 + j] = fmaf(__uint_as_float(r[j]), sc, acc[c0 + j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[b]));
      if (quad == 0 && lane == 0) RK_TRACE_REC(8, g);
    }
    if (alive && n_ok) {
      const float bias = p.bias ? __bfloat162float(p.bias[n]) : 0.0f;
#pragma unroll
      for (int j = 0; j < BN; ++j) {
        const int m = m0 + j;
        if (m < p.m) p.out[static_cast<long long>(m) * p.ldo + n] = __float2bfloat16_rn(acc[j] + bias);
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
