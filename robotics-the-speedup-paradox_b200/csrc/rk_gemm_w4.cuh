// W4A16 group-wise int4 GEMM: bf16 activations x signed-int4 weights (group 128 along K,
// bf16 group scales), fp32 accumulation, bf16 output.
//
// Packed weights stream from HBM by TMA as raw bytes; four "unpack" warps expand each 128 x 128
// group tile to bf16 integers (exact) in the 128-byte-swizzled UMMA layout in shared memory; one
// thread issues tcgen05 kind::f16 MMAs that produce the *unscaled* partial sum of one K group in a
// double-buffered TMEM accumulator; four epilogue warps drain each group's partial sum, multiply
// by that group's scale in fp32 and keep the running total in registers.  The weights sit on the
// MMA M axis (one TMEM lane per output channel) so the group scale is a per-thread scalar.
//
// Warp roles (320 threads): 0 = TMA producer, 1 = TMEM owner + MMA issuer, 2..5 = unpack,
// 6..9 = epilogue.
#pragma once

#include <cuda.h>

#include "rk_common.cuh"

namespace rk {

constexpr int kW4Threads = 320;
constexpr int kW4Group = 128;       // K elements per scale group == K elements per pipeline step
constexpr int kW4RawBytes = 128 * 64;        // packed 128 x 128 int4 tile
constexpr int kW4AtomBytes = 128 * 128;      // one 128-row x 64-element bf16 swizzle atom
constexpr int kW4XfBytes = 2 * kW4AtomBytes; // unpacked 128 x 128 bf16 tile
constexpr int kW4MaxStages = 8;
constexpr int kW4MaxXf = 4;

struct W4Params {
  int m, n, groups;  // activation rows, weight rows, K / 128
  int stages;        // TMA ring depth (raw weights + activations)
  int xf_stages;     // unpacked-weight ring depth
  long long ldo;
  const __nv_bfloat16* scales;  // [groups, n]
  const __nv_bfloat16* bias;    // [n] or null
  __nv_bfloat16* out;           // [m, ldo]
  int* status;
};

// Eight two's-complement nibbles (k ascending from the low nibble) -> eight bf16 integers.
__device__ __forceinline__ uint4 w4_unpack8(uint32_t w) {
  w ^= 0x88888888u;  // n -> n + 8 (offset binary, 0..15)
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t t = w >> (8 * j);
    // bf16 0x4300 | u == 128 + u exactly; subtracting 136 gives n.
    const uint32_t v = (t & 0x0000000Fu) | ((t << 12) & 0x000F0000u) | 0x43004300u;
    const uint32_t c = 0x43084308u;
    __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v),
                               *reinterpret_cast<const __nv_bfloat162*>(&c));
    o[j] = *reinterpret_cast<uint32_t*>(&d);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int BN>
__global__ void __launch_bounds__(kW4Threads, 1)
rk_gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                     const W4Params p) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 128, "activation tile must be 16..128 rows");
  constexpr int kXBytes = 2 * BN * 128;              // two 64-element atoms of BN rows
  constexpr int kStageBytes = kW4RawBytes + kXBytes;  // multiple of 1024
  constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : 256));

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kW4MaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kW4MaxStages];
  __shared__ __align__(8) uint64_t bar_xf_full[kW4MaxXf];
  __shared__ __align__(8) uint64_t bar_xf_empty[kW4MaxXf];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t xf_base = smem_base + p.stages * kStageBytes;
  const int n0 = blockIdx.x * 128;
  const int m0 = blockIdx.y * BN;
  const int G = p.groups;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < p.xf_stages; ++s) {
      mbar_init(smem_u32(&bar_xf_full[s]), 128);
      mbar_init(smem_u32(&bar_xf_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), 128);
    }
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      for (int g = 0; g < G; ++g) {
        const int s = g % p.stages;
        const uint32_t ph = (g / p.stages) & 1;
        if (!mbar_wait_bounded(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, RK_DEV_TIMEOUT_EMPTY)) break;
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t raw = smem_base + s * kStageBytes;
        const uint32_t xs = raw + kW4RawBytes;
        mbar_arrive_expect_tx(full, kStageBytes);
        tma_load_2d_hint(raw, &tm_w, g * 64, n0, full, pol_w);                    // 64 packed bytes x 128 rows
        tma_load_2d_hint(xs, &tm_x, g * 128, m0, full, pol_x);                    // k 0..63 of the group
        tma_load_2d_hint(xs + BN * 128, &tm_x, g * 128 + 64, m0, full, pol_x);    // k 64..127
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 128, BN);
      for (int g = 0; g < G; ++g) {
        const int s = g % p.stages;
        const int t = g % p.xf_stages;
        const int b = g & 1;
        if (!mbar_wait_bounded(smem_u32(&bar_full[s]), (g / p.stages) & 1, &abort_flag, p.status,
                               RK_DEV_TIMEOUT_FULL)) break;
        if (!mbar_wait_bounded(smem_u32(&bar_xf_full[t]), (g / p.xf_stages) & 1, &abort_flag, p.status,
                               RK_DEV_TIMEOUT_XFORM)) break;
        if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[b]), ((g >> 1) & 1) ^ 1, &abort_flag, p.status,
                               RK_DEV_TIMEOUT_ACC_FREE)) break;
        tc_fence_after();
        const uint32_t xs = smem_base + s * kStageBytes + kW4RawBytes;
        const uint32_t ws = xf_base + t * kW4XfBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // 16 bf16 (32 bytes) of K per MMA; four MMAs per 64-element atom.
          const uint64_t ad = umma_desc_k128(ws + (k >> 2) * kW4AtomBytes) + static_cast<uint64_t>((k & 3) * 2);
          const uint64_t bd = umma_desc_k128(xs + (k >> 2) * (BN * 128)) + static_cast<uint64_t>((k & 3) * 2);
          mma_f16(tmem_base + b * BN, ad, bd, idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_empty[s]));
        tc_commit(smem_u32(&bar_xf_empty[t]));
        tc_commit(smem_u32(&bar_acc_full[b]));
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ unpack int4 -> bf16 (one weight row per thread)
    const int r = threadIdx.x - 64;  // 0..127
    for (int g = 0; g < G; ++g) {
      const int s = g % p.stages;
      const int t = g % p.xf_stages;
      if (!mbar_wait_bounded(smem_u32(&bar_full[s]), (g / p.stages) & 1, &abort_flag, p.status,
                             RK_DEV_TIMEOUT_RAW)) break;
      if (!mbar_wait_bounded(smem_u32(&bar_xf_empty[t]), ((g / p.xf_stages) & 1) ^ 1, &abort_flag, p.status,
                             RK_DEV_TIMEOUT_XFORM)) break;
      const uint8_t* raw = smem_dyn + (smem_base - smem_u32(smem_dyn)) + s * kStageBytes;
      uint8_t* dst = smem_dyn + (xf_base - smem_u32(smem_dyn)) + t * kW4XfBytes;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        // The raw tile was written with the 64-byte swizzle: 16-byte chunk c of row r sits at c ^ ((r >> 1) & 3).
        const uint4 pk = *reinterpret_cast<const uint4*>(raw + r * 64 + ((c4 ^ ((r >> 1) & 3)) << 4));
        const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const int c = c4 * 4 + w;  // 16-byte bf16 chunk index along K (8 weights), 0..15
          const int atom = c >> 3;
          const int cc = c & 7;
          // 128-byte swizzle: chunk cc of row r sits at cc ^ (r & 7).
          *reinterpret_cast<uint4*>(dst + atom * kW4AtomBytes + r * 128 + ((cc ^ (r & 7)) << 4)) =
              w4_unpack8(words[w]);
        }
      }
      fence_proxy_async_smem();  // make these generic-proxy writes visible to the tensor core
      mbar_arrive(smem_u32(&bar_xf_full[t]));
    }
  } else {
    // ------------------------------------------------------------ epilogue: scale each group, accumulate, store
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    const bool n_ok = n < p.n;
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.0f;
    bool alive = true;
    for (int g = 0; g < G && alive; ++g) {
      const int b = g & 1;
      const float sc = n_ok ? __bfloat162float(p.scales[static_cast<long long>(g) * p.n + n]) : 0.0f;
      alive = mbar_wait_bounded(smem_u32(&bar_acc_full[b]), (g >> 1) & 1, &abort_flag, p.status, RK_DEV_TIMEOUT_ACC);
      __syncwarp();
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld_16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + b * BN + c0, r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c0 + j] = fmaf(__uint_as_float(r[j]), sc, acc[c0 + j]);
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bar_acc_empty[b]));
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
