// W4A16 group-wise int4 GEMV: ONE activation row (decode batch 1).
//
// With a single activation row the tensor pipe is the wrong tool: a `tcgen05.mma` of K = 16 costs
// 64 cycles whatever N <= 128 is, which puts a floor of 4.3 us per CTA under the kernels of
// rk_gemm_w4.cuh at K = 2048, above the 2.65 us the packed weights need to arrive from HBM.  One
// row is 2 flops per weight - byte-streaming work - so this kernel does it on the CUDA cores and is
// bound by the weight stream.
//
// K is cut into slabs of 1024; a warp owns eight consecutive output channels and one slab at a time:
// lane l holds the 32 activations of the slab's chunk l in registers (fp32) and, per channel, loads
// the matching 16-byte piece of the packed row - the eight loads are issued before the first is
// used.  The warps of a CTA that share a row batch take different slabs (so that all their loads are
// in flight together) and combine their partial sums through shared memory.
//
// Arithmetic per weight: the offset-binary nibble u = q + 8, isolated in its own byte with bit 7
// set, is placed by one byte-permute under the exponent byte 0x3F: the float 1 + u / 128, exactly;
// acc += x * f.  Per chunk the identity
//   sum x * q = 128 * acc - 136 * sum x
// recovers the group's partial sum (11 integer operations per eight weights and one FMA per
// weight; no int -> float conversion, which runs at an eighth of the FMA rate).  The partial sums are
// scaled by their bf16 group scale in fp32, reduced over the warp by shuffles and over the slabs in
// shared memory; eight bf16 outputs leave in one store.  Summation is fp32 throughout (a different
// order than the tensor-core kernels; same tolerance).
//
// The kernel is issue bound, not latency bound: a variant that streamed the packed rows through
// per-team shared-memory rings with bulk copies (192 KB of weights in flight per SM instead of
// 64 KB at best) measured 9.0 us against 8.2 us for this form at N = 16384, K = 2048.
//
// Packed word format as everywhere: byte b of a word holds weights k_b (low nibble) and k_{b+4}.
#pragma once

#include <cuda_bf16.h>

#include "rk_common.cuh"

namespace rk {

constexpr int kGemvSlab = 1024;   // K elements per pass: 32 chunks of 32, one per lane
constexpr int kGemvRows = 8;      // output channels per warp
constexpr int kGemvWarps = 8;

struct GemvParams {
  const uint8_t* q;              // [n, k / 2]
  const __nv_bfloat16* scales;   // [k / 128, n]
  const __nv_bfloat16* x;        // [k]
  const __nv_bfloat16* bias;     // [n] or null
  __nv_bfloat16* out;            // [n]
  int n, k;
};

// sum over the 32 weights of one 16-byte piece of x[e] * (1 + u / 128).  xs2[4 * j + b] holds the
// chunk's activations (8 j + b, 8 j + 4 + b): the two weights that share byte b of word j.  One packed
// `fma.rn.f32x2` advances both running sums (the same two chains, rounded identically, as two FMAs).
__device__ __forceinline__ float gemv_chunk(const uint4& piece, const float2 (&xs2)[16]) {
  const uint32_t words[4] = {piece.x, piece.y, piece.z, piece.w};
  float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // bytes of `lo`: 0x80 | (k_b + 8) for weights k_0..k_3 of the word, of `hi`: k_4..k_7
    // (one logic op each: inside the mask the xor flips the sign bit of the nibble, outside it sets bit 7)
    const uint32_t lo = (words[j] & 0x0F0F0F0Fu) ^ 0x88888888u;
    const uint32_t hi = ((words[j] >> 4) & 0x0F0F0F0Fu) ^ 0x88888888u;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      // result bytes (low to high): 0, 0, byte b of the source, 0x3F
      const float f_lo = __uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7044u | (b << 8)));
      const float f_hi = __uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7044u | (b << 8)));
      acc = __ffma2_rn(xs2[4 * j + b], make_float2(f_lo, f_hi), acc);
    }
  }
  return acc.x + acc.y;
}

__global__ void __launch_bounds__(kGemvWarps * 32, 2)
rk_gemv_w4a16_kernel(const GemvParams p) {
  __shared__ float partial[kGemvWarps][kGemvRows];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int slabs = p.k / kGemvSlab;
  const int share = slabs < kGemvWarps ? slabs : kGemvWarps;  // warps of this CTA per row batch (1, 2, 4 or 8)
  const int batches_per_cta = kGemvWarps / share;
  const int batch = blockIdx.x * batches_per_cta + warp / share;
  const int first_slab = warp % share;
  const int n0 = batch * kGemvRows;
  const bool active = n0 < p.n;  // n is a multiple of 8: a batch's eight channels exist or none does
  pdl_launch_dependents();
  pdl_wait();  // the activations (and, in tests, freshly packed weights) come from the preceding kernel
  const int row_bytes = p.k >> 1;
  float total[kGemvRows];
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r) total[r] = 0.0f;
  for (int slab = first_slab; active && slab < slabs; slab += share) {
    const int k0 = slab * kGemvSlab;
    // the weight pieces of all eight channels first, streaming (read once)
    uint4 piece[kGemvRows];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      const uint8_t* row = p.q + static_cast<long long>(n0 + r) * row_bytes + (k0 >> 1);
      piece[r] = __ldcs(reinterpret_cast<const uint4*>(row + lane * 16));
    }
    // this lane's chunk of the slab: activations to registers (paired as gemv_chunk wants them), and their plain sum
    float2 xs2[16];
    float xsum = 0.0f;
    {
      const uint4* src = reinterpret_cast<const uint4*>(p.x + k0 + lane * 32);
      float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int v = 0; v < 4; ++v) {  // eight activations: words 0, 1 hold elements 0..3, words 2, 3 elements 4..7
        const uint4 t = src[v];
        const uint32_t tw[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          xs2[4 * v + 2 * c] = make_float2(__uint_as_float(tw[c] << 16), __uint_as_float(tw[c + 2] << 16));
          xs2[4 * v + 2 * c + 1] = make_float2(__uint_as_float(tw[c] & 0xFFFF0000u), __uint_as_float(tw[c + 2] & 0xFFFF0000u));
        }
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) sum2 = __fadd2_rn(sum2, xs2[e]);
      xsum = sum2.x + sum2.y;
    }
    // group scales of the eight channels: chunk c lies in group c / 4
    const int group = (k0 >> 7) + (lane >> 2);
    const uint4 sc = *reinterpret_cast<const uint4*>(p.scales + static_cast<long long>(group) * p.n + n0);
    const uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      const float acc = gemv_chunk(piece[r], xs2);
      const float dot = fmaf(128.0f, acc, -136.0f * xsum);  // sum x * q over the chunk
      const float scale = (r & 1) ? __uint_as_float(sw[r >> 1] & 0xFFFF0000u) : __uint_as_float(sw[r >> 1] << 16);
      total[r] = fmaf(scale, dot, total[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) total[r] += __shfl_xor_sync(0xffffffffu, total[r], off);
  }
  if (lane < kGemvRows) {
    float mine = total[0];
#pragma unroll
    for (int r = 1; r < kGemvRows; ++r) mine = lane == r ? total[r] : mine;
    partial[warp][lane] = mine;
  }
  __syncthreads();
  if (active && first_slab == 0 && lane == 0) {
    uint32_t o[4];
#pragma unroll
    for (int r = 0; r < kGemvRows; r += 2) {
      float a = 0.0f, b = 0.0f;
      for (int s = 0; s < share; ++s) {  // fixed order: deterministic
        a += partial[warp + s][r];
        b += partial[warp + s][r + 1];
      }
      if (p.bias != nullptr) {
        a += __bfloat162float(p.bias[n0 + r]);
        b += __bfloat162float(p.bias[n0 + r + 1]);
      }
      o[r >> 1] = pack_bf16x2(a, b);
    }
    *reinterpret_cast<uint4*>(p.out + n0) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace rk
