// Activation / weight quantizers and block-scale packers (HBM-bound, SIMT).
//
// Row quantizers: one CTA of 256 threads per row, 128-bit loads, the row cached in registers
// (8192 elements at most on the cached path), warp-shuffle + shared-memory reductions, and the
// producer op (GELU table, AdaLN modulation, LayerNorm, RMSNorm, gated residual) fused in front
// of the absmax so the bf16 intermediate never round-trips through HBM.
//
// All divisions and reciprocals that define a stored scale or code use the IEEE-rounded
// intrinsics (__fdiv_rn, __frcp_rn); this file must not be built with fast-math.

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "rk_blockscale.cuh"
#include "rk_common.cuh"
#include "rk_host.h"

namespace rk {
namespace {

constexpr int kRowThreads = 256;
constexpr int kMaxVec = 4;                              // 8-element vectors cached per thread
constexpr int kCachedK = kRowThreads * kMaxVec * 8;     // 8192

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from a previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
  return r;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, bool vec, int valid, float (&v)[8]) {
  if (vec && valid >= 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = bf16_bits_to_float(w[i] & 0xFFFFu);
      v[2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = i < valid ? __bfloat162float(p[i]) : 0.0f;
  }
}

// eight values that are already bf16-representable (or are to be rounded to nearest even) as one 16-byte store
__device__ __forceinline__ void store8(__nv_bfloat16* p, bool vec, int valid, const float (&v)[8]) {
  if (vec && valid >= 8) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < valid) p[i] = __float2bfloat16_rn(v[i]);
  }
}

// clamp(rint(v / scale)) as an int in [-limit, limit]
__device__ __forceinline__ int quant_code(float v, float scale, float limit) {
  float q = rintf(__fdiv_rn(v, scale));
  q = fminf(fmaxf(q, -limit), limit);
  return __float2int_rn(q);
}

// Writes eight codes starting at element index `idx` of a padded row.
template <int BITS>
__device__ __forceinline__ void store_codes8(uint8_t* qrow, int idx, const int (&c)[8]) {
  if constexpr (BITS == 8) {
    uint2 o;
    o.x = (c[0] & 255) | ((c[1] & 255) << 8) | ((c[2] & 255) << 16) | ((c[3] & 255) << 24);
    o.y = (c[4] & 255) | ((c[5] & 255) << 8) | ((c[6] & 255) << 16) | ((c[7] & 255) << 24);
    *reinterpret_cast<uint2*>(qrow + idx) = o;
  } else {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) o |= static_cast<uint32_t>(c[i] & 15) << (4 * i);
    *reinterpret_cast<uint32_t*>(qrow + idx / 2) = o;
  }
}

// Eight codes at once, bit-identical to quant_code() on every element but without a division, a
// round instruction and a float -> int conversion per element (those made the row quantizers
// instruction-bound: ~31 instructions per element at 17% of DRAM bandwidth).
//   u = v * rcp, rcp = fl(1 / scale), lies within 3 * 2^-24 * |q| <= 2.3e-5 of the correctly rounded
//   quotient wherever the result is not clamped anyway (|q| <= 127.5); t = u + 1.5 * 2^23 rounds u to
//   the nearest integer (ties to even) and leaves that integer in the low mantissa bits, so the low
//   byte of the clamped t IS the two's-complement code.  Only if some u lies within 4e-5 of a tie (or
//   is not a number) could the exact quotient round the other way; then all eight take the exact
//   sequence (about one group of eight in a thousand).
// Elements at and beyond `k` must already be zero in v.
template <int BITS>
__device__ __forceinline__ void quantize_store8(uint8_t* qrow, int idx, const float (&v)[8], float scale, float rcp,
                                                float limit) {
  const float magic = 12582912.0f;  // 1.5 * 2^23, bits 0x4B400000
  float t[8];
  bool near_tie = false;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float u = __fmul_rn(v[i], rcp);
    t[i] = __fadd_rn(u, magic);
    const float e = __fsub_rn(u, __fsub_rn(t[i], magic));  // exact: distance of u from the integer it rounded to
    near_tie |= !(fabsf(e) < 0.49996f);
  }
  if (near_tie) {
    int c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = quant_code(v[i], scale, limit);
    store_codes8<BITS>(qrow, idx, c);
    return;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) t[i] = fminf(fmaxf(t[i], magic - limit), magic + limit);
  if constexpr (BITS == 8) {
    uint32_t b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) b[i] = __float_as_uint(t[i]);
    uint2 o;
    o.x = __byte_perm(__byte_perm(b[0], b[1], 0x0040u), __byte_perm(b[2], b[3], 0x0040u), 0x5410u);
    o.y = __byte_perm(__byte_perm(b[4], b[5], 0x0040u), __byte_perm(b[6], b[7], 0x0040u), 0x5410u);
    *reinterpret_cast<uint2*>(qrow + idx) = o;
  } else {
    int c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = __float_as_int(t[i]) - 0x4B400000;
    store_codes8<BITS>(qrow, idx, c);
  }
}

__device__ __forceinline__ float row_scale_from_max(float maximum, float limit, bool true_division) {
  if (!(maximum > 0.0f)) return 1.0f;
  // activations: max * fl32(1/limit); weights: max / limit
  return true_division ? __fdiv_rn(maximum, limit) : __fmul_rn(maximum, static_cast<float>(1.0 / limit));
}

// Common tail: absmax over cached values, scale, quantize, store (zero padding to kpad).
template <int BITS>
__device__ __forceinline__ void finish_row(float (&vals)[kMaxVec][8], int k, int kpad, uint8_t* qrow, float* scale_out,
                                           bool true_division, float* scratch) {
  const float limit = static_cast<float>((1 << (BITS - 1)) - 1);
  float local = 0.0f;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it)
#pragma unroll
    for (int i = 0; i < 8; ++i) local = fmaxf(local, fabsf(vals[it][i]));
  const float maximum = block_reduce(local, true, scratch);
  const float scale = row_scale_from_max(maximum, limit, true_division);
  if (threadIdx.x == 0) *scale_out = scale;
  const float rcp = __frcp_rn(scale);
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * static_cast<int>(blockDim.x) + threadIdx.x) * 8;
    if (idx < kpad) {
      if (idx + 8 > k) {  // ragged end of the row: codes beyond k are zero
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (idx + i >= k) vals[it][i] = 0.0f;
      }
      quantize_store8<BITS>(qrow, idx, vals[it], scale, rcp, limit);
    }
  }
}

// ------------------------------------------------------------------ plain / GELU-table rows
template <int BITS, int MODE>
__global__ void __launch_bounds__(kRowThreads)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const __nv_bfloat16* __restrict__ up,
                  long long up_stride, const __nv_bfloat16* __restrict__ lut, int k, int kpad, int n_rows,
                  uint8_t* __restrict__ q, float* __restrict__ scales, int true_division, int vec_ok) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  __shared__ float scratch[kRowThreads / 32];
  const int row = blockIdx.x;
  const int qbytes = BITS == 8 ? kpad : kpad / 2;
  uint8_t* qrow = q + static_cast<long long>(row) * qbytes;
  if (row >= n_rows) {  // padding row of a weight matrix: zero codes, unit scale
    for (int i = threadIdx.x * 4; i < qbytes; i += static_cast<int>(blockDim.x) * 4) *reinterpret_cast<uint32_t*>(qrow + i) = 0;
    if (threadIdx.x == 0) scales[row] = 1.0f;
    return;
  }
  const __nv_bfloat16* xr = x + row * x_stride;
  const __nv_bfloat16* ur = MODE == RK_ACT_LUT_MUL ? up + row * up_stride : nullptr;
  auto values_at = [&](int idx, float (&v)[8]) {
    const int valid = k - idx;
    load8(xr + idx, vec_ok, valid, v);
    if constexpr (MODE != RK_ACT_PLAIN) {
      float u[8];
      if constexpr (MODE == RK_ACT_LUT_MUL) load8(ur + idx, vec_ok, valid, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i < valid) {
          const uint32_t bits = __float_as_uint(v[i]) >> 16;
          float t = __bfloat162float(lut[bits]);
          if constexpr (MODE == RK_ACT_LUT_MUL) t = round_bf16(__fmul_rn(t, u[i]));
          v[i] = t;
        }
      }
    }
  };
  const int threads = static_cast<int>(blockDim.x);  // 64, 128 or 256: see launch_quant_rows
  if (k <= threads * kMaxVec * 8) {
    float vals[kMaxVec][8];
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int idx = (it * threads + threadIdx.x) * 8;
      if (idx < k) {
        values_at(idx, vals[it]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) vals[it][i] = 0.0f;
      }
    }
    finish_row<BITS>(vals, k, kpad, qrow, scales + row, true_division != 0, scratch);
  } else {
    // long rows: two passes over global memory (the second one hits L2)
    const float limit = static_cast<float>((1 << (BITS - 1)) - 1);
    float local = 0.0f;
    for (int idx = threadIdx.x * 8; idx < k; idx += threads * 8) {
      float v[8];
      values_at(idx, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) local = fmaxf(local, fabsf(v[i]));
    }
    const float maximum = block_reduce(local, true, scratch);
    const float scale = row_scale_from_max(maximum, limit, true_division != 0);
    if (threadIdx.x == 0) scales[row] = scale;
    const float rcp = __frcp_rn(scale);
    for (int idx = threadIdx.x * 8; idx < kpad; idx += threads * 8) {
      float v[8];
      if (idx < k) {
        values_at(idx, v);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (idx + i >= k) v[i] = 0.0f;
      quantize_store8<BITS>(qrow, idx, v, scale, rcp, limit);
    }
  }
}

// ------------------------------------------------------------------ table activation * up -> bf16 + tensor amax
// out = bf16(table[x] * up) element by element (the arithmetic of the GELU-table mode of the row
// quantizer above) and the absolute maximum of the finite results, for a per-tensor scale that a
// block packer needs before it can run.  Eight elements per thread and step; rows may be strided.
__global__ void __launch_bounds__(256)
lut_mul_amax_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const __nv_bfloat16* __restrict__ up,
                    long long up_stride, const __nv_bfloat16* __restrict__ lut, long long rows, int k,
                    __nv_bfloat16* __restrict__ out, unsigned* __restrict__ staging) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  __shared__ float scratch[8];
  const int per_row = k >> 3;
  const long long total = rows * per_row;
  float local = 0.0f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / per_row;
    const int col = static_cast<int>(i - row * per_row) << 3;
    const uint4 xv = *reinterpret_cast<const uint4*>(x + row * x_stride + col);
    const uint4 uv = *reinterpret_cast<const uint4*>(up + row * up_stride + col);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t ow[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float t0 = __bfloat162float(lut[xw[w] & 0xFFFFu]);
      const float t1 = __bfloat162float(lut[xw[w] >> 16]);
      const float r0 = round_bf16(__fmul_rn(t0, __uint_as_float(uw[w] << 16)));
      const float r1 = round_bf16(__fmul_rn(t1, __uint_as_float(uw[w] & 0xFFFF0000u)));
      const float a0 = fabsf(r0), a1 = fabsf(r1);
      if (a0 <= 3.4028234664e38f) local = fmaxf(local, a0);
      if (a1 <= 3.4028234664e38f) local = fmaxf(local, a1);
      ow[w] = (__float_as_uint(r0) >> 16) | (__float_as_uint(r1) & 0xFFFF0000u);
    }
    *reinterpret_cast<uint4*>(out + row * k + col) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
  if (staging != nullptr) {
    const float block_max = block_reduce(local, true, scratch);
    if (threadIdx.x == 0 && block_max > 0.0f) atomicMax(staging, __float_as_uint(block_max));
  }
}

// ------------------------------------------------------------------ AdaLN modulation (+LayerNorm, +gated residual)
template <int BITS>
__global__ void __launch_bounds__(kRowThreads)
quant_rows_modulated_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ mod_scale,
                            const __nv_bfloat16* __restrict__ mod_shift, int k, int kpad, int tokens, int layer_norm,
                            float eps, const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ gate,
                            __nv_bfloat16* __restrict__ residual_out, uint8_t* __restrict__ q,
                            float* __restrict__ scales) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  __shared__ float scratch[kRowThreads / 32];
  const int row = blockIdx.x;
  const long long xoff = static_cast<long long>(row) * k;
  const long long moff = static_cast<long long>(row / tokens) * k;
  uint8_t* qrow = q + static_cast<long long>(row) * (BITS == 8 ? kpad : kpad / 2);
  const bool vec = (k % 8) == 0;
  float vals[kMaxVec][8];
  float sum = 0.0f;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * kRowThreads + threadIdx.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) vals[it][i] = 0.0f;
    if (idx < k) {
      const int valid = k - idx;
      load8(x + xoff + idx, vec, valid, vals[it]);
      if (y != nullptr) {
        float yv[8], gv[8];
        load8(y + xoff + idx, vec, valid, yv);
        load8(gate + moff + idx, vec, valid, gv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          // residual = bf16(x + bf16(y * gate))
          vals[it][i] = round_bf16(__fadd_rn(vals[it][i], round_bf16(__fmul_rn(yv[i], gv[i]))));
        }
        store8(residual_out + xoff + idx, vec, valid, vals[it]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += (i < valid) ? vals[it][i] : 0.0f;
    }
  }
  if (layer_norm) {
    const float mean = __fdiv_rn(block_reduce(sum, false, scratch), static_cast<float>(k));
    float sq = 0.0f;
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int idx = (it * kRowThreads + threadIdx.x) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = (idx + i < k) ? __fsub_rn(vals[it][i], mean) : 0.0f;
        vals[it][i] = c;
        sq += c * c;
      }
    }
    const float var = __fdiv_rn(block_reduce(sq, false, scratch), static_cast<float>(k));
    const float inv = rsqrtf(var + eps);
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it)
#pragma unroll
      for (int i = 0; i < 8; ++i) vals[it][i] = round_bf16(__fmul_rn(vals[it][i], inv));
  }
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * kRowThreads + threadIdx.x) * 8;
    if (idx < k) {
      const int valid = k - idx;
      float sc[8], sh[8];
      load8(mod_scale + moff + idx, vec, valid, sc);
      load8(mod_shift + moff + idx, vec, valid, sh);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // bf16(bf16(x * bf16(1 + scale)) + shift)
        const float factor = round_bf16(__fadd_rn(1.0f, sc[i]));
        const float product = round_bf16(__fmul_rn(vals[it][i], factor));
        vals[it][i] = (i < valid) ? round_bf16(__fadd_rn(product, sh[i])) : 0.0f;
      }
    }
  }
  finish_row<BITS>(vals, k, kpad, qrow, scales + row, false, scratch);
}

// ------------------------------------------------------------------ RMSNorm (Gemma) -> quantize
// n = bf16( fl(fl(s * inv) * fl(1 + a)) + b ), inv = rsqrt(mean(s^2) + eps);
//   plain:    a = weight[k], b absent;  adaptive: a = scale[row / tokens, k], b = shift[row / tokens, k].
template <int BITS>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                          const __nv_bfloat16* __restrict__ gate,
                          const __nv_bfloat16* __restrict__ a_ptr, const __nv_bfloat16* __restrict__ b_ptr,
                          int tokens, int k, int kpad, float eps, __nv_bfloat16* __restrict__ sum_out,
                          __nv_bfloat16* __restrict__ norm_out, uint8_t* __restrict__ q, float* __restrict__ scales) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  __shared__ float scratch[kRowThreads / 32];
  const int row = blockIdx.x;
  const long long xoff = static_cast<long long>(row) * k;
  const long long aoff = tokens > 0 ? static_cast<long long>(row / tokens) * k : 0;
  uint8_t* qrow = BITS == 16 ? q : q + static_cast<long long>(row) * (BITS == 8 ? kpad : kpad / 2);
  const bool vec = (k % 8) == 0;
  float vals[kMaxVec][8];
  float sq = 0.0f;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * kRowThreads + threadIdx.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) vals[it][i] = 0.0f;
    if (idx < k) {
      const int valid = k - idx;
      load8(x + xoff + idx, vec, valid, vals[it]);
      if (residual != nullptr) {
        float rv[8];
        load8(residual + xoff + idx, vec, valid, rv);
        if (gate != nullptr) {  // gated residual: the branch is scaled per (batch entry, channel) first
          float gv[8];
          load8(gate + aoff + idx, vec, valid, gv);
#pragma unroll
          for (int i = 0; i < 8; ++i) rv[i] = round_bf16(__fmul_rn(rv[i], gv[i]));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) vals[it][i] = round_bf16(__fadd_rn(vals[it][i], rv[i]));
      }
      if (sum_out != nullptr) store8(sum_out + xoff + idx, vec, valid, vals[it]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < valid) sq += vals[it][i] * vals[it][i];
    }
  }
  const float var = __fdiv_rn(block_reduce(sq, false, scratch), static_cast<float>(k));
  const float inv = rsqrtf(var + eps);
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * kRowThreads + threadIdx.x) * 8;
    if (idx < k) {
      const int valid = k - idx;
      float av[8], bv[8];
      load8(a_ptr + aoff + idx, vec, valid, av);
      if (b_ptr != nullptr) load8(b_ptr + aoff + idx, vec, valid, bv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = __fmul_rn(__fmul_rn(vals[it][i], inv), __fadd_rn(1.0f, av[i]));
        if (b_ptr != nullptr) t = __fadd_rn(t, bv[i]);
        t = (i < valid) ? round_bf16(t) : 0.0f;
        vals[it][i] = t;
      }
      if (norm_out != nullptr) store8(norm_out + xoff + idx, vec, valid, vals[it]);
    }
  }
  if constexpr (BITS == 16) {
    // no row quantizer: the bf16 result is the output (norm_out) and the tensor's absolute maximum
    // (finite values only) is collected for a per-tensor scale; `q` is that staging word, or null
    if (q != nullptr) {
      float local = 0.0f;
#pragma unroll
      for (int it = 0; it < kMaxVec; ++it)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float a = fabsf(vals[it][i]);
          if (a <= 3.4028234664e38f) local = fmaxf(local, a);
        }
      const float row_max = block_reduce(local, true, scratch);
      if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned*>(q), __float_as_uint(row_max));
    }
  } else {
    finish_row<BITS>(vals, k, kpad, qrow, scales + row, false, scratch);
  }
}

// ------------------------------------------------------------------ W4 group-128 weight packer
// One warp per (row, group of 128): four consecutive elements per lane.
__global__ void __launch_bounds__(256)
pack_w4_g128_kernel(const __nv_bfloat16* __restrict__ w, int n, int k, uint8_t* __restrict__ q,
                    __nv_bfloat16* __restrict__ scales) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const int groups = k / 128;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(n) * groups) return;
  const int row = static_cast<int>(gw / groups);
  const int g = static_cast<int>(gw % groups);
  const __nv_bfloat16* src = w + static_cast<long long>(row) * k + g * 128 + lane * 4;
  const uint2 u = *reinterpret_cast<const uint2*>(src);
  float v[4] = {bf16_bits_to_float(u.x & 0xFFFFu), bf16_bits_to_float(u.x >> 16), bf16_bits_to_float(u.y & 0xFFFFu),
                bf16_bits_to_float(u.y >> 16)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  // s = bf16(amax / 7) (1.0 for an all-zero group); codes use float(s)
  __nv_bfloat16 sb = __float2bfloat16_rn(amax > 0.0f ? __fdiv_rn(amax, 7.0f) : 1.0f);
  if (!(__bfloat162float(sb) > 0.0f)) sb = __float2bfloat16_rn(1.0f);  // amax / 7 flushed to zero in bf16
  const float s = __bfloat162float(sb);
  if (lane == 0) scales[static_cast<long long>(g) * n + row] = sb;
  // Eight consecutive weights k0..k7 share one 32-bit word whose byte b holds k_b in its low nibble
  // and k_{b+4} in its high nibble (the order the GEMM's expansion step consumes cheapest).  An
  // even lane owns k0..k3, its odd neighbour k4..k7.
  uint32_t spread = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) spread |= static_cast<uint32_t>(quant_code(v[i], s, 7.0f) & 15) << (8 * i);
  const uint32_t upper = __shfl_xor_sync(0xffffffffu, spread, 1);
  if (!(lane & 1))
    *reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * (k / 2) + g * 64 + (lane >> 1) * 4) =
        spread | (upper << 4);
}

// ------------------------------------------------------------------ per-tensor FP8
__global__ void __launch_bounds__(256)
amax_finite_kernel(const __nv_bfloat16* __restrict__ x, long long elements, unsigned* __restrict__ amax_bits) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  __shared__ float scratch[8];
  float local = 0.0f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; idx < elements;
       idx += stride) {
    float v[8];
    const long long left = elements - idx;
    load8(x + idx, true, left >= 8 ? 8 : static_cast<int>(left), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = fabsf(v[i]);
      if (a <= 3.4028234664e38f) local = fmaxf(local, a);  // skips inf and NaN
    }
  }
  local = warp_max(local);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = scratch[0];
    for (int w = 1; w < 8; ++w) r = fmaxf(r, scratch[w]);
    atomicMax(amax_bits, __float_as_uint(r));  // non-negative floats order like their bit patterns
  }
}

// scale = max(amax / divisor, 1e-12); also clears the staging word for the next call
__global__ void finalize_scale_kernel(unsigned* amax_bits, float divisor, float* scale_out) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const float amax = __uint_as_float(*amax_bits);
  *scale_out = fmaxf(__fdiv_rn(amax, divisor), 1e-12f);
  *amax_bits = 0u;
}

__global__ void __launch_bounds__(256)
to_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long elements, const float* __restrict__ scale,
              uint8_t* __restrict__ q) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const float inverse = __fdiv_rn(1.0f, *scale);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; idx < elements;
       idx += stride) {
    float v[8];
    const long long left = elements - idx;
    const int valid = left >= 8 ? 8 : static_cast<int>(left);
    load8(x + idx, true, valid, v);
    uint8_t c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float t = __fmul_rn(v[i], inverse);
      t = fminf(448.0f, fmaxf(-448.0f, t));
      c[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3));
    }
    if (valid == 8) {
      uint2 o;
      o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (static_cast<uint32_t>(c[3]) << 24);
      o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (static_cast<uint32_t>(c[7]) << 24);
      *reinterpret_cast<uint2*>(q + idx) = o;
    } else {
      for (int i = 0; i < valid; ++i) q[idx + i] = c[i];
    }
  }
}

// ------------------------------------------------------------------ block-scale packers
// MXFP8: eight lanes per 32-element block, four elements per lane.  The thread grid covers the
// padded scale-factor domain so that every byte of the SF buffer is written.
// SWIGLU: x is [rows, 2 k] (gate first, then up) and the packed value is bf16(table[gate] * up), `table`
// being SiLU on all 65536 bf16 bit patterns (blackwell/csrc/mxfp8_swiglu.cu:20-78).
template <bool SWIGLU>
__global__ void __launch_bounds__(256)
pack_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, long long rows, long long k, uint8_t* __restrict__ q,
                  uint8_t* __restrict__ sf, const __nv_bfloat16* __restrict__ table) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const long long groups_padded = (k + 127) / 128 * 4;
  const long long rows_padded = (rows + 127) / 128 * 128;
  const long long thread = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long block_index = thread / 8;
  const int lane8 = static_cast<int>(thread % 8);
  const long long row = block_index / groups_padded;
  const long long group = block_index % groups_padded;
  if (row >= rows_padded) return;
  const long long sfi = sf_offset(row, group, groups_padded / 4);
  if (row >= rows || group * 32 >= k) {
    if (lane8 == 0) sf[sfi] = 0;
    return;
  }
  const long long base = row * k + group * 32 + lane8 * 4;
  float v[4];
  if constexpr (SWIGLU) {
    const long long in = row * 2 * k + group * 32 + lane8 * 4;
    const uint2 g = *reinterpret_cast<const uint2*>(x + in);
    const uint2 u = *reinterpret_cast<const uint2*>(x + in + k);
    const uint32_t gb[4] = {g.x & 0xFFFFu, g.x >> 16, g.y & 0xFFFFu, g.y >> 16};
    const uint32_t ub[4] = {u.x & 0xFFFFu, u.x >> 16, u.y & 0xFFFFu, u.y >> 16};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = round_bf16(__fmul_rn(__bfloat162float(table[gb[i]]), bf16_bits_to_float(ub[i])));
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(x + base);
    v[0] = bf16_bits_to_float(u.x & 0xFFFFu), v[1] = bf16_bits_to_float(u.x >> 16);
    v[2] = bf16_bits_to_float(u.y & 0xFFFFu), v[3] = bf16_bits_to_float(u.y >> 16);
  }
  float amax = 0.0f;
  unsigned invalid = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    amax = fmaxf(amax, fabsf(v[i]));
    invalid |= !(fabsf(v[i]) <= 3.4028234664e38f);
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 8));
    invalid |= __shfl_xor_sync(0xffffffffu, invalid, o, 8);
  }
  const uint32_t e = mxfp8_block_scale(amax, invalid != 0);
  if (lane8 == 0) sf[sfi] = static_cast<uint8_t>(e);
  const float inverse = mxfp8_inverse_scale(e);
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fmul_rn(v[i], inverse), __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  *reinterpret_cast<uint32_t*>(q + base) = out;
}

// The scale of the W4A8-MX formats: the smallest power of two >= v, as a UE8M0 exponent byte (1.0 for
// v <= 0 or NaN; blackwell/csrc/fp4_mx_cutlass_linear.cu:47-58, `ceil_power_of_two`).
__device__ __forceinline__ uint32_t ceil_pow2_ue8m0(float v) {
  if (!(v > 0.0f)) return 127u;
  const uint32_t bits = __float_as_uint(v);
  uint32_t e = bits >> 23;             // biased exponent (v > 0: no sign bit)
  if (e == 0u) return 1u;              // subnormal input: below 2^-126, the smallest normal scale covers it
  if (bits & 0x7FFFFFu) ++e;           // not a power of two: round up
  return e > 254u ? 254u : e;
}

// W4A8-MX, 32-element blocks, eight lanes per block (four elements per lane); FMT 0: MXFP8 activations
// q = e4m3(clamp(x / s, +-448)), s = ceil_pow2(amax / 448); FMT 1: MXFP4 weights q = e2m1(x / s),
// s = ceil_pow2(amax / 6), two codes per byte, low nibble = even k.  Reference:
// blackwell/csrc/fp4_mx_cutlass_linear.cu:59-132.  Every byte of the scale buffer is written.
template <int FMT>
__global__ void __launch_bounds__(256)
pack_mx_ceil_kernel(const __nv_bfloat16* __restrict__ x, long long rows, long long k, uint8_t* __restrict__ q,
                    uint8_t* __restrict__ sf) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const long long groups_padded = (k + 127) / 128 * 4;
  const long long rows_padded = (rows + 127) / 128 * 128;
  const long long thread = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long block_index = thread / 8;
  const int lane8 = static_cast<int>(thread % 8);
  const long long row = block_index / groups_padded;
  const long long group = block_index % groups_padded;
  if (row >= rows_padded) return;
  const long long sfi = sf_offset(row, group, groups_padded / 4);
  if (row >= rows || group * 32 >= k) {
    if (lane8 == 0) sf[sfi] = 0;
    return;
  }
  const long long base = row * k + group * 32 + lane8 * 4;
  const uint2 u = *reinterpret_cast<const uint2*>(x + base);
  const float v[4] = {bf16_bits_to_float(u.x & 0xFFFFu), bf16_bits_to_float(u.x >> 16), bf16_bits_to_float(u.y & 0xFFFFu),
                      bf16_bits_to_float(u.y >> 16)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 8));
  const uint32_t e = ceil_pow2_ue8m0(__fdiv_rn(amax, FMT == 0 ? 448.0f : 6.0f));
  if (lane8 == 0) sf[sfi] = static_cast<uint8_t>(e);
  const float inverse = __uint_as_float((254u - e) << 23);  // 2^(127 - e), e in 1..254
  if constexpr (FMT == 0) {
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float t = fminf(448.0f, fmaxf(-448.0f, __fmul_rn(v[i], inverse)));
      out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    }
    *reinterpret_cast<uint32_t*>(q + base) = out;
  } else {
    const uint32_t lo = __nv_cvt_float2_to_fp4x2(make_float2(__fmul_rn(v[0], inverse), __fmul_rn(v[1], inverse)), __NV_E2M1,
                                                 cudaRoundNearest);
    const uint32_t hi = __nv_cvt_float2_to_fp4x2(make_float2(__fmul_rn(v[2], inverse), __fmul_rn(v[3], inverse)), __NV_E2M1,
                                                 cudaRoundNearest);
    *reinterpret_cast<unsigned short*>(q + base / 2) = static_cast<unsigned short>((lo & 0xFFu) | ((hi & 0xFFu) << 8));
  }
}

// NVFP4: one thread per 16-element block (two 128-bit loads, one 64-bit store).
__global__ void __launch_bounds__(256)
pack_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, long long rows, long long k, const float* __restrict__ global,
                  uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const long long groups = k / 16;
  const long long groups_padded = (groups + 3) / 4 * 4;
  const long long rows_padded = (rows + 127) / 128 * 128;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = idx / groups_padded;
  const long long group = idx % groups_padded;
  if (row >= rows_padded) return;
  const long long sfi = sf_offset(row, group, groups_padded / 4);
  if (row >= rows || group >= groups) {
    sf[sfi] = 0;
    return;
  }
  float v[16];
  load8(x + row * k + group * 16, true, 8, *reinterpret_cast<float(*)[8]>(&v[0]));
  load8(x + row * k + group * 16 + 8, true, 8, *reinterpret_cast<float(*)[8]>(&v[8]));
  if (global != nullptr) {
    // v / g for sixteen values and one divisor.  With r = fl(1 / g) correctly rounded, q = fl(v r)
    // corrected by its exact residual - e = fma(-q, g, v), q' = fma(e, r, q) - IS the correctly rounded
    // quotient (Markstein's theorem) unless the significand of g is all ones; the magnitude window
    // keeps every intermediate in the normal range.  Everything else (zeros, whose sign the division
    // keeps, tiny and huge values, such a divisor) takes the IEEE division.  16 divisions cost ~10
    // instructions each and made this kernel instruction bound.
    const float g = *global;
    const float r = __frcp_rn(g);
    const bool divisor_ok = (__float_as_uint(g) & 0x7FFFFFu) != 0x7FFFFFu && g >= 0x1p-40f && g <= 0x1p40f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float a = fabsf(v[i]);
      if (divisor_ok && a >= 0x1p-60f && a <= 0x1p60f) {
        const float q = __fmul_rn(v[i], r);
        v[i] = __fmaf_rn(__fmaf_rn(-q, g, v[i]), r, q);
      } else {
        v[i] = __fdiv_rn(v[i], g);
      }
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float scale = amax > 0.0f ? __fdiv_rn(amax, 6.0f) : 1.0f;
  const uint8_t code = static_cast<uint8_t>(__nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E4M3)) & 0x7F;
  float deq = __half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3)));
  if (!(deq > 0.0f)) deq = scale;
  const float reciprocal = __fdiv_rn(1.0f, deq);
  unsigned long long packed = 0;
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const __nv_fp4x2_storage_t pair = __nv_cvt_float2_to_fp4x2(
        make_float2(__fmul_rn(v[i], reciprocal), __fmul_rn(v[i + 1], reciprocal)), __NV_E2M1, cudaRoundNearest);
    packed |= static_cast<unsigned long long>(static_cast<uint8_t>(pair)) << (4 * i);
  }
  *reinterpret_cast<unsigned long long*>(q + row * (k / 2) + group * 8) = packed;
  sf[sfi] = code;
}

// ------------------------------------------------------------------ fused producers for the FP8 / NVFP4 GEMMs
// SwiGLU in fp32, as the reference's per-tensor FP8 producer evaluates it
// (blackwell/csrc/fp8_cutlass_linear.cu:271-279): bf16( gate / (1 + exp(-gate)) * up ).
__device__ __forceinline__ float swiglu_f32(float gate, float up) {
  return round_bf16(__fmul_rn(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))), up));
}
// Eight consecutive SwiGLU outputs of row-major gate_up [rows, 2 * inter]: gate first, then up; or
// `interleaved`: blocks of 128 columns, 64 up values followed by their 64 gate values (the layout a
// fused gate/up projection writes: blackwell/csrc/fp4_cutlass_linear.cu:958-965).
template <bool BF16_STEPS>
__device__ __forceinline__ void load8_swiglu(const __nv_bfloat16* gate_up, long long inter, long long idx, int valid,
                                             float (&v)[8], bool interleaved = false) {
  const long long row = idx / inter, col = idx - row * inter;
  const __nv_bfloat16* g = gate_up + row * 2 * inter + col;
  const __nv_bfloat16* u = g + inter;
  if (interleaved) {  // eight consecutive columns never straddle a 64-column block
    u = gate_up + row * 2 * inter + (col >> 6) * 128 + (col & 63);
    g = u + 64;
  }
  float gv[8], uv[8];
  const bool vec = (inter % 8) == 0;
  load8(g, vec, valid, gv);
  load8(u, vec, valid, uv);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = i < valid ? (BF16_STEPS ? swiglu_bf16_steps(gv[i], uv[i]) : swiglu_f32(gv[i], uv[i])) : 0.0f;
}

// SwiGLU -> MXFP8 with power-of-two (ceil) block scales, the activation side of W4A8-MX
// (blackwell/csrc/fp4_mx_cutlass_linear.cu:134-179, `pack_swiglu_mxfp8_warp_kernel`): the product
// gate / (1 + exp(-gate)) * up stays in fp32 (no bf16 rounding) before the block quantizer.
__global__ void __launch_bounds__(256)
swiglu_pack_mxfp8_ceil_kernel(const __nv_bfloat16* __restrict__ gate_up, long long rows, long long inter, int interleaved,
                              uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const long long groups_padded = (inter + 127) / 128 * 4;
  const long long rows_padded = (rows + 127) / 128 * 128;
  const long long thread = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long block_index = thread / 8;
  const int lane8 = static_cast<int>(thread % 8);
  const long long row = block_index / groups_padded;
  const long long group = block_index % groups_padded;
  if (row >= rows_padded) return;
  const long long sfi = sf_offset(row, group, groups_padded / 4);
  if (row >= rows || group * 32 >= inter) {
    if (lane8 == 0) sf[sfi] = 0;
    return;
  }
  const long long col = group * 32 + lane8 * 4;
  const __nv_bfloat16* g = gate_up + row * 2 * inter + col;
  const __nv_bfloat16* u = g + inter;
  if (interleaved) {
    u = gate_up + row * 2 * inter + (col >> 6) * 128 + (col & 63);
    g = u + 64;
  }
  const uint2 gw = *reinterpret_cast<const uint2*>(g), uw = *reinterpret_cast<const uint2*>(u);
  const float gv[4] = {bf16_bits_to_float(gw.x & 0xFFFFu), bf16_bits_to_float(gw.x >> 16), bf16_bits_to_float(gw.y & 0xFFFFu),
                       bf16_bits_to_float(gw.y >> 16)};
  const float uv[4] = {bf16_bits_to_float(uw.x & 0xFFFFu), bf16_bits_to_float(uw.x >> 16), bf16_bits_to_float(uw.y & 0xFFFFu),
                       bf16_bits_to_float(uw.y >> 16)};
  float v[4], amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = __fmul_rn(__fdiv_rn(gv[i], __fadd_rn(1.0f, expf(-gv[i]))), uv[i]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 8));
  const uint32_t e = ceil_pow2_ue8m0(__fdiv_rn(amax, 448.0f));
  if (lane8 == 0) sf[sfi] = static_cast<uint8_t>(e);
  const float inverse = __uint_as_float((254u - e) << 23);
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float t = fminf(448.0f, fmaxf(-448.0f, __fmul_rn(v[i], inverse)));
    out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(q + row * inter + col) = out;
}

__global__ void __launch_bounds__(256)
swiglu_amax_kernel(const __nv_bfloat16* __restrict__ gate_up, long long rows, long long inter,
                   unsigned* __restrict__ amax_bits) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  __shared__ float scratch[8];
  float local = 0.0f;
  const long long elements = rows * inter;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; idx < elements;
       idx += stride) {
    float v[8];
    load8_swiglu<false>(gate_up, inter, idx, 8, v);  // inter % 8 == 0: a vector never straddles rows
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = fabsf(v[i]);
      if (a <= 3.4028234664e38f) local = fmaxf(local, a);
    }
  }
  local = warp_max(local);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = scratch[0];
    for (int w = 1; w < 8; ++w) r = fmaxf(r, scratch[w]);
    atomicMax(amax_bits, __float_as_uint(r));
  }
}

__global__ void __launch_bounds__(256)
swiglu_to_fp8_kernel(const __nv_bfloat16* __restrict__ gate_up, long long rows, long long inter,
                     const float* __restrict__ scale, uint8_t* __restrict__ q) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const float inverse = __fdiv_rn(1.0f, *scale);
  const long long elements = rows * inter;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; idx < elements;
       idx += stride) {
    float v[8];
    load8_swiglu<false>(gate_up, inter, idx, 8, v);
    uint32_t c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float t = fminf(448.0f, fmaxf(-448.0f, __fmul_rn(v[i], inverse)));
      c[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3));
    }
    uint2 o;
    o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
    o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
    *reinterpret_cast<uint2*>(q + idx) = o;
  }
}

// SwiGLU -> NVFP4: one thread per 16-element block of the [rows, inter] activation.
__global__ void __launch_bounds__(256)
swiglu_pack_nvfp4_kernel(const __nv_bfloat16* __restrict__ gate_up, long long rows, long long inter, int interleaved,
                         uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const long long groups = inter / 16;
  const long long groups_padded = (groups + 3) / 4 * 4;
  const long long rows_padded = (rows + 127) / 128 * 128;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = idx / groups_padded;
  const long long group = idx % groups_padded;
  if (row >= rows_padded) return;
  const long long sfi = sf_offset(row, group, groups_padded / 4);
  if (row >= rows || group >= groups) {
    sf[sfi] = 0;
    return;
  }
  float v[16];
  load8_swiglu<true>(gate_up, inter, row * inter + group * 16, 8, *reinterpret_cast<float(*)[8]>(&v[0]), interleaved != 0);
  load8_swiglu<true>(gate_up, inter, row * inter + group * 16 + 8, 8, *reinterpret_cast<float(*)[8]>(&v[8]), interleaved != 0);
  uint8_t code;
  const unsigned long long packed = nvfp4_block(v, &code);
  *reinterpret_cast<unsigned long long*>(q + row * (inter / 2) + group * 8) = packed;
  sf[sfi] = code;
}

// SwiGLU alone, bf16 in the reference's bf16x2 steps (blackwell/csrc/fp4_cutlass_linear.cu:944-995,
// `silu_mul_bf16`): eight outputs per thread; either gate/up layout.
__global__ void __launch_bounds__(256)
silu_mul_bf16_kernel(const __nv_bfloat16* __restrict__ gate_up, long long rows, long long inter, int interleaved,
                     __nv_bfloat16* __restrict__ out) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const long long total = rows * inter;
  for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    float v[8];
    load8_swiglu<true>(gate_up, inter, idx, 8, v, interleaved != 0);  // inter % 8 == 0: a vector never straddles rows
    store8(out + idx, true, 8, v);
  }
}

// (residual add +) RMSNorm feeding a per-tensor FP8 quantizer (FMT 0: writes the bf16 results and the
// tensor's absolute maximum), an NVFP4 packer (FMT 1: packs straight from registers) or nothing (FMT 2: the
// plain norm of blackwell/csrc/fp4_cutlass_linear.cu:429-476).  Arithmetic
// of blackwell/csrc/fp8_cutlass_linear.cu:145-203 and blackwell/csrc/fp4_cutlass_linear.cu:843-929:
// s = bf16(x + residual); r = rsqrt(mean(s^2) + eps); y = bf16( bf16(s * r) * weight ).
// One CTA per row (FMT 1: per row of the 128-row padded scale-factor domain), row cached in registers.
template <int FMT>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_producer_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                        const __nv_bfloat16* __restrict__ weight, int rows, int k, float eps,
                        __nv_bfloat16* __restrict__ sum_out, __nv_bfloat16* __restrict__ norm_out,
                        unsigned* __restrict__ amax_bits, uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  __shared__ float scratch[kRowThreads / 32];
  const int row = blockIdx.x;
  const int groups = k / 16;
  const int groups_padded = (groups + 3) / 4 * 4;
  if (row >= rows) {  // FMT 1 only: padding rows of the scale-factor buffer read as zero
    for (int g = threadIdx.x; g < groups_padded; g += kRowThreads) sf[sf_offset(row, g, groups_padded / 4)] = 0;
    return;
  }
  const long long xoff = static_cast<long long>(row) * k;
  float vals[kMaxVec][8];
  float sq = 0.0f;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * kRowThreads + threadIdx.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) vals[it][i] = 0.0f;
    if (idx < k) {  // k % 16 == 0: whole vectors only
      load8(x + xoff + idx, true, 8, vals[it]);
      if (residual != nullptr) {
        float rv[8];
        load8(residual + xoff + idx, true, 8, rv);
#pragma unroll
        for (int i = 0; i < 8; ++i) vals[it][i] = round_bf16(__fadd_rn(vals[it][i], rv[i]));
        if (sum_out != nullptr) store8(sum_out + xoff + idx, true, 8, vals[it]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sq = fmaf(vals[it][i], vals[it][i], sq);
    }
  }
  const float inv = rsqrtf(__fadd_rn(__fdiv_rn(block_reduce(sq, false, scratch), static_cast<float>(k)), eps));
  float local_max = 0.0f;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * kRowThreads + threadIdx.x) * 8;
    if (idx < k) {
      float wv[8];
      load8(weight + idx, true, 8, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float y = round_bf16(__fmul_rn(round_bf16(__fmul_rn(vals[it][i], inv)), wv[i]));
        vals[it][i] = y;
        const float a = fabsf(y);
        if (a <= 3.4028234664e38f) local_max = fmaxf(local_max, a);
      }
      if (norm_out != nullptr) store8(norm_out + xoff + idx, true, 8, vals[it]);
    }
  }
  if (FMT == 2) return;  // the plain norm: the bf16 result is the output
  if (FMT == 0) {
    const float m = block_reduce(local_max, true, scratch);
    if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(m));
    return;
  }
  // FMT 1: a 16-element block is held by an even thread (low half) and its odd neighbour (high half)
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int idx = (it * kRowThreads + threadIdx.x) * 8;  // warp-uniform validity: k % 256 handled by the mask below
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, vals[it][i], 1);
      v[i] = (threadIdx.x & 1) ? other : vals[it][i];
      v[8 + i] = (threadIdx.x & 1) ? vals[it][i] : other;
    }
    if (idx < k) {
      uint8_t code;
      const unsigned long long packed = nvfp4_block(v, &code);
      const int group = idx / 16;
      // each thread stores the four code bytes of its own eight values
      const uint32_t mine = static_cast<uint32_t>((threadIdx.x & 1) ? (packed >> 32) : packed);
      *reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * (k / 2) + idx / 2) = mine;
      if (!(threadIdx.x & 1)) sf[sf_offset(row, group, groups_padded / 4)] = code;
    }
  }
  // scale factors of the padded groups of this row
  for (int g = groups + threadIdx.x; g < groups_padded; g += kRowThreads) sf[sf_offset(row, g, groups_padded / 4)] = 0;
}

__global__ void probe_rcp_kernel(uint32_t* out) { *out = __float_as_uint(rcp_approx_ftz(448.0f)); }

template <int BITS>
int launch_quant_rows(const void* x, int64_t rows, int64_t total_rows, int64_t k, int64_t xs, const void* up,
                      int64_t us, const void* lut, int mode, void* q, float* scales, int true_division,
                      cudaStream_t st) {
  const int kpad = static_cast<int>(round_up(k, 128));
  const int vec_ok = aligned16(x) && xs % 8 == 0 && (mode != RK_ACT_LUT_MUL || (aligned16(up) && us % 8 == 0));
  auto xb = static_cast<const __nv_bfloat16*>(x);
  auto ub = static_cast<const __nv_bfloat16*>(up);
  auto lb = static_cast<const __nv_bfloat16*>(lut);
  auto qb = static_cast<uint8_t*>(q);
  const dim3 grid(static_cast<unsigned>(total_rows));
  // One CTA per row.  With 256 threads a short row is one 16-byte load per thread and eight warps
  // to reduce over; once there are enough rows to give every SM several CTAs, 64 or 128 threads per
  // row (four vectors per thread, two or four warps to reduce, up to 32 resident CTAs per SM) are
  // faster (1764 x 2048: 8.3 -> 6.8 us; 16384 x 2048: 64.5 -> 37.8 us).  With few rows the machine
  // is not full and the per-thread latency decides, so those keep the full 256 threads
  // (400 x 4096: 4.5 us with 256 threads, 9.5 us with 64).
  int threads = kRowThreads;
  if (total_rows >= 1024) threads = kpad <= 2048 ? 64 : (kpad <= 4096 ? 128 : kRowThreads);
  switch (mode) {
    case RK_ACT_PLAIN:
      launch_pdl(quant_rows_kernel<BITS, RK_ACT_PLAIN>, grid, threads, st, xb, xs, ub, us, lb, static_cast<int>(k), kpad,
                                                                          static_cast<int>(rows), qb, scales,
                                                                          true_division, vec_ok);
      break;
    case RK_ACT_LUT_MUL:
      launch_pdl(quant_rows_kernel<BITS, RK_ACT_LUT_MUL>, grid, threads, st, 
          xb, xs, ub, us, lb, static_cast<int>(k), kpad, static_cast<int>(rows), qb, scales, true_division, vec_ok);
      break;
    default:
      launch_pdl(quant_rows_kernel<BITS, RK_ACT_LUT>, grid, threads, st, xb, xs, ub, us, lb, static_cast<int>(k), kpad,
                                                                        static_cast<int>(rows), qb, scales,
                                                                        true_division, vec_ok);
  }
  return check_launch("quant_rows");
}

}  // namespace
}  // namespace rk

namespace rk {
int launch_finalize_scale(unsigned* staging, float divisor, float* scale_out, cudaStream_t stream) {
  launch_pdl(finalize_scale_kernel, 1, 1, stream, staging, divisor, scale_out);
  return check_launch("finalize_scale");
}
}  // namespace rk

using namespace rk;

extern "C" int rk_quant_rows(const void* x, int64_t rows, int64_t k, int64_t x_stride, const void* up,
                             int64_t up_stride, const void* lut, int mode, int bits, void* q, float* scales,
                             void* stream) {
  if (!x || !q || !scales) return fail(RK_EINVAL, "rk_quant_rows: null pointer");
  if (bits != 4 && bits != 8) return fail(RK_EINVAL, "rk_quant_rows: bits must be 4 or 8");
  if (rows < 1 || k < 1 || k > 65536) return fail(RK_EINVAL, "rk_quant_rows: unsupported activation dimensions");
  if (mode < 0 || mode > 2) return fail(RK_EINVAL, "rk_quant_rows: unknown mode");
  if (mode != RK_ACT_PLAIN && !lut) return fail(RK_EINVAL, "rk_quant_rows: table required");
  if (mode == RK_ACT_LUT_MUL && !up) return fail(RK_EINVAL, "rk_quant_rows: gated mode needs `up`");
  if (x_stride < k || (mode == RK_ACT_LUT_MUL && up_stride < k)) return fail(RK_EINVAL, "rk_quant_rows: row stride < k");
  return bits == 8 ? launch_quant_rows<8>(x, rows, rows, k, x_stride, up, up_stride, lut, mode, q, scales, 0,
                                          as_stream(stream))
                   : launch_quant_rows<4>(x, rows, rows, k, x_stride, up, up_stride, lut, mode, q, scales, 0,
                                          as_stream(stream));
}

extern "C" int rk_quant_weight_int(const void* w, int64_t n, int64_t k, int bits, void* q, float* scales,
                                   void* stream) {
  if (!w || !q || !scales) return fail(RK_EINVAL, "rk_quant_weight_int: null pointer");
  if (bits != 4 && bits != 8) return fail(RK_EINVAL, "rk_quant_weight_int: bits must be 4 or 8");
  if (n < 1 || k < 1 || k > 65536) return fail(RK_EINVAL, "rk_quant_weight_int: unsupported weight dimensions");
  const int64_t npad = round_up(n, 8);
  return bits == 8 ? launch_quant_rows<8>(w, n, npad, k, k, nullptr, 0, nullptr, RK_ACT_PLAIN, q, scales, 1,
                                          as_stream(stream))
                   : launch_quant_rows<4>(w, n, npad, k, k, nullptr, 0, nullptr, RK_ACT_PLAIN, q, scales, 1,
                                          as_stream(stream));
}

extern "C" int rk_quant_rows_modulated(const void* x, const void* scale, const void* shift, int64_t rows, int64_t k,
                                       int64_t tokens, int layer_norm, float eps, const void* y, const void* gate,
                                       void* residual_out, int bits, void* q, float* scales, void* stream) {
  if (!x || !scale || !shift || !q || !scales) return fail(RK_EINVAL, "rk_quant_rows_modulated: null pointer");
  if (bits != 4 && bits != 8) return fail(RK_EINVAL, "rk_quant_rows_modulated: bits must be 4 or 8");
  if (rows < 1 || k < 1 || tokens < 1 || rows % tokens != 0)
    return fail(RK_EINVAL, "rk_quant_rows_modulated: rows must be a positive multiple of tokens");
  if (k > kCachedK) return fail(RK_EUNSUPPORTED, "rk_quant_rows_modulated: k > %d", kCachedK);
  if ((y == nullptr) != (gate == nullptr) || (y != nullptr && residual_out == nullptr))
    return fail(RK_EINVAL, "rk_quant_rows_modulated: y, gate and residual_out go together");
  if (!aligned16(x) || !aligned16(scale) || !aligned16(shift) || (y && (!aligned16(y) || !aligned16(gate))) ||
      (residual_out && !aligned16(residual_out)))
    return fail(RK_EINVAL, "rk_quant_rows_modulated: pointers must be 16-byte aligned");
  const int kpad = static_cast<int>(round_up(k, 128));
  auto b = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  if (bits == 8)
    launch_pdl(quant_rows_modulated_kernel<8>, static_cast<unsigned>(rows), kRowThreads, as_stream(stream), 
        b(x), b(scale), b(shift), static_cast<int>(k), kpad, static_cast<int>(tokens), layer_norm, eps, b(y), b(gate),
        static_cast<__nv_bfloat16*>(residual_out), static_cast<uint8_t*>(q), scales);
  else
    launch_pdl(quant_rows_modulated_kernel<4>, static_cast<unsigned>(rows), kRowThreads, as_stream(stream), 
        b(x), b(scale), b(shift), static_cast<int>(k), kpad, static_cast<int>(tokens), layer_norm, eps, b(y), b(gate),
        static_cast<__nv_bfloat16*>(residual_out), static_cast<uint8_t*>(q), scales);
  return check_launch("quant_rows_modulated");
}

namespace {
int launch_rmsnorm_quant_rows(const char* who, const void* x, const void* residual, const void* gate, const void* scale,
                              const void* shift, int64_t tokens, int64_t rows, int64_t k, float eps, int bits,
                              void* sum_out, void* norm_out, void* q, float* scales, void* stream) {
  if (!x || !scale || !q || !scales) return fail(RK_EINVAL, "%s: null pointer", who);
  if (bits != 4 && bits != 8) return fail(RK_EINVAL, "%s: bits must be 4 or 8", who);
  if (rows < 1 || k < 1 || tokens < 0 || (tokens > 0 && rows % tokens != 0))
    return fail(RK_EINVAL, "%s: bad row / token counts", who);
  if (gate && (!residual || tokens < 1)) return fail(RK_EINVAL, "%s: a gate needs a residual branch and tokens > 0", who);
  if (k > kCachedK) return fail(RK_EUNSUPPORTED, "%s: k > %d", who, kCachedK);
  if (!aligned16(x) || !aligned16(scale) || (residual && !aligned16(residual)) || (shift && !aligned16(shift)) ||
      (gate && !aligned16(gate)) || (sum_out && !aligned16(sum_out)) || (norm_out && !aligned16(norm_out)))
    return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  const int kpad = static_cast<int>(round_up(k, 128));
  auto b = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  if (bits == 8)
    launch_pdl(rmsnorm_quant_rows_kernel<8>, static_cast<unsigned>(rows), kRowThreads, as_stream(stream), 
        b(x), b(residual), b(gate), b(scale), b(shift), static_cast<int>(tokens), static_cast<int>(k), kpad, eps,
        static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(norm_out), static_cast<uint8_t*>(q), scales);
  else
    launch_pdl(rmsnorm_quant_rows_kernel<4>, static_cast<unsigned>(rows), kRowThreads, as_stream(stream), 
        b(x), b(residual), b(gate), b(scale), b(shift), static_cast<int>(tokens), static_cast<int>(k), kpad, eps,
        static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(norm_out), static_cast<uint8_t*>(q), scales);
  return check_launch(who);
}
}  // namespace

extern "C" int rk_rmsnorm_quant_rows(const void* x, const void* residual, const void* scale, const void* shift,
                                     int64_t tokens, int64_t rows, int64_t k, float eps, int bits, void* sum_out,
                                     void* norm_out, void* q, float* scales, void* stream) {
  return launch_rmsnorm_quant_rows("rk_rmsnorm_quant_rows", x, residual, nullptr, scale, shift, tokens, rows, k, eps, bits,
                                   sum_out, norm_out, q, scales, stream);
}

extern "C" int rk_gated_rmsnorm_quant_rows(const void* x, const void* branch, const void* gate, const void* scale,
                                           const void* shift, int64_t tokens, int64_t rows, int64_t k, float eps,
                                           int bits, void* sum_out, void* norm_out, void* q, float* scales,
                                           void* stream) {
  if (!branch || !gate) return fail(RK_EINVAL, "rk_gated_rmsnorm_quant_rows: null pointer");
  return launch_rmsnorm_quant_rows("rk_gated_rmsnorm_quant_rows", x, branch, gate, scale, shift, tokens, rows, k, eps,
                                   bits, sum_out, norm_out, q, scales, stream);
}

extern "C" int rk_rmsnorm_tensor_scale(const void* x, const void* residual, const void* scale, const void* shift,
                                       int64_t tokens, int64_t rows, int64_t k, float eps, float divisor, void* sum_out,
                                       void* norm_out, float* scale_out, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  const char* who = "rk_rmsnorm_tensor_scale";
  if (!x || !scale || !norm_out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || k < 1 || tokens < 0 || (tokens > 0 && rows % tokens != 0))
    return fail(RK_EINVAL, "%s: bad row / token counts", who);
  if (k > kCachedK) return fail(RK_EUNSUPPORTED, "%s: k > %d", who, kCachedK);
  if (!aligned16(x) || !aligned16(scale) || !aligned16(norm_out) || (residual && !aligned16(residual)) ||
      (shift && !aligned16(shift)) || (sum_out && !aligned16(sum_out)))
    return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  unsigned* staging = nullptr;
  if (scale_out != nullptr) {
    if (!(divisor > 0.0f)) return fail(RK_EINVAL, "%s: the divisor must be positive", who);
    if (!workspace || workspace_bytes < RK_WORKSPACE_HEADER) return fail(RK_EWORKSPACE, "%s: workspace too small", who);
    staging = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(workspace) + 64);  // zero between calls
  }
  auto b = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  launch_pdl(rmsnorm_quant_rows_kernel<16>, static_cast<unsigned>(rows), kRowThreads, as_stream(stream), 
      b(x), b(residual), nullptr, b(scale), b(shift), static_cast<int>(tokens), static_cast<int>(k), 0, eps,
      static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(norm_out), reinterpret_cast<uint8_t*>(staging), nullptr);
  if (staging != nullptr) launch_pdl(finalize_scale_kernel, 1, 1, as_stream(stream), staging, divisor, scale_out);
  return check_launch(who);
}

extern "C" int rk_lut_mul_tensor_scale(const void* x, int64_t x_stride, const void* up, int64_t up_stride,
                                       const void* lut, int64_t rows, int64_t k, float divisor, void* out,
                                       float* scale_out, void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "rk_lut_mul_tensor_scale";
  if (!x || !up || !lut || !out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || k < 8 || k % 8 != 0 || k > (1 << 30)) return fail(RK_EINVAL, "%s: rows >= 1 and k a multiple of 8", who);
  if (x_stride < k || up_stride < k || x_stride % 8 != 0 || up_stride % 8 != 0)
    return fail(RK_EINVAL, "%s: row strides must be multiples of 8 and >= k", who);
  if (!aligned16(x) || !aligned16(up) || !aligned16(out)) return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  unsigned* staging = nullptr;
  if (scale_out != nullptr) {
    if (!(divisor > 0.0f)) return fail(RK_EINVAL, "%s: the divisor must be positive", who);
    if (!workspace || workspace_bytes < RK_WORKSPACE_HEADER) return fail(RK_EWORKSPACE, "%s: workspace too small", who);
    staging = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(workspace) + 64);  // zero between calls
  }
  const long long vectors = rows * (k / 8);
  const unsigned blocks = static_cast<unsigned>(std::min<long long>((vectors + 255) / 256, 148LL * 8));
  auto b = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  launch_pdl(lut_mul_amax_kernel, blocks, 256, as_stream(stream), b(x), x_stride, b(up), up_stride, b(lut), rows,
                                                             static_cast<int>(k), static_cast<__nv_bfloat16*>(out), staging);
  if (staging != nullptr) launch_pdl(finalize_scale_kernel, 1, 1, as_stream(stream), staging, divisor, scale_out);
  return check_launch(who);
}

extern "C" int rk_pack_w4_g128(const void* w, int64_t n, int64_t k, void* q, void* scales, void* stream) {
  if (!w || !q || !scales) return fail(RK_EINVAL, "rk_pack_w4_g128: null pointer");
  if (n < 1 || k < 128 || k % 128 != 0) return fail(RK_EINVAL, "rk_pack_w4_g128: k must be a positive multiple of 128");
  if (!aligned16(w)) return fail(RK_EINVAL, "rk_pack_w4_g128: w must be 16-byte aligned");
  const long long warps = static_cast<long long>(n) * (k / 128);
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  launch_pdl(pack_w4_g128_kernel, blocks, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(w), static_cast<int>(n),
                                                             static_cast<int>(k), static_cast<uint8_t*>(q),
                                                             static_cast<__nv_bfloat16*>(scales));
  return check_launch("pack_w4_g128");
}

namespace {
int tensor_amax_scale(const void* x, int64_t elements, float divisor, float* scale_out, void* workspace,
                      size_t workspace_bytes, cudaStream_t st, const char* who) {
  if (!x || !scale_out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (!workspace || workspace_bytes < RK_WORKSPACE_HEADER) return fail(RK_EWORKSPACE, "%s: workspace too small", who);
  if (elements < 1 || !aligned16(x)) return fail(RK_EINVAL, "%s: bad size or alignment", who);
  unsigned* staging = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(workspace) + 64);
  long long blocks = (elements + 2047) / 2048;
  if (blocks > 1184) blocks = 1184;  // 148 SMs x 8 CTAs
  launch_pdl(amax_finite_kernel, static_cast<unsigned>(blocks), 256, st, static_cast<const __nv_bfloat16*>(x), elements,
                                                                    staging);
  launch_pdl(finalize_scale_kernel, 1, 1, st, staging, divisor, scale_out);
  return check_launch(who);
}
}  // namespace

extern "C" int rk_quant_tensor_fp8_with_scale(const void* x, int64_t elements, const float* scale, void* q,
                                              void* stream) {
  if (!x || !scale || !q) return fail(RK_EINVAL, "rk_quant_tensor_fp8_with_scale: null pointer");
  if (elements < 1 || !aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7u))
    return fail(RK_EINVAL, "rk_quant_tensor_fp8_with_scale: bad size or alignment");
  long long blocks = (elements + 2047) / 2048;
  if (blocks > 2368) blocks = 2368;
  launch_pdl(to_fp8_kernel, static_cast<unsigned>(blocks), 256, as_stream(stream), static_cast<const __nv_bfloat16*>(x),
                                                                              elements, scale, static_cast<uint8_t*>(q));
  return check_launch("to_fp8");
}

extern "C" int rk_quant_tensor_fp8(const void* x, int64_t elements, void* q, float* scale_out, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  int rc = tensor_amax_scale(x, elements, 448.0f, scale_out, workspace, workspace_bytes, as_stream(stream),
                             "rk_quant_tensor_fp8");
  if (rc != RK_OK) return rc;
  return rk_quant_tensor_fp8_with_scale(x, elements, scale_out, q, stream);
}

extern "C" int rk_nvfp4_global_scale(const void* x, int64_t elements, float* scale_out, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  return tensor_amax_scale(x, elements, 6.0f * 448.0f, scale_out, workspace, workspace_bytes, as_stream(stream),
                           "rk_nvfp4_global_scale");
}

extern "C" size_t rk_sf_bytes(int64_t rows, int64_t groups) {
  if (rows < 1 || groups < 1) return 0;
  return static_cast<size_t>(((rows + 127) / 128) * ((groups + 3) / 4) * 512);
}

extern "C" int rk_pack_mxfp8(const void* x, int64_t rows, int64_t k, void* q, void* sf, void* stream) {
  if (!x || !q || !sf) return fail(RK_EINVAL, "rk_pack_mxfp8: null pointer");
  if (rows < 1 || k < 32 || k % 32 != 0) return fail(RK_EINVAL, "rk_pack_mxfp8: k must be a positive multiple of 32");
  if (!aligned16(x) || !aligned16(q)) return fail(RK_EINVAL, "rk_pack_mxfp8: pointers must be 16-byte aligned");
  const long long blocks32 = ((rows + 127) / 128 * 128) * ((k + 127) / 128 * 4);
  const unsigned grid = static_cast<unsigned>((blocks32 * 8 + 255) / 256);
  launch_pdl(pack_mxfp8_kernel<false>, grid, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(x), rows, k,
             static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), nullptr);
  return check_launch("pack_mxfp8");
}

extern "C" int rk_swiglu_pack_mxfp8(const void* gate_up, int64_t rows, int64_t inter, const void* silu_table, void* q,
                                    void* sf, void* stream) {
  const char* who = "rk_swiglu_pack_mxfp8";
  if (!gate_up || !silu_table || !q || !sf) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || inter < 32 || inter % 32 != 0) return fail(RK_EINVAL, "%s: the intermediate size must be a positive multiple of 32", who);
  if (!aligned16(gate_up) || !aligned16(q)) return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  const long long blocks32 = ((rows + 127) / 128 * 128) * ((inter + 127) / 128 * 4);
  const unsigned grid = static_cast<unsigned>((blocks32 * 8 + 255) / 256);
  launch_pdl(pack_mxfp8_kernel<true>, grid, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(gate_up), rows, inter,
             static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), static_cast<const __nv_bfloat16*>(silu_table));
  return check_launch(who);
}

extern "C" int rk_pack_nvfp4(const void* x, int64_t rows, int64_t k, const float* global_scale, void* q, void* sf,
                             void* stream) {
  if (!x || !q || !sf) return fail(RK_EINVAL, "rk_pack_nvfp4: null pointer");
  if (rows < 1 || k < 32 || k % 32 != 0) return fail(RK_EINVAL, "rk_pack_nvfp4: k must be a positive multiple of 32");
  if (!aligned16(x) || !aligned16(q)) return fail(RK_EINVAL, "rk_pack_nvfp4: pointers must be 16-byte aligned");
  const long long threads = ((rows + 127) / 128 * 128) * ((k / 16 + 3) / 4 * 4);
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  launch_pdl(pack_nvfp4_kernel, grid, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(x), rows, k, global_scale,
                                                         static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf));
  return check_launch("pack_nvfp4");
}

extern "C" int rk_rmsnorm_quant_fp8(const void* x, const void* residual, const void* weight, int64_t rows, int64_t k,
                                    float eps, void* sum_out, void* norm_out, void* q, float* scale_out,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "rk_rmsnorm_quant_fp8";
  if (!x || !weight || !norm_out || !q || !scale_out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (!workspace || workspace_bytes < RK_WORKSPACE_HEADER) return fail(RK_EWORKSPACE, "%s: workspace too small", who);
  if (rows < 1 || k < 16 || k % 16 != 0 || k > rk::kCachedK) return fail(RK_EINVAL, "%s: k must be a multiple of 16, at most %d", who, rk::kCachedK);
  if (!aligned16(x) || !aligned16(weight) || (residual && !aligned16(residual)) || !aligned16(norm_out) ||
      (sum_out && !aligned16(sum_out)))
    return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  cudaStream_t st = as_stream(stream);
  unsigned* staging = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(workspace) + 64);
  auto b = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  launch_pdl(rk::rmsnorm_producer_kernel<0>, static_cast<unsigned>(rows), rk::kRowThreads, st, 
      b(x), b(residual), b(weight), static_cast<int>(rows), static_cast<int>(k), eps,
      static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(norm_out), staging, nullptr, nullptr);
  launch_pdl(rk::finalize_scale_kernel, 1, 1, st, staging, 448.0f, scale_out);
  int rc = check_launch(who);
  if (rc != RK_OK) return rc;
  return rk_quant_tensor_fp8_with_scale(norm_out, rows * k, scale_out, q, stream);
}

extern "C" int rk_swiglu_quant_fp8(const void* gate_up, int64_t rows, int64_t inter, const float* scale_in, void* q,
                                   float* scale_out, void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "rk_swiglu_quant_fp8";
  if (!gate_up || !q || (!scale_in && !scale_out)) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || inter < 16 || inter % 16 != 0) return fail(RK_EINVAL, "%s: the intermediate size must be a multiple of 16", who);
  if (!aligned16(gate_up) || (reinterpret_cast<uintptr_t>(q) & 7u)) return fail(RK_EINVAL, "%s: bad alignment", who);
  cudaStream_t st = as_stream(stream);
  const long long elements = rows * inter;
  long long blocks = (elements + 2047) / 2048;
  if (blocks > 2368) blocks = 2368;
  const float* scale = scale_in;
  if (scale_in == nullptr) {
    if (!workspace || workspace_bytes < RK_WORKSPACE_HEADER) return fail(RK_EWORKSPACE, "%s: workspace too small", who);
    unsigned* staging = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(workspace) + 64);
    launch_pdl(rk::swiglu_amax_kernel, static_cast<unsigned>(blocks > 1184 ? 1184 : blocks), 256, st, 
        static_cast<const __nv_bfloat16*>(gate_up), rows, inter, staging);
    launch_pdl(rk::finalize_scale_kernel, 1, 1, st, staging, 448.0f, scale_out);
    scale = scale_out;
  }
  launch_pdl(rk::swiglu_to_fp8_kernel, static_cast<unsigned>(blocks), 256, st, static_cast<const __nv_bfloat16*>(gate_up), rows,
                                                                          inter, scale, static_cast<uint8_t*>(q));
  return check_launch(who);
}

extern "C" int rk_rmsnorm_pack_nvfp4(const void* x, const void* residual, const void* weight, int64_t rows, int64_t k,
                                     float eps, void* sum_out, void* norm_out, void* q, void* sf, void* stream) {
  const char* who = "rk_rmsnorm_pack_nvfp4";
  if (!x || !weight || !q || !sf) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || k < 32 || k % 32 != 0 || k > rk::kCachedK) return fail(RK_EINVAL, "%s: k must be a multiple of 32, at most %d", who, rk::kCachedK);
  if (!aligned16(x) || !aligned16(weight) || (residual && !aligned16(residual)) || !aligned16(q) ||
      (sum_out && !aligned16(sum_out)) || (norm_out && !aligned16(norm_out)))
    return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  auto b = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  const unsigned rows_padded = static_cast<unsigned>((rows + 127) / 128 * 128);
  launch_pdl(rk::rmsnorm_producer_kernel<1>, rows_padded, rk::kRowThreads, as_stream(stream), 
      b(x), b(residual), b(weight), static_cast<int>(rows), static_cast<int>(k), eps,
      static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(norm_out), nullptr, static_cast<uint8_t*>(q),
      static_cast<uint8_t*>(sf));
  return check_launch(who);
}

extern "C" int rk_rmsnorm_bf16(const void* x, const void* residual, const void* weight, int64_t rows, int64_t k, float eps,
                               void* sum_out, void* norm_out, void* stream) {
  const char* who = "rk_rmsnorm_bf16";
  if (!x || !weight || !norm_out || (residual && !sum_out)) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || k < 16 || k % 16 != 0 || k > rk::kCachedK) return fail(RK_EINVAL, "%s: k must be a multiple of 16, at most %d", who, rk::kCachedK);
  if (!aligned16(x) || !aligned16(weight) || (residual && !aligned16(residual)) || !aligned16(norm_out) ||
      (sum_out && !aligned16(sum_out)))
    return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  auto b = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  launch_pdl(rk::rmsnorm_producer_kernel<2>, static_cast<unsigned>(rows), rk::kRowThreads, as_stream(stream),
             b(x), b(residual), b(weight), static_cast<int>(rows), static_cast<int>(k), eps,
             static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(norm_out), nullptr, nullptr, nullptr);
  return check_launch(who);
}

extern "C" int rk_silu_mul_bf16(const void* gate_up, int64_t rows, int64_t inter, int interleaved, void* out, void* stream) {
  const char* who = "rk_silu_mul_bf16";
  if (!gate_up || !out) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || inter < 8 || inter % 8 != 0) return fail(RK_EINVAL, "%s: the intermediate size must be a positive multiple of 8", who);
  if (interleaved && inter % 64 != 0) return fail(RK_EINVAL, "%s: the interleaved layout needs a multiple of 64 columns", who);
  if (!aligned16(gate_up) || !aligned16(out)) return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  const long long vectors = rows * inter / 8;
  const unsigned blocks = static_cast<unsigned>(std::min<long long>((vectors + 255) / 256, 148LL * 8));
  launch_pdl(rk::silu_mul_bf16_kernel, blocks, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(gate_up), rows, inter,
             interleaved, static_cast<__nv_bfloat16*>(out));
  return check_launch(who);
}

extern "C" int rk_swiglu_pack_nvfp4_layout(const void* gate_up, int64_t rows, int64_t inter, int interleaved, void* q,
                                           void* sf, void* stream) {
  const char* who = "rk_swiglu_pack_nvfp4";
  if (!gate_up || !q || !sf) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || inter < 32 || inter % 32 != 0) return fail(RK_EINVAL, "%s: the intermediate size must be a multiple of 32", who);
  if (interleaved && inter % 64 != 0) return fail(RK_EINVAL, "%s: the interleaved layout needs a multiple of 64 columns", who);
  if (!aligned16(gate_up) || !aligned16(q)) return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  const long long threads = ((rows + 127) / 128 * 128) * ((inter / 16 + 3) / 4 * 4);
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  launch_pdl(rk::swiglu_pack_nvfp4_kernel, grid, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(gate_up), rows, inter,
                                                                   interleaved ? 1 : 0, static_cast<uint8_t*>(q),
                                                                   static_cast<uint8_t*>(sf));
  return check_launch(who);
}

extern "C" int rk_swiglu_pack_nvfp4(const void* gate_up, int64_t rows, int64_t inter, void* q, void* sf, void* stream) {
  return rk_swiglu_pack_nvfp4_layout(gate_up, rows, inter, 0, q, sf, stream);
}

static int pack_mx_ceil(const void* x, int64_t rows, int64_t k, int fmt, void* q, void* sf, void* stream, const char* who) {
  if (!x || !q || !sf) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || k < 32 || k % 32 != 0) return fail(RK_EINVAL, "%s: k must be a positive multiple of 32", who);
  if (!aligned16(x) || !aligned16(q)) return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  const long long blocks32 = ((rows + 127) / 128 * 128) * ((k + 127) / 128 * 4);
  const unsigned grid = static_cast<unsigned>((blocks32 * 8 + 255) / 256);
  if (fmt == 0)
    launch_pdl(rk::pack_mx_ceil_kernel<0>, grid, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(x), rows, k,
                                                                   static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf));
  else
    launch_pdl(rk::pack_mx_ceil_kernel<1>, grid, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(x), rows, k,
                                                                   static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf));
  return check_launch(who);
}

extern "C" int rk_swiglu_pack_mxfp8_w4a8(const void* gate_up, int64_t rows, int64_t inter, int interleaved, void* q, void* sf,
                                         void* stream) {
  const char* who = "rk_swiglu_pack_mxfp8_w4a8";
  if (!gate_up || !q || !sf) return fail(RK_EINVAL, "%s: null pointer", who);
  if (rows < 1 || inter < 32 || inter % 32 != 0) return fail(RK_EINVAL, "%s: the intermediate size must be a multiple of 32", who);
  if (interleaved && inter % 64 != 0) return fail(RK_EINVAL, "%s: the interleaved layout needs a multiple of 64 columns", who);
  if (!aligned16(gate_up) || !aligned16(q)) return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  const long long blocks32 = ((rows + 127) / 128 * 128) * ((inter + 127) / 128 * 4);
  const unsigned grid = static_cast<unsigned>((blocks32 * 8 + 255) / 256);
  launch_pdl(rk::swiglu_pack_mxfp8_ceil_kernel, grid, 256, as_stream(stream), static_cast<const __nv_bfloat16*>(gate_up), rows, inter,
                                                                        interleaved ? 1 : 0, static_cast<uint8_t*>(q),
                                                                        static_cast<uint8_t*>(sf));
  return check_launch(who);
}

extern "C" int rk_pack_mxfp8_act_w4a8(const void* x, int64_t rows, int64_t k, void* q, void* sf, void* stream) {
  return pack_mx_ceil(x, rows, k, 0, q, sf, stream, "rk_pack_mxfp8_act_w4a8");
}

extern "C" int rk_pack_mxfp4_weight(const void* w, int64_t rows, int64_t k, void* q, void* sf, void* stream) {
  return pack_mx_ceil(w, rows, k, 1, q, sf, stream, "rk_pack_mxfp4_weight");
}

extern "C" int rk_probe_rcp_approx_448(uint32_t* bits) {
  if (!bits) return fail(RK_EINVAL, "rk_probe_rcp_approx_448: null pointer");
  uint32_t* d = nullptr;
  if (cudaMalloc(&d, 4) != cudaSuccess) return fail(RK_ECUDA, "rk_probe_rcp_approx_448: cudaMalloc failed");
  probe_rcp_kernel<<<1, 1>>>(d);
  cudaError_t e = cudaMemcpy(bits, d, 4, cudaMemcpyDeviceToHost);
  cudaFree(d);
  if (e != cudaSuccess) return fail(RK_ECUDA, "rk_probe_rcp_approx_448: %s", cudaGetErrorString(e));
  return RK_OK;
}
