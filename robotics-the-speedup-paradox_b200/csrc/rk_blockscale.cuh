// Device helpers shared by the packers (rk_quant.cu) and by GEMM epilogues that re-quantize their
// output: the 128 x 4 scale-factor layout, one NVFP4 block, SwiGLU in the reference's bf16 steps.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace rk {
namespace {

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// byte offset of the factor of (row, group) in the swizzled scale-factor buffer; kt = 512-byte chunks per 128-row block
__device__ __forceinline__ long long sf_offset(long long row, long long group, long long kt) {
  return ((row / 128) * kt + group / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + group % 4;
}

__device__ __forceinline__ float rcp_approx_ftz(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// smallest power of two >= x as a biased exponent byte (x >= 0, finite)
__device__ __forceinline__ uint32_t ue8m0_roundup(float x) {
  const uint32_t b = __float_as_uint(x);
  const uint32_t e = (b >> 23) & 0xFFu, mant = b & 0x7FFFFFu;
  uint32_t r = e == 0 ? (mant > 0x400000u ? 1u : 0u) : e + (mant != 0u ? 1u : 0u);
  return r > 254u ? 254u : r;
}

// MXFP8 block of 32 (blackwell/csrc/mxfp8_common.cuh:12-32): the UE8M0 scale byte of a block with absolute
// maximum `amax` (255 when the block holds a non-finite value), and the multiplier 2^(127 - e) that goes with it,
// built as the exponent byte 254 - e (255 stays NaN, 0 becomes the subnormal 2^-127).
__device__ __forceinline__ uint32_t mxfp8_block_scale(float amax, bool invalid) {
  return invalid ? 255u : ue8m0_roundup(__fmul_rn(amax, rcp_approx_ftz(448.0f)));
}
__device__ __forceinline__ float mxfp8_inverse_scale(uint32_t e) {
  const uint32_t ie = (254u - e) & 255u;
  return ie == 255u ? __uint_as_float(0x7FC00000u) : (ie == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(ie << 23));
}

// SwiGLU in bf16 steps, as the reference's NVFP4 producer evaluates it with packed bf16 arithmetic
// (blackwell/csrc/fp4_cutlass_linear.cu:1029-1033): every intermediate is rounded to bf16.
__device__ __forceinline__ float swiglu_bf16_steps(float gate, float up) {
  const float e = round_bf16(expf(-gate));
  const float d = round_bf16(__fadd_rn(1.0f, e));
  const float r = round_bf16(__frcp_rn(d));  // the correctly rounded reciprocal: what 1 / d gives
  return round_bf16(__fmul_rn(round_bf16(__fmul_rn(gate, r)), up));
}

// One 16-element NVFP4 block: UE4M3 scale byte and eight code bytes (two E2M1 codes each, low nibble first).
// Same arithmetic as pack_nvfp4_kernel (blackwell/csrc/fp4_cutlass_linear.cu:789-841, no per-tensor scale).
__device__ __forceinline__ unsigned long long nvfp4_block(const float (&v)[16], uint8_t* code_out) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float scale = amax > 0.0f ? __fdiv_rn(amax, 6.0f) : 1.0f;
  const uint8_t code = static_cast<uint8_t>(__nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E4M3)) & 0x7F;
  float deq = __half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3)));
  if (!(deq > 0.0f)) deq = scale;
  const float reciprocal = __frcp_rn(deq);  // == 1 / deq, correctly rounded
  unsigned long long packed = 0;
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const __nv_fp4x2_storage_t pair = __nv_cvt_float2_to_fp4x2(
        make_float2(__fmul_rn(v[i], reciprocal), __fmul_rn(v[i + 1], reciprocal)), __NV_E2M1, cudaRoundNearest);
    packed |= static_cast<unsigned long long>(static_cast<uint8_t>(pair)) << (4 * i);
  }
  *code_out = code;
  return packed;
}

}  // namespace
}  // namespace rk
