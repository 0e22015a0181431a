// TEST INFRASTRUCTURE ONLY - part of the oracle, never linked into the shipped library.
//
// Thin C shim over the number-format conversions the reference itself calls when it packs FP8,
// MXFP8 and NVFP4 operands, compiled for the HOST from the headers where they lie in the reference
// tree (its vendored CUTLASS 4.4.2 under src/robotics_kernels/ampere_ada/third_party/cutlass, the
// CUDA toolkit's cuda_fp8.h, and its own blackwell/csrc/mxfp8_common.cuh).  The numpy restatement
// in oracle/formats.py and oracle/blockscale.py is checked against these functions.
//
// Call sites being mirrored (reference paths):
//   blackwell/csrc/fp8_cutlass_linear.cu:99,133   __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3)
//   blackwell/csrc/mxfp8_cutlass_linear.cu:77     cutlass::NumericArrayConverter<float_e4m3_t, float, 4>
//                                                 (device-only; its scalar fallback is bound here)
//   blackwell/csrc/mxfp8_common.cuh:24-27         cutlass::NumericConverter<float_ue8m0_t, float>
//   blackwell/csrc/mxfp8_common.cuh:29-32         inverse scale = bitcast(254 - raw)
//   blackwell/csrc/mxfp8_common.cuh:18-22         scale_offset(row, group, k_tiles)
//   blackwell/csrc/fp4_cutlass_linear.cu:742,822  cutlass::float_e2m1_t(float), cutlass::float_ue4m3_t(float)
//
// Built by oracle/build_ref.py into oracle/_ref/ (never committed).

#include <cstdint>
#include <cuda_fp8.h>

#include "cutlass/array.h"
#include "cutlass/float8.h"
#include "cutlass/float_subbyte.h"
#include "cutlass/numeric_conversion.h"
#include "mxfp8_common.cuh"  // the reference's own header: scale_offset, SF

extern "C" {

// per-tensor FP8 path: the toolkit conversion the reference calls
void ref_nv_e4m3(const float* x, int64_t n, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = __nv_cvt_float_to_fp8(x[i], __NV_SATFINITE, __NV_E4M3);
}

// MXFP8 element conversion.  The reference converts four values at a time with a converter that
// only exists on the device; its portable branch is this scalar converter applied per element
// (cutlass/numeric_conversion.h, "Array<float_e4m3_t, 4> <= Array<float, 4>").
void ref_cutlass_e4m3(const float* x, int64_t n, uint8_t* out) {
  cutlass::NumericConverter<cutlass::float_e4m3_t, float> convert;
  for (int64_t i = 0; i < n; ++i) out[i] = convert(x[i]).raw();
}

// block scale of MXFP8 from (amax * multiplier): the caller supplies the product, because the
// multiplier is a device-only approximate reciprocal
void ref_cutlass_ue8m0(const float* x, int64_t n, uint8_t* out) {
  cutlass::NumericConverter<SF, float> convert;
  for (int64_t i = 0; i < n; ++i) out[i] = convert(x[i]).raw();
}

// value of the "inverse" scale the reference multiplies elements by
void ref_cutlass_ue8m0_inverse(const uint8_t* code, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) {
    SF inverse = SF::bitcast(static_cast<uint8_t>(254 - code[i]));
    out[i] = static_cast<float>(inverse);
  }
}

void ref_cutlass_ue8m0_value(const uint8_t* code, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = static_cast<float>(SF::bitcast(code[i]));
}

void ref_cutlass_e2m1(const float* x, int64_t n, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) {
    cutlass::float_e2m1_t q(x[i]);
    out[i] = static_cast<uint8_t>(q.raw() & 0xF);
  }
}

void ref_cutlass_e2m1_value(const uint8_t* code, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i)
    out[i] = static_cast<float>(cutlass::float_e2m1_t::bitcast(static_cast<uint8_t>(code[i] & 0xF)));
}

void ref_cutlass_ue4m3(const float* x, int64_t n, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) {
    cutlass::float_ue4m3_t s(x[i]);
    out[i] = s.raw();
  }
}

void ref_cutlass_ue4m3_value(const uint8_t* code, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = static_cast<float>(cutlass::float_ue4m3_t::bitcast(code[i]));
}

void ref_cutlass_e4m3_value(const uint8_t* code, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = static_cast<float>(cutlass::float_e4m3_t::bitcast(code[i]));
}

int64_t ref_scale_offset(int64_t row, int64_t group, int64_t k_tiles) { return scale_offset(row, group, k_tiles); }

int64_t ref_scale_storage_size(int64_t rows, int64_t columns) { return scale_storage_size(rows, columns); }

}  // extern "C"
