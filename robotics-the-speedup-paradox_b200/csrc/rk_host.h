// Host-side helpers shared by the C-ABI translation units: error reporting and stream casts.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/rk_b200.h"

namespace rk {

// Records a formatted message for rk_last_error_string() on this thread and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(RK_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  }
  return RK_OK;
}

// rk_quant.cu: scale = max(staged maximum / divisor, 1e-12) from the staging word of a workspace header
// (cleared for the next call); for entry points of other translation units whose kernels collect a maximum.
int launch_finalize_scale(unsigned* staging, float divisor, float* scale_out, cudaStream_t stream);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t round_up(int64_t v, int64_t q) { return (v + q - 1) / q * q; }

}  // namespace rk
