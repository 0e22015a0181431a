// Library-level entry points: version, device support, per-thread error text.

#include <cstring>

#include "rk_host.h"

namespace rk {
namespace {
thread_local char g_error[512] = "";
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_error[0] = '\0'; }

}  // namespace rk

extern "C" int rk_version(void) { return 1000; }

extern "C" const char* rk_last_error_string(void) { return rk::g_error; }

extern "C" int rk_supports_device(int cc_major, int cc_minor) { return (cc_major == 10 && cc_minor == 0) ? 1 : 0; }

// ------------------------------------------------------------------ exchange memory shared between the GPUs of a node
// Device memory that the other processes of a node map into their own address space, for the
// column-parallel GEMM whose epilogue stores into every rank's output buffer.  Plain CUDA runtime
// inter-process handles; the opening side maps the memory with its own device current, which is
// what makes the mapping usable by kernels running on that device (peer access is switched on by
// the runtime as part of the open).
extern "C" int rk_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  const char* who = "rk_peer_alloc";
  if (!ptr || !handle64 || bytes == 0) return rk::fail(RK_EINVAL, "%s: null pointer or zero size", who);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "inter-process handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    cudaGetLastError();
    return rk::fail(RK_ECUDA, "%s: %s", who, cudaGetErrorString(e));
  }
  std::memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return RK_OK;
}

extern "C" int rk_peer_open(const void* handle64, int owner_device, void** ptr) {
  const char* who = "rk_peer_open";
  if (!handle64 || !ptr) return rk::fail(RK_EINVAL, "%s: null pointer", who);
  int dev = 0, can = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && owner_device != dev) e = cudaDeviceCanAccessPeer(&can, dev, owner_device);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return rk::fail(RK_ECUDA, "%s: %s", who, cudaGetErrorString(e));
  }
  if (owner_device != dev && !can)
    return rk::fail(RK_EUNSUPPORTED, "%s: device %d cannot address the memory of device %d", who, dev, owner_device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e == cudaSuccess) {
    // prove that the mapping answers from this device before any kernel is pointed at it
    unsigned probe = 0;
    e = cudaMemcpy(&probe, p, sizeof(probe), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) cudaIpcCloseMemHandle(p);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return rk::fail(RK_ECUDA, "%s: %s", who, cudaGetErrorString(e));
  }
  *ptr = p;
  return RK_OK;
}

extern "C" int rk_peer_close(void* ptr) {
  if (!ptr) return RK_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return rk::fail(RK_ECUDA, "rk_peer_close: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}

extern "C" int rk_peer_free(void* ptr) {
  if (!ptr) return RK_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return rk::fail(RK_ECUDA, "rk_peer_free: %s", cudaGetErrorString(e));
  }
  return RK_OK;
}
