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
