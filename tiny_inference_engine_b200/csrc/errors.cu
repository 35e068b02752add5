// The last error message of a launcher, per thread, and the library's version probe.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace tie {
static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("TIE_NO_PDL");
    return !(v != nullptr && v[0] == '1');
  }();
  return on;
}
}  // namespace tie

TIE_API const char* tie_last_error() { return tie::g_error; }

// The architecture this library was compiled for, so that Python can refuse another GPU loudly.
TIE_API int tie_compiled_arch() { return 100; }
