// Process-wide pieces of libsoup_b200: version, the thread-local error string, cached device facts.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace soup {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  // Cached per device ordinal; a wrong value only changes a grid size, never correctness.
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace soup

extern "C" int soup_version(void) { return 1; }

extern "C" const char* soup_last_error_string(void) { return soup::g_error; }
