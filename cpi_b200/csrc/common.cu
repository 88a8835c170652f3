// Error reporting shared by every entry point of the library.
#include "common.cuh"
#include <cstring>

namespace cpi {
static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static long g_launches = 0;
void count_launch() { ++g_launches; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 1; }
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) { cudaGetLastError(); n = 1; }
    cached[dev] = n;
  }
  return cached[dev];
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 2;
  }
  return 0;
}
}  // namespace cpi

// Kernels launched by this library from host code since it was loaded (replays of a captured graph are
// not host launches and are not counted here).
extern "C" long cpi_launch_count() { return cpi::g_launches; }

extern "C" int cpi_sm_count() { return cpi::sm_count(); }

extern "C" const char* cpi_last_error() { return cpi::g_error; }

// The calling convention of this library's entry points; the loader refuses a library that answers another number.
extern "C" int cpi_abi_version() { return 1; }
