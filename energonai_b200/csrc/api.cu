// Error reporting and device queries behind the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace eb {

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char *what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();   // clear the non-sticky launch error so later calls are not poisoned
    return fail(EB_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  }
  return EB_OK;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool pdl_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char *e = getenv("EB_PDL");
    cached = (e && e[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

}  // namespace eb

extern "C" int eb_version(void) { return 100; }
extern "C" const char *eb_last_error(void) { return eb::g_err; }
