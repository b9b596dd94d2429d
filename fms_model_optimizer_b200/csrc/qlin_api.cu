// Library-level entry points of libqlin_b200.so: version, error text, device query.
#include <cstring>

#include "qlin_internal.h"

namespace qlin {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace qlin

extern "C" int qlin_version(void) { return QLIN_VERSION; }

extern "C" const char* qlin_last_error_string(void) { return qlin::g_err; }

extern "C" int qlin_device_supported(int device) {
  int major = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) return qlin::fail(QLIN_ERR_DEVICE, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
  return major == 10 ? 1 : 0;
}
