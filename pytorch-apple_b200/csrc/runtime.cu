// Library-wide host helpers: thread-local error string, device queries.
#include <stdarg.h>
#include <stdlib.h>

#include "common.cuh"

namespace b200 {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static int cached[64] = {0};
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
  static int state = -1;
  if (state < 0) {
    const char* e = getenv("B200NN_PDL");
    state = (e && e[0] == '0') ? 0 : 1;
  }
  return state == 1;
}

}  // namespace b200

extern "C" int b200_version(void) { return B200NN_VERSION; }

extern "C" const char* b200_last_error(void) { return b200::g_err; }

extern "C" int b200_device_info(int dev, int* sm_count, int* cc_major, int* cc_minor, int64_t* smem_optin_bytes) {
  int v = 0;
  cudaError_t e;
  if ((e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
    B200_FAIL(B200_ELAUNCH, "b200_device_info: %s", cudaGetErrorString(e));
  if (sm_count) *sm_count = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev);
  if (cc_major) *cc_major = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, dev);
  if (cc_minor) *cc_minor = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (smem_optin_bytes) *smem_optin_bytes = v;
  return B200_OK;
}
