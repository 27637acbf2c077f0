// Error reporting and small host-side helpers of the kernel library.
#include "common.cuh"
#include <stdarg.h>
#include <stdlib.h>

static thread_local char g_error[512] = "";

int hfee_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int hfee_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return HFEE_OK;
}

HFEE_API const char* hfee_last_error() { return g_error; }

// 1 if the current device is compute capability 10.x (the only target of this library).
HFEE_API int hfee_device_is_sm100() {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
  return major == 10;
}

// Streaming multiprocessors of the current device (asked once per device); 0 if the query fails.
HFEE_API int hfee_sm_count() {
  static int cached[64] = {0};
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 0;
  if (dev >= 0 && dev < 64) cached[dev] = sms;
  return sms;
}

int hfee_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) enabled = getenv("HFEE_NO_PDL") == nullptr ? 1 : 0;
  return enabled;
}
