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

// Shared-memory carve-out that every launch asks for (percent of the SM's maximum; -1: the driver's
// choice per kernel).  An SM changes its split between shared memory and L1 only when it is empty, so
// neighbouring kernels that ask for different splits cannot overlap and pay for the change; a decode
// step is a chain of short kernels, and one split for the whole chain measured 3 % faster (batch 8)
// than the driver's per-kernel choices.  The environment variable HFEE_CARVE overrides every setting.
static int g_carveout = -1;
static int g_carveout_forced = -2;

int hfee_carveout() {
  if (g_carveout_forced == -2) {
    const char* e = getenv("HFEE_CARVE");
    g_carveout_forced = e ? atoi(e) : -1;
  }
  return g_carveout_forced >= 0 ? g_carveout_forced : g_carveout;
}

// percent in 0..100, or -1 for the driver's choice; returns the previous setting.
HFEE_API int hfee_set_carveout(int percent) {
  const int before = g_carveout;
  g_carveout = percent < 0 ? -1 : (percent > 100 ? 100 : percent);
  return before;
}

int hfee_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) enabled = getenv("HFEE_NO_PDL") == nullptr ? 1 : 0;
  return enabled;
}
