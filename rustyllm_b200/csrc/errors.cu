// Error text of the last failed call, per host thread, and library identity.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_last_error[1024] = "";

void rl_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

extern "C" const char* rl_last_error() { return g_last_error; }

extern "C" int rl_page_size() { return RL_PAGE; }

// Compute capability of the current device as major*10+minor, or a negative code.
extern "C" int rl_device_arch() {
  int dev = 0, major = 0, minor = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RL_ERR_CUDA;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return RL_ERR_CUDA;
  if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return RL_ERR_CUDA;
  return major * 10 + minor;
}

// Number of SMs of the current device, asked once per device; grids and the choice of split
// counts are sized by it.  Without a device (a build machine), the B200's 148.
int rl_num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); return 148; }
    cached[dev] = n;
  }
  return cached[dev];
}

extern "C" int rl_sm_count() { return rl_num_sms(); }

int g_rl_pdl_enabled = 1;

// Switch programmatic dependent launch on (1, default) or off (0) for all later launches.
extern "C" void rl_set_pdl(int enabled) { g_rl_pdl_enabled = enabled ? 1 : 0; }
