// Launch bookkeeping shared by all launchers: the last CUDA error as text, and a
// device query used at start-up to refuse anything that is not an sm_100 part.
#include "common.cuh"

#include <stdio.h>
#include <string.h>

static thread_local char g_last_error[512] = "";

int iert_pdl_enabled = 1;

// Programmatic dependent launch on (1, default) or off (0) for every later launch.
IERT_API void iert_set_pdl(int on) { iert_pdl_enabled = on ? 1 : 0; }

int iert_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return IERT_OK;
  snprintf(g_last_error, sizeof g_last_error, "%s: %s", what, cudaGetErrorString(e));
  return IERT_CUDA_ERROR;
}

IERT_API const char* iert_last_cuda_error() { return g_last_error; }

// Compute capability of the current device as major*10+minor, or a negative CUDA error.
IERT_API int iert_device_arch() {
  int dev = 0, major = 0, minor = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  if (e != cudaSuccess) {
    snprintf(g_last_error, sizeof g_last_error, "device query: %s", cudaGetErrorString(e));
    return -(int)e;
  }
  return major * 10 + minor;
}

// The SM count of the current device, asked once (grids of grid-stride kernels are sized by it).
int iert_sm_count_cached() {
  static int n = 0;
  if (n <= 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
      n = v;
    else
      return 1;
  }
  return n;
}

IERT_API int iert_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}
