// Host-side error text of the kernel library.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

int sprout_fail(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, args);
  va_end(args);
  return 1;
}

int sprout_check_launch(const char* what) {
  cudaError_t err = cudaPeekAtLastError();
  if (err != cudaSuccess) {
    cudaGetLastError();
    return sprout_fail("%s: %s", what, cudaGetErrorString(err));
  }
  return 0;
}

// Text of the last failure on the calling thread.
SPROUT_API const char* sprout_last_error() { return g_error; }

static int g_pdl = 1;
int sprout_pdl_enabled() { return g_pdl; }
// Turn programmatic dependent launch on (default) or off for all later launches.
SPROUT_API void sprout_set_pdl(int enabled) { g_pdl = enabled ? 1 : 0; }

SPROUT_API int sprout_sm_count() {
  static int counts[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) { cudaGetLastError(); return 148; }
  if (!counts[device]) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) { cudaGetLastError(); return 148; }
    counts[device] = count;
  }
  return counts[device];
}

// Version of the exported interface; the Python side checks it after loading.
SPROUT_API int sprout_abi_version() { return 5; }
