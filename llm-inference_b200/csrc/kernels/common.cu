#include "common.cuh"

#include <cstring>

static thread_local char g_error[1024] = "";

int b200_fail(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return -1;
}

int b200_check_launch(const char* what) {
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return b200_fail("%s: %s", what, cudaGetErrorString(status));
  return 0;
}

static bool g_overlap = true;

bool b200_overlap_enabled() { return g_overlap; }

// Switches programmatic dependent launch (kernels overlapping their predecessor's tail) on or
// off for every later launch of this library.
B200_API void b200_set_overlap(int enabled) { g_overlap = enabled != 0; }

B200_API const char* b200_last_error() { return g_error; }

B200_API int b200_abi_version() { return 1; }
