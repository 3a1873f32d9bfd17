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

// The number of SMs of the current device, asked once per device. Grids and split rules are
// sized from it; 148 (a B200) only if the device cannot be asked.
int b200_sm_count_host() {
  constexpr int kMaxDevices = 64;
  static int known[kMaxDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    cudaGetLastError();
    return 148;
  }
  if (known[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) {
      cudaGetLastError();
      return 148;
    }
    known[device] = count;
  }
  return known[device];
}

B200_API int b200_sm_count() { return b200_sm_count_host(); }

B200_API const char* b200_last_error() { return g_error; }

B200_API int b200_abi_version() { return 1; }
