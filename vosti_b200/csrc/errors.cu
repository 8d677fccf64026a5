// Last-error text of the launchers (thread-local), and the library's version probe.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void vosti_set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

VOSTI_API const char* vosti_last_error() { return g_error; }

// The compute capability this library was compiled for; the loader refuses to run
// it on anything else.
VOSTI_API int vosti_built_for_sm() { return 100; }

VOSTI_API int vosti_device_sm(int device) {
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return -1;
  return prop.major * 10 + prop.minor;
}
