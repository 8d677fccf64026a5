// Last-error text of the launchers (thread-local), and the library's version probe.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

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

// Dependent launches (see common.cuh) are on unless VOSTI_PDL=0 is set or they are switched
// off through vosti_set_pdl.
static int g_pdl = -1;

int vosti_pdl_enabled() {
  if (g_pdl < 0) {
    const char* env = getenv("VOSTI_PDL");
    g_pdl = (env != nullptr && env[0] == '0') ? 0 : 1;
  }
  return g_pdl;
}

VOSTI_API void vosti_set_pdl(int enabled) { g_pdl = enabled ? 1 : 0; }

// One order of arithmetic for every way of cutting the work (vosti_set_fixed_order): a product
// never splits its K range, and no kernel is chosen by the number of tokens in the launch, so a
// token's values are the same bits whether it comes alone, in a batch or inside a long portion.
int g_vosti_fixed_order = 0;

VOSTI_API void vosti_set_fixed_order(int enabled) { g_vosti_fixed_order = enabled ? 1 : 0; }
VOSTI_API int vosti_fixed_order() { return g_vosti_fixed_order; }

// The weight range the next product will stream (see common.cuh): set by the host just before it
// launches a kernel that can request it into L2, taken by that kernel's launcher. bytes 0 or a
// null pointer clears the hint.
static thread_local VostiPrefetch g_prefetch = {nullptr, 0};

VOSTI_API int vosti_hint_prefetch(const void* ptr, long long bytes) {
  g_prefetch = {nullptr, 0};
  if (ptr == nullptr || bytes < 16) return VOSTI_OK;
  VOSTI_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "hint_prefetch: the range must start on a 16-byte boundary");
  g_prefetch.ptr = (const char*)ptr;
  g_prefetch.bytes = bytes & ~15ll;
  return VOSTI_OK;
}

VostiPrefetch vosti_take_prefetch() {
  const VostiPrefetch taken = g_prefetch;
  g_prefetch = {nullptr, 0};
  return taken;
}
