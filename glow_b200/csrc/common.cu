#include "common.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>

namespace glowb200 {

char *last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int set_error(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

std::atomic<int> g_pdl_override{-1};  // -1: the environment decides

bool pdl_enabled() {
  const int o = g_pdl_override.load(std::memory_order_relaxed);
  if (o >= 0) return o != 0;
  static const bool on = [] {
    const char *e = getenv("GLOWB200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace glowb200

extern "C" const char *glowb200_last_error(void) { return glowb200::last_error_buffer(); }
extern "C" const char *glowb200_version(void) { return "glow_b200 0.1 (sm_100a)"; }
extern "C" int glowb200_set_programmatic_launch(int enabled) {
  const bool before = glowb200::pdl_enabled();
  glowb200::g_pdl_override.store(enabled < 0 ? -1 : (enabled != 0), std::memory_order_relaxed);
  return before ? 1 : 0;
}
