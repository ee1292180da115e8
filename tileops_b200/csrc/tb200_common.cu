// Host-side plumbing shared by every entry point: per-thread error text, device facts.
#include "tb200_common.cuh"

namespace tb200 {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace tb200

extern "C" const char* tb200_last_error(void) { return tb200::error_buffer(); }
extern "C" int tb200_version(void) { return 102; }  // 1.02: prefill entry points take window sizes; paged prefill, RoPE and FP8-cache entry points
