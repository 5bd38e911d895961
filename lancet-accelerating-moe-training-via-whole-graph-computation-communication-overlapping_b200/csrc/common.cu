#include "common.cuh"

namespace lancet {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
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

}  // namespace lancet

extern "C" {
const char* lancet_last_error(void) { return lancet::error_buffer(); }
const char* lancet_version(void) { return "lancet_b200 0.1 (sm_100a)"; }
int lancet_abi_version(void) { return 1; }
int lancet_moe_capacity(int S, int E, float capacity_factor, int k) {
  if (S < 0 || E <= 0 || k <= 0) return -1;
  // integer ceil-div, float multiply, truncate: src/op/declare/moe.cc:46 of the reference
  long long per = ((long long)k * S + E - 1) / E;
  return static_cast<int>(capacity_factor * static_cast<float>(per));
}
}
