#include "common.cuh"

#include <cstring>
#include <mutex>
#include <vector>

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

static unsigned long long g_launches = 0;
void count_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }
unsigned long long launches() { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

namespace {
struct Profiler {
  std::mutex mu;
  bool on = false;
  char pattern[64] = {0};
  std::vector<cudaEvent_t> events;  // pairs: before, after
  size_t used = 0;
};
Profiler& prof() {
  static Profiler p;
  return p;
}
}  // namespace

bool prof_enabled_for(const char* name) {
  Profiler& p = prof();
  if (!p.on) return false;
  return std::strstr(name, p.pattern) != nullptr;
}

void prof_record(cudaStream_t stream, bool after) {
  Profiler& p = prof();
  std::lock_guard<std::mutex> lk(p.mu);
  if (!after && (p.used & 1)) return;  // unbalanced: ignore
  if (p.used >= p.events.size()) {
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    p.events.push_back(e);
  }
  cudaEventRecord(p.events[p.used++], stream);
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

static int g_exchange_ctas = 0, g_gemm_ctas = 0, g_gemm_paired = 1, g_chained = 1;
bool chained_launch_enabled() { return __atomic_load_n(&g_chained, __ATOMIC_RELAXED) != 0; }
bool gemm_paired_enabled() { return (__atomic_load_n(&g_gemm_paired, __ATOMIC_RELAXED) & 1) != 0; }
int gemm_option(int bit) { return (__atomic_load_n(&g_gemm_paired, __ATOMIC_RELAXED) >> bit) & 1; }
int exchange_cta_limit() { return __atomic_load_n(&g_exchange_ctas, __ATOMIC_RELAXED); }
int gemm_cta_limit() { return __atomic_load_n(&g_gemm_ctas, __ATOMIC_RELAXED); }

}  // namespace lancet

extern "C" {
int lancet_set_cta_limits(int exchange_ctas, int gemm_ctas) {
  if (exchange_ctas < 0 || gemm_ctas < 0) return lancet::fail(LANCET_ERR_INVALID, "lancet_set_cta_limits: negative limit");
  __atomic_store_n(&lancet::g_exchange_ctas, exchange_ctas, __ATOMIC_RELAXED);
  __atomic_store_n(&lancet::g_gemm_ctas, gemm_ctas, __ATOMIC_RELAXED);
  return LANCET_OK;
}

int lancet_set_chained_launch(int on) {
  __atomic_store_n(&lancet::g_chained, on ? 1 : 0, __ATOMIC_RELAXED);
  return LANCET_OK;
}

int lancet_set_gemm_paired(int on) {
  __atomic_store_n(&lancet::g_gemm_paired, on, __ATOMIC_RELAXED);
  return LANCET_OK;
}

int lancet_peer_copy(void* dst, const void* src, size_t bytes, lancet_stream_t stream) {
  if (bytes == 0) return LANCET_OK;
  if (!dst || !src) return lancet::fail(LANCET_ERR_NULL, "lancet_peer_copy: null pointer");
  LANCET_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
  return LANCET_OK;
}

const char* lancet_last_error(void) { return lancet::error_buffer(); }
const char* lancet_version(void) { return "lancet_b200 0.1 (sm_100a)"; }
int lancet_abi_version(void) { return 1; }
unsigned long long lancet_launch_count(void) { return lancet::launches(); }

int lancet_profile_begin(const char* kernel_substr) {
  if (!kernel_substr || !*kernel_substr) return lancet::fail(LANCET_ERR_NULL, "lancet_profile_begin: empty pattern");
  lancet::Profiler& p = lancet::prof();
  std::lock_guard<std::mutex> lk(p.mu);
  std::strncpy(p.pattern, kernel_substr, sizeof(p.pattern) - 1);
  p.used = 0;
  p.on = true;
  return LANCET_OK;
}

int lancet_profile_end(double* total_ms, long long* launches) {
  lancet::Profiler& p = lancet::prof();
  std::lock_guard<std::mutex> lk(p.mu);
  p.on = false;
  double tot = 0;
  long long n = 0;
  for (size_t i = 0; i + 1 < p.used; i += 2) {
    cudaError_t e = cudaEventSynchronize(p.events[i + 1]);
    if (e != cudaSuccess) return lancet::fail(LANCET_ERR_CUDA, "lancet_profile_end: %s", cudaGetErrorString(e));
    float ms = 0;
    e = cudaEventElapsedTime(&ms, p.events[i], p.events[i + 1]);
    if (e != cudaSuccess) return lancet::fail(LANCET_ERR_CUDA, "lancet_profile_end: %s", cudaGetErrorString(e));
    tot += ms;
    ++n;
  }
  p.used = 0;
  if (total_ms) *total_ms = tot;
  if (launches) *launches = n;
  return LANCET_OK;
}
int lancet_moe_capacity(int S, int E, float capacity_factor, int k) {
  if (S < 0 || E <= 0 || k <= 0) return -1;
  // integer ceil-div, float multiply, truncate: src/op/declare/moe.cc:46 of the reference
  long long per = ((long long)k * S + E - 1) / E;
  return static_cast<int>(capacity_factor * static_cast<float>(per));
}
}
