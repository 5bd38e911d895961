// Shared host/device helpers of the C-ABI layer: status codes, the thread-local error text,
// dtype dispatch and small device utilities.
#pragma once
#include <utility>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/lancet_b200.h"

namespace lancet {

char* error_buffer();  // thread-local, 512 bytes
int fail(int code, const char* fmt, ...);

#define LANCET_REQUIRE(cond, code, ...)                 \
  do {                                                  \
    if (!(cond)) return ::lancet::fail(code, __VA_ARGS__); \
  } while (0)

#define LANCET_CUDA(expr)                                                                    \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess)                                                                   \
      return ::lancet::fail(LANCET_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

void count_launch();

// Optional per-kernel timing with CUDA events on the launching stream (see lancet_profile_begin).
// A ProfScope placed around a launch records an event pair when the kernel name matches the
// selected pattern; otherwise it costs one branch.
bool prof_enabled_for(const char* name);
void prof_record(cudaStream_t stream, bool after);
struct ProfScope {
  cudaStream_t s;
  bool on;
  ProfScope(const char* name, cudaStream_t stream) : s(stream), on(prof_enabled_for(name)) {
    if (on) prof_record(s, false);
  }
  ~ProfScope() {
    if (on) prof_record(s, true);
  }
};

inline int launch_status(const char* what) {
  count_launch();
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LANCET_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  }
  return LANCET_OK;
}

// Chains of short dependent kernels (gate -> slot assignment -> scatter -> combine) are launched with programmatic
// stream serialization: the CTAs of the next kernel may become resident while the last CTAs of the previous one drain,
// and wait in chain_enter() until that kernel has completed and its writes are visible.  Only the launch latency and the
// drain overlap; nothing a chained kernel reads or writes is touched before the wait.  Every kernel launched this way
// calls chain_enter() first, so completion is transitive along the chain; after a kernel that never releases its
// dependents (any other kernel) the launch behaves like a plain one.  lancet_set_chained_launch(0) switches it off.
bool chained_launch_enabled();
__device__ __forceinline__ void chain_enter() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename... KArgs, typename... Args>
inline void launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = chained_launch_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

inline bool valid_dtype(int d) { return d == LANCET_F32 || d == LANCET_F16 || d == LANCET_BF16; }
inline int dtype_bytes(int d) { return d == LANCET_F32 ? 4 : 2; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();
// Process-wide caps on the grids of the exchange kernels and of the persistent expert GEMM (lancet_set_cta_limits);
// 0 = no cap.  A schedule that runs an exchange stage next to a GEMM gives each a share of the SMs with them.
int exchange_cta_limit();
int gemm_cta_limit();
int gemm_option(int bit);      // experiment switches, bit >= 1 of the value given to lancet_set_gemm_paired
bool gemm_paired_enabled();   // lancet_set_gemm_paired: the two-CTA form of the grouped GEMM (default on)

template <typename T>
struct Num;
template <>
struct Num<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Num<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <>
struct Num<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Scalar load of element i of an array whose dtype is only known at run time.
__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
  if (dtype == LANCET_F32) return static_cast<const float*>(p)[i];
  if (dtype == LANCET_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void store_from_float(void* p, int dtype, size_t i, float v) {
  if (dtype == LANCET_F32)
    static_cast<float*>(p)[i] = v;
  else if (dtype == LANCET_F16)
    static_cast<__half*>(p)[i] = __float2half_rn(v);
  else
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// launchers shared between translation units
size_t gate_workspace_bytes(int S, int E, int k, int n_chunks);
int gate_launch(const void* gate, int gate_dtype, int S, int E, int k, int n_chunks, const int32_t* in_capused, int C,
                int M, void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused,
                uint64_t* out_elems, void* ws, int global_loc, cudaStream_t stream, int32_t* chain_row0 = nullptr);
int dispatch_launch(const int32_t* idx_loc, int k, const int32_t* in_cap, const int32_t* rows_hi, const int32_t* rows_lo,
                    const void* x, void* out, int S, int Sp, int M, int C, int E, int dtype, int flags,
                    cudaStream_t stream);
int combine_launch(const void* gates, int gates_dtype, const int32_t* idx_loc, int k, const void* src, void* out, int S,
                   int Sp, int M, int C, int E, int dtype, cudaStream_t stream);

}  // namespace lancet

// Calls FN<T>(...) with T chosen from a LANCET_* dtype code.
#define LANCET_DISPATCH_DTYPE(dtype, FN, ...)                  \
  ((dtype) == LANCET_F32   ? FN<float>(__VA_ARGS__)            \
   : (dtype) == LANCET_F16 ? FN<__half>(__VA_ARGS__)           \
                           : FN<__nv_bfloat16>(__VA_ARGS__))
