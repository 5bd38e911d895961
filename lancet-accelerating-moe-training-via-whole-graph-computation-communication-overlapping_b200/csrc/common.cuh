// Shared host/device helpers of the C-ABI layer: status codes, the thread-local error text,
// dtype dispatch and small device utilities.
#pragma once
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

inline int launch_status(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LANCET_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  }
  return LANCET_OK;
}

inline bool valid_dtype(int d) { return d == LANCET_F32 || d == LANCET_F16 || d == LANCET_BF16; }
inline int dtype_bytes(int d) { return d == LANCET_F32 ? 4 : 2; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();

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

}  // namespace lancet

// Calls FN<T>(...) with T chosen from a LANCET_* dtype code.
#define LANCET_DISPATCH_DTYPE(dtype, FN, ...)                  \
  ((dtype) == LANCET_F32   ? FN<float>(__VA_ARGS__)            \
   : (dtype) == LANCET_F16 ? FN<__half>(__VA_ARGS__)           \
                           : FN<__nv_bfloat16>(__VA_ARGS__))
