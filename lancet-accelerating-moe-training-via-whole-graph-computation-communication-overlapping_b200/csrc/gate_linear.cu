// Gate projection of the MoE layer: probs = softmax(h * wg^T), and its data gradient.
//
// In the reference the gate is a Linear(model_dim, experts, bias = False) followed by softmax (the Gate module,
// models/benchmark/pytorch/utils.py:565-573; TopKGate.forward, docker/resources/sharded_moe.py:370-390): two library
// operators in front of moe_encode.  The reference's forward optimisation splits such operators next to the MoE
// layer into token chunks so that a chunk's projection runs under the previous chunk's all-to-all
// (src/pass/dist_optimization/partition_exprs.cc:1709-1795).  A library GEMM may choose another blocking when the
// row count changes, so a chunked and an unchunked run could differ in the last bit of a probability and, once in
// a while, in an expert choice.  Here every token is handled by one warp in a fixed order of operations, so the
// result of a token does not depend on which other tokens are in the call.
#include "common.cuh"

namespace lancet {

constexpr int kGateMaxE = 64;   // experts per layer this kernel handles
constexpr int kGateWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kGateWarps * 32)
gate_softmax_kernel(const T* __restrict__ h, const float* __restrict__ wg, float* __restrict__ probs, int S, int M, int E) {
  __shared__ float s_logit[kGateWarps][kGateMaxE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x * kGateWarps + warp;
  if (s >= S) return;
  const T* row = h + (size_t)s * M;
  for (int e0 = 0; e0 < E; e0 += 16) {
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;
    for (int m = lane; m < M; m += 32) {
      const float hv = Num<T>::to_f(row[m]);
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (e0 + j < E) acc[j] = fmaf(hv, __ldg(wg + (size_t)(e0 + j) * M + m), acc[j]);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float v = acc[j];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
      if (lane == 0 && e0 + j < E) s_logit[warp][e0 + j] = v;
    }
  }
  __syncwarp();
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, s_logit[warp][e]);
  float sum = 0.f;
  for (int e = 0; e < E; ++e) sum += expf(s_logit[warp][e] - mx);
  const float inv = 1.0f / sum;
  for (int e = lane; e < E; e += 32) probs[(size_t)s * E + e] = expf(s_logit[warp][e] - mx) * inv;
}

// dlogits[s,e] = p[s,e] * (dp[s,e] - sum_e' dp[s,e'] p[s,e']);   dh[s,m] = sum_e dlogits[s,e] * wg[e,m]
template <typename T>
__global__ void __launch_bounds__(kGateWarps * 32)
gate_softmax_bwd_kernel(const float* __restrict__ probs, const float* __restrict__ dprobs, const float* __restrict__ wg,
                        float* __restrict__ dlogits, T* __restrict__ dh, int S, int M, int E) {
  __shared__ float s_dl[kGateWarps][kGateMaxE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x * kGateWarps + warp;
  if (s >= S) return;
  const float* p = probs + (size_t)s * E;
  const float* dp = dprobs + (size_t)s * E;
  float dot = 0.f;
  for (int e = 0; e < E; ++e) dot = fmaf(dp[e], p[e], dot);
  for (int e = lane; e < E; e += 32) {
    const float v = p[e] * (dp[e] - dot);
    s_dl[warp][e] = v;
    dlogits[(size_t)s * E + e] = v;
  }
  __syncwarp();
  for (int m = lane; m < M; m += 32) {
    float acc = 0.f;
    for (int e = 0; e < E; ++e) acc = fmaf(s_dl[warp][e], __ldg(wg + (size_t)e * M + m), acc);
    dh[(size_t)s * M + m] = Num<T>::from_f(acc);
  }
}

// Vector form for rows whose length is a multiple of 4: a lane owns four consecutive elements per step (one 8- or 16-byte load
// of the row, one float4 per expert of the weights) and EB experts are accumulated at a time, EB the smallest of 2, 4, 8, 16
// that holds E (the generic kernel above always runs 16 predicated accumulators).  The order of operations of a token is
// fixed, so its probabilities do not depend on which other tokens are in the call.
template <typename T>
__device__ __forceinline__ float4 gate_load4(const T* p);
template <>
__device__ __forceinline__ float4 gate_load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 gate_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <>
__device__ __forceinline__ float4 gate_load4<__half>(const __half* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <typename T>
__device__ __forceinline__ void gate_store4(T* p, float4 v);
template <>
__device__ __forceinline__ void gate_store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void gate_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
template <>
__device__ __forceinline__ void gate_store4<__half>(__half* p, float4 v) {
  __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename T, int EB>
__global__ void __launch_bounds__(kGateWarps * 32)
gate_softmax_vec_kernel(const T* __restrict__ h, const float* __restrict__ wg, float* __restrict__ probs, int S, int M, int E) {
  __shared__ float s_logit[kGateWarps][kGateMaxE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x * kGateWarps + warp;
  if (s >= S) return;
  const T* row = h + (size_t)s * M;
  for (int e0 = 0; e0 < E; e0 += EB) {
    float acc[EB];
#pragma unroll
    for (int j = 0; j < EB; ++j) acc[j] = 0.f;
    for (int m = lane * 4; m < M; m += 128) {
      const float4 hv = gate_load4<T>(row + m);
#pragma unroll
      for (int j = 0; j < EB; ++j) {
        if (e0 + j < E) {
          const float4 w = __ldg(reinterpret_cast<const float4*>(wg + (size_t)(e0 + j) * M + m));
          acc[j] = fmaf(hv.x, w.x, acc[j]);
          acc[j] = fmaf(hv.y, w.y, acc[j]);
          acc[j] = fmaf(hv.z, w.z, acc[j]);
          acc[j] = fmaf(hv.w, w.w, acc[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < EB; ++j) {
      float v = acc[j];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
      if (lane == 0 && e0 + j < E) s_logit[warp][e0 + j] = v;
    }
  }
  __syncwarp();
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, s_logit[warp][e]);
  float sum = 0.f;
  for (int e = 0; e < E; ++e) sum += expf(s_logit[warp][e] - mx);
  const float inv = 1.0f / sum;
  for (int e = lane; e < E; e += 32) probs[(size_t)s * E + e] = expf(s_logit[warp][e] - mx) * inv;
}

template <typename T>
__global__ void __launch_bounds__(kGateWarps * 32)
gate_softmax_bwd_vec_kernel(const float* __restrict__ probs, const float* __restrict__ dprobs, const float* __restrict__ wg,
                            float* __restrict__ dlogits, T* __restrict__ dh, int S, int M, int E) {
  __shared__ float s_dl[kGateWarps][kGateMaxE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x * kGateWarps + warp;
  if (s >= S) return;
  const float* p = probs + (size_t)s * E;
  const float* dp = dprobs + (size_t)s * E;
  float dot = 0.f;
  for (int e = 0; e < E; ++e) dot = fmaf(dp[e], p[e], dot);
  for (int e = lane; e < E; e += 32) {
    const float v = p[e] * (dp[e] - dot);
    s_dl[warp][e] = v;
    dlogits[(size_t)s * E + e] = v;
  }
  __syncwarp();
  for (int m = lane * 4; m < M; m += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int e = 0; e < E; ++e) {
      const float d = s_dl[warp][e];
      const float4 w = __ldg(reinterpret_cast<const float4*>(wg + (size_t)e * M + m));
      acc.x = fmaf(d, w.x, acc.x);
      acc.y = fmaf(d, w.y, acc.y);
      acc.z = fmaf(d, w.z, acc.z);
      acc.w = fmaf(d, w.w, acc.w);
    }
    gate_store4<T>(dh + (size_t)s * M + m, acc);
  }
}

template <typename T>
static int gate_softmax_t(const void* h, const float* wg, float* probs, int S, int M, int E, cudaStream_t st) {
  const int grid = (S + kGateWarps - 1) / kGateWarps;
  const T* hp = static_cast<const T*>(h);
  if (M % 4 == 0 && aligned(h, 16) && aligned(wg, 16)) {
    if (E <= 2) gate_softmax_vec_kernel<T, 2><<<grid, kGateWarps * 32, 0, st>>>(hp, wg, probs, S, M, E);
    else if (E <= 4) gate_softmax_vec_kernel<T, 4><<<grid, kGateWarps * 32, 0, st>>>(hp, wg, probs, S, M, E);
    else if (E <= 8) gate_softmax_vec_kernel<T, 8><<<grid, kGateWarps * 32, 0, st>>>(hp, wg, probs, S, M, E);
    else gate_softmax_vec_kernel<T, 16><<<grid, kGateWarps * 32, 0, st>>>(hp, wg, probs, S, M, E);
  } else {
    gate_softmax_kernel<T><<<grid, kGateWarps * 32, 0, st>>>(hp, wg, probs, S, M, E);
  }
  return launch_status("gate_softmax_kernel");
}

template <typename T>
static int gate_softmax_bwd_t(const float* probs, const float* dprobs, const float* wg, float* dlogits, void* dh, int S, int M,
                              int E, cudaStream_t st) {
  const int grid = (S + kGateWarps - 1) / kGateWarps;
  if (M % 4 == 0 && aligned(dh, 16) && aligned(wg, 16))
    gate_softmax_bwd_vec_kernel<T><<<grid, kGateWarps * 32, 0, st>>>(probs, dprobs, wg, dlogits, static_cast<T*>(dh), S, M, E);
  else
    gate_softmax_bwd_kernel<T><<<grid, kGateWarps * 32, 0, st>>>(probs, dprobs, wg, dlogits, static_cast<T*>(dh), S, M, E);
  return launch_status("gate_softmax_bwd_kernel");
}

}  // namespace lancet

extern "C" {
using namespace lancet;

int lancet_gate_softmax(const void* h, int dtype, const float* wg, float* probs, int S, int M, int E, lancet_stream_t stream) {
  LANCET_REQUIRE(valid_dtype(dtype) && S >= 0 && M >= 1 && E >= 1 && E <= kGateMaxE, LANCET_ERR_INVALID,
                 "lancet_gate_softmax: bad dtype or sizes S=%d M=%d E=%d (at most %d experts)", S, M, E, kGateMaxE);
  if (S == 0) return LANCET_OK;
  LANCET_REQUIRE(h && wg && probs, LANCET_ERR_NULL, "lancet_gate_softmax: null pointer argument");
  return LANCET_DISPATCH_DTYPE(dtype, gate_softmax_t, h, wg, probs, S, M, E, static_cast<cudaStream_t>(stream));
}

int lancet_gate_softmax_bwd(const float* probs, const float* dprobs, const float* wg, float* dlogits, void* dh, int dtype, int S,
                            int M, int E, lancet_stream_t stream) {
  LANCET_REQUIRE(valid_dtype(dtype) && S >= 0 && M >= 1 && E >= 1 && E <= kGateMaxE, LANCET_ERR_INVALID,
                 "lancet_gate_softmax_bwd: bad dtype or sizes S=%d M=%d E=%d (at most %d experts)", S, M, E, kGateMaxE);
  if (S == 0) return LANCET_OK;
  LANCET_REQUIRE(probs && dprobs && wg && dlogits && dh, LANCET_ERR_NULL, "lancet_gate_softmax_bwd: null pointer argument");
  return LANCET_DISPATCH_DTYPE(dtype, gate_softmax_bwd_t, probs, dprobs, wg, dlogits, dh, S, M, E, static_cast<cudaStream_t>(stream));
}
}
