// Layer normalisation of the residual stream in front of the attention, FFN and MoE blocks, forward and backward.
//
// In the reference this is raf.op.layer_norm / layer_norm_dx (src/op/declare/nn.cc; the benchmark models call it through
// the GPT-2 / BERT builders, models/benchmark/pytorch/nlp.py), one of the non-MoE operators its forward partition splits
// along the token axis next to the MoE layer (src/pass/dist_optimization/partition_exprs.cc:1709-1795).  The result of a row
// depends on that row only and is computed by one warp in a fixed order, so chunking the tokens does not change a bit.
//   forward : float32 rows in, normalised rows out in float32 or directly in the 16-bit type the next GEMM reads
//             (no separate cast pass), mean and 1/std kept per row;
//   backward: dx in float32 (one warp per row), and the weight / bias gradients as column sums over row splits that a small
//             kernel adds up in a fixed order (no atomics: reproducible).
// HBM-bound: forward reads 4 B and writes 2-4 B per element, backward reads 4 B + the dy width and writes 4 B.
#include "common.cuh"

namespace lancet {

constexpr int kLnWarps = 8;
constexpr int kLnThreads = kLnWarps * 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

template <typename T>
__device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, float a, float b, float c, float d) {
  __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <>
__device__ __forceinline__ float4 load4<__half>(const __half* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// One warp per row; lane l holds the float4 vectors l, l + 32, ... of the row (M = 128 * VPL elements).
template <typename TO, int VPL>
__global__ void __launch_bounds__(kLnThreads)
layer_norm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                      TO* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int R, float eps) {
  constexpr int M = 128 * VPL;
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kLnWarps;
  for (long long r = warp; r < R; r += nwarps) {
    const float* row = x + r * M;
    float4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) v[i] = __ldcs(reinterpret_cast<const float4*>(row) + i * 32 + lane);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mu = warp_sum(s) * (1.0f / M);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const float a = v[i].x - mu, b = v[i].y - mu, c = v[i].z - mu, d = v[i].w - mu;
      q += (a * a + b * b) + (c * c + d * d);
    }
    const float rs = rsqrtf(warp_sum(q) * (1.0f / M) + eps);
    if (lane == 0) {
      mean[r] = mu;
      rstd[r] = rs;
    }
    TO* out = y + r * M;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * 32 + lane) * 4;
      const float4 g = __ldg(reinterpret_cast<const float4*>(gamma + c));
      const float4 b = __ldg(reinterpret_cast<const float4*>(beta + c));
      store4<TO>(out + c, fmaf((v[i].x - mu) * rs, g.x, b.x), fmaf((v[i].y - mu) * rs, g.y, b.y),
                 fmaf((v[i].z - mu) * rs, g.z, b.z), fmaf((v[i].w - mu) * rs, g.w, b.w));
    }
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) with g = dy * gamma, xhat = (x - mean) * rstd: one warp per row.
template <typename TD, int VPL>
__global__ void __launch_bounds__(kLnThreads)
layer_norm_dx_kernel(const float* __restrict__ x, const TD* __restrict__ dy, const float* __restrict__ gamma,
                     const float* __restrict__ mean, const float* __restrict__ rstd, float* __restrict__ dx, int R) {
  constexpr int M = 128 * VPL;
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kLnWarps;
  for (long long r = warp; r < R; r += nwarps) {
    const float mu = mean[r], rs = rstd[r];
    float4 xh[VPL], g[VPL];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * 32 + lane) * 4;
      const float4 xv = __ldcs(reinterpret_cast<const float4*>(x + r * M + c));
      const float4 d = load4<TD>(dy + r * M + c);
      const float4 gm = __ldg(reinterpret_cast<const float4*>(gamma + c));
      xh[i] = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
      g[i] = make_float4(d.x * gm.x, d.y * gm.y, d.z * gm.z, d.w * gm.w);
      s1 += (g[i].x + g[i].y) + (g[i].z + g[i].w);
      s2 += (g[i].x * xh[i].x + g[i].y * xh[i].y) + (g[i].z * xh[i].z + g[i].w * xh[i].w);
    }
    const float m1 = warp_sum(s1) * (1.0f / M), m2 = warp_sum(s2) * (1.0f / M);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * 32 + lane) * 4;
      *reinterpret_cast<float4*>(dx + r * M + c) =
          make_float4(rs * (g[i].x - m1 - xh[i].x * m2), rs * (g[i].y - m1 - xh[i].y * m2),
                      rs * (g[i].z - m1 - xh[i].z * m2), rs * (g[i].w - m1 - xh[i].w * m2));
    }
  }
}

// Weight and bias gradients: column sums of dy * xhat and of dy.  Block (tile, split) covers 128 columns and every
// `splits`-th group of rows; its eight warps take rows in turn, a lane owns four columns.  The warps are added in shared
// memory in warp order and the block writes one partial pair [2][128 of M]; layer_norm_param_grad_kernel adds the splits
// in order.  No atomics: the sums are reproducible.
template <typename TD>
__global__ void __launch_bounds__(kLnThreads)
layer_norm_col_partial_kernel(const float* __restrict__ x, const TD* __restrict__ dy, const float* __restrict__ mean,
                              const float* __restrict__ rstd, float* __restrict__ partial, int R, int M) {
  __shared__ float4 red[2][kLnWarps][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 128 + lane * 4;
  const int split = blockIdx.y, splits = gridDim.y;
  float4 ag = make_float4(0.f, 0.f, 0.f, 0.f), ab = ag;
  for (long long r = (long long)split * kLnWarps + w; r < R; r += (long long)splits * kLnWarps) {
    const float mu = mean[r], rs = rstd[r];
    const float4 xv = __ldcs(reinterpret_cast<const float4*>(x + r * M + c));
    const float4 d = load4<TD>(dy + r * M + c);
    ag.x = fmaf(d.x, (xv.x - mu) * rs, ag.x);
    ag.y = fmaf(d.y, (xv.y - mu) * rs, ag.y);
    ag.z = fmaf(d.z, (xv.z - mu) * rs, ag.z);
    ag.w = fmaf(d.w, (xv.w - mu) * rs, ag.w);
    ab.x += d.x;
    ab.y += d.y;
    ab.z += d.z;
    ab.w += d.w;
  }
  red[0][w][lane] = ag;
  red[1][w][lane] = ab;
  __syncthreads();
  if (w < 2) {
    float4 s = red[w][0][lane];
    for (int k = 1; k < kLnWarps; ++k) {
      const float4 t = red[w][k][lane];
      s.x += t.x;
      s.y += t.y;
      s.z += t.z;
      s.w += t.w;
    }
    *reinterpret_cast<float4*>(partial + ((size_t)split * 2 + w) * M + c) = s;
  }
}

// dgamma[c] = sum over the row splits of partial[split][0][c], dbeta[c] likewise.  A block owns 128 of the 2 M columns (a lane
// four of them); its eight warps take every eighth split and are added in warp order: a fixed order, and a short chain of loads.
__global__ void __launch_bounds__(kLnThreads)
layer_norm_param_grad_kernel(const float* __restrict__ partial, int splits, int M, float* __restrict__ dgamma,
                             float* __restrict__ dbeta) {
  __shared__ float4 red[kLnWarps][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 128 + lane * 4;       // column of the [2][M] pair
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int b = w; b < splits; b += kLnWarps) {
    const float4 t = *reinterpret_cast<const float4*>(partial + (size_t)b * 2 * M + c);
    s.x += t.x;
    s.y += t.y;
    s.z += t.z;
    s.w += t.w;
  }
  red[w][lane] = s;
  __syncthreads();
  if (w == 0) {
    float4 a = red[0][lane];
    for (int k = 1; k < kLnWarps; ++k) {
      const float4 t = red[k][lane];
      a.x += t.x;
      a.y += t.y;
      a.z += t.z;
      a.w += t.w;
    }
    float* out = c < M ? dgamma + c : dbeta + (c - M);
    *reinterpret_cast<float4*>(out) = a;
  }
}

static int ln_blocks(int R) {
  const int want = (R + kLnWarps - 1) / kLnWarps;
  const int cap = sm_count() * 4;
  return want < cap ? (want > 0 ? want : 1) : cap;
}
// row splits of the column-sum kernel: about four blocks per SM over all column tiles, at least 8 rows per warp turn
static int ln_splits(int R, int M) {
  const int tiles = M / 128;
  int s = (sm_count() * 4 + tiles - 1) / tiles;
  const int most = (R + kLnWarps - 1) / kLnWarps;
  if (s > most) s = most;
  return s > 0 ? s : 1;
}

template <typename TO, int VPL>
static void ln_fwd_launch(const float* x, const float* g, const float* b, void* y, float* mean, float* rstd, int R, float eps,
                          cudaStream_t st) {
  layer_norm_fwd_kernel<TO, VPL><<<ln_blocks(R), kLnThreads, 0, st>>>(x, g, b, static_cast<TO*>(y), mean, rstd, R, eps);
}
template <typename TD, int VPL>
static void ln_dx_launch(const float* x, const void* dy, const float* g, const float* mean, const float* rstd, float* dx, int R,
                         cudaStream_t st) {
  layer_norm_dx_kernel<TD, VPL><<<ln_blocks(R), kLnThreads, 0, st>>>(x, static_cast<const TD*>(dy), g, mean, rstd, dx, R);
}
template <typename TD>
static void ln_col_launch(const float* x, const void* dy, const float* mean, const float* rstd, float* partial, int R, int M,
                          int splits, cudaStream_t st) {
  layer_norm_col_partial_kernel<TD><<<dim3(M / 128, splits), kLnThreads, 0, st>>>(x, static_cast<const TD*>(dy), mean, rstd,
                                                                                 partial, R, M);
}

#define LANCET_LN_VPL(V, CALL)   \
  switch (V) {                    \
    case 1: { CALL(1); break; }   \
    case 2: { CALL(2); break; }   \
    case 4: { CALL(4); break; }   \
    case 6: { CALL(6); break; }   \
    case 8: { CALL(8); break; }   \
    case 12: { CALL(12); break; } \
    case 16: { CALL(16); break; } \
    default: return fail(LANCET_ERR_UNSUPPORTED, "layer norm: row length %d is not 128 x {1,2,4,6,8,12,16}", 128 * (V)); \
  }

}  // namespace lancet

extern "C" {
using namespace lancet;

size_t lancet_layer_norm_workspace_bytes(int rows, int M) {
  if (rows < 0 || M <= 0) return 0;
  if (M % 128 != 0) return 0;
  return (size_t)ln_splits(rows, M) * 2 * M * sizeof(float);
}

int lancet_layer_norm_fwd(const float* x, const float* gamma, const float* beta, void* y, int out_dtype, float* mean, float* rstd,
                          int rows, int M, float eps, lancet_stream_t stream) {
  LANCET_REQUIRE(rows >= 0 && M > 0 && M % 128 == 0 && valid_dtype(out_dtype), LANCET_ERR_INVALID,
                 "lancet_layer_norm_fwd: bad rows=%d, M=%d (a multiple of 128) or dtype", rows, M);
  if (rows == 0) return LANCET_OK;
  LANCET_REQUIRE(x && gamma && beta && y && mean && rstd, LANCET_ERR_NULL, "lancet_layer_norm_fwd: null pointer argument");
  LANCET_REQUIRE(aligned(x, 16) && aligned(y, 8) && aligned(gamma, 16) && aligned(beta, 16), LANCET_ERR_INVALID,
                 "lancet_layer_norm_fwd: operands must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vpl = M / 128;
  if (out_dtype == LANCET_F32) {
#define CALL(V) ln_fwd_launch<float, V>(x, gamma, beta, y, mean, rstd, rows, eps, st)
    LANCET_LN_VPL(vpl, CALL)
#undef CALL
  } else if (out_dtype == LANCET_F16) {
#define CALL(V) ln_fwd_launch<__half, V>(x, gamma, beta, y, mean, rstd, rows, eps, st)
    LANCET_LN_VPL(vpl, CALL)
#undef CALL
  } else {
#define CALL(V) ln_fwd_launch<__nv_bfloat16, V>(x, gamma, beta, y, mean, rstd, rows, eps, st)
    LANCET_LN_VPL(vpl, CALL)
#undef CALL
  }
  return launch_status("layer_norm_fwd_kernel");
}

int lancet_layer_norm_bwd(const float* x, const void* dy, int dy_dtype, const float* gamma, const float* mean, const float* rstd,
                          float* dx, float* dgamma, float* dbeta, int rows, int M, void* ws, size_t ws_bytes,
                          lancet_stream_t stream) {
  LANCET_REQUIRE(rows >= 0 && M > 0 && M % 128 == 0 && valid_dtype(dy_dtype), LANCET_ERR_INVALID,
                 "lancet_layer_norm_bwd: bad rows=%d, M=%d (a multiple of 128) or dtype", rows, M);
  LANCET_REQUIRE(dgamma && dbeta, LANCET_ERR_NULL, "lancet_layer_norm_bwd: null gradient pointer");
  LANCET_REQUIRE(aligned(dgamma, 16) && aligned(dbeta, 16), LANCET_ERR_INVALID,
                 "lancet_layer_norm_bwd: the gradient vectors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    LANCET_CUDA(cudaMemsetAsync(dgamma, 0, (size_t)M * sizeof(float), st));
    LANCET_CUDA(cudaMemsetAsync(dbeta, 0, (size_t)M * sizeof(float), st));
    return LANCET_OK;
  }
  LANCET_REQUIRE(x && dy && gamma && mean && rstd && dx && ws, LANCET_ERR_NULL, "lancet_layer_norm_bwd: null pointer argument");
  LANCET_REQUIRE(ws_bytes >= lancet_layer_norm_workspace_bytes(rows, M) && aligned(ws, 16), LANCET_ERR_INVALID,
                 "lancet_layer_norm_bwd: workspace of %zu bytes is too small or unaligned", ws_bytes);
  LANCET_REQUIRE(aligned(x, 16) && aligned(dy, 8) && aligned(dx, 16) && aligned(gamma, 16), LANCET_ERR_INVALID,
                 "lancet_layer_norm_bwd: operands must be 16-byte aligned");
  const int splits = ln_splits(rows, M);
  float* partial = static_cast<float*>(ws);
  const int vpl = M / 128;
  if (dy_dtype == LANCET_F32) {
#define CALL(V) ln_dx_launch<float, V>(x, dy, gamma, mean, rstd, dx, rows, st)
    LANCET_LN_VPL(vpl, CALL)
#undef CALL
    ln_col_launch<float>(x, dy, mean, rstd, partial, rows, M, splits, st);
  } else if (dy_dtype == LANCET_F16) {
#define CALL(V) ln_dx_launch<__half, V>(x, dy, gamma, mean, rstd, dx, rows, st)
    LANCET_LN_VPL(vpl, CALL)
#undef CALL
    ln_col_launch<__half>(x, dy, mean, rstd, partial, rows, M, splits, st);
  } else {
#define CALL(V) ln_dx_launch<__nv_bfloat16, V>(x, dy, gamma, mean, rstd, dx, rows, st)
    LANCET_LN_VPL(vpl, CALL)
#undef CALL
    ln_col_launch<__nv_bfloat16>(x, dy, mean, rstd, partial, rows, M, splits, st);
  }
  if (int rc = launch_status("layer_norm_dx_kernel / layer_norm_col_partial_kernel")) return rc;
  layer_norm_param_grad_kernel<<<2 * M / 128, kLnThreads, 0, st>>>(partial, splits, M, dgamma, dbeta);
  return launch_status("layer_norm_param_grad_kernel");
}
}
