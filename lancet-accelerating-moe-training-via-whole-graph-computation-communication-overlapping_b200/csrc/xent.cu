// Softmax cross-entropy over a padded vocabulary, forward and backward, for the language-model head of the GPT-MoE step.
//
// The reference's benchmark models end in log_softmax + nll_loss (models/benchmark/raf/raf_bencher.py:84,
// models/benchmark/pytorch/torch_bencher.py:463; operators raf.op.nll_loss / nll_loss_dpred, src/op/declare/loss.cc:55-92):
// a float32 copy of the [tokens, vocab] logits, a second [tokens, vocab] tensor of log-probabilities, and the same two
// again on the way back.  With 8192 tokens and 50257 classes those copies are 1.6 GB each and cost a sixth of the step.
// Here the forward pass reads the 16-bit logits once (one block per row, online maximum and sum) and keeps log-sum-exp per
// row; the backward pass reads them once more and writes the gradient in the logits' own type:
//     loss[r]   = lse[r] - x[r, t_r]                                   (0 where t_r < 0: ignored row)
//     dx[r, j]  = (exp(x[r, j] - lse[r]) - [j == t_r]) * g * scale     (0 in ignored rows and in padded columns j >= V)
// g is the upstream gradient of the summed loss, read from device memory, so nothing synchronises with the host.
#include "common.cuh"

namespace lancet {

constexpr int kXentThreads = 256;

template <typename T>
struct XVec;   // 16-byte vector of T
template <>
struct XVec<float> {
  static constexpr int N = 4;
  float v[4];
};
template <>
struct XVec<__half> {
  static constexpr int N = 8;
  __half v[8];
};
template <>
struct XVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __nv_bfloat16 v[8];
};

__device__ __forceinline__ void online_add(float& m, float& s, float x) {
  if (x > m) {
    s = s * __expf(m - x) + 1.0f;
    m = x;
  } else {
    s += __expf(x - m);
  }
}
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) return;
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

template <typename T>
__global__ void __launch_bounds__(kXentThreads)
xent_fwd_kernel(const T* __restrict__ x, long long ld, const long long* __restrict__ target, int V, float* __restrict__ loss,
                float* __restrict__ lse) {
  using X = XVec<T>;
  __shared__ float sm[kXentThreads / 32], ss[kXentThreads / 32];
  const long long r = blockIdx.x;
  const T* row = x + r * ld;
  float m = -INFINITY, s = 0.f;
  const bool vec = (ld % X::N == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (vec) {
    const int nv = V / X::N;
    const X* rv = reinterpret_cast<const X*>(row);
    int i = threadIdx.x;
    for (; i + kXentThreads < nv; i += 2 * kXentThreads) {     // two vectors in flight
      const X a = rv[i], b = rv[i + kXentThreads];
#pragma unroll
      for (int j = 0; j < X::N; ++j) online_add(m, s, Num<T>::to_f(a.v[j]));
#pragma unroll
      for (int j = 0; j < X::N; ++j) online_add(m, s, Num<T>::to_f(b.v[j]));
    }
    for (; i < nv; i += kXentThreads) {
      const X a = rv[i];
#pragma unroll
      for (int j = 0; j < X::N; ++j) online_add(m, s, Num<T>::to_f(a.v[j]));
    }
    for (int c = nv * X::N + threadIdx.x; c < V; c += kXentThreads) online_add(m, s, Num<T>::to_f(row[c]));
  } else {
    for (int c = threadIdx.x; c < V; c += kXentThreads) online_add(m, s, Num<T>::to_f(row[c]));
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, d), s2 = __shfl_xor_sync(0xffffffffu, s, d);
    online_merge(m, s, m2, s2);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sm[warp] = m;
    ss[warp] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = sm[0], S = ss[0];
    for (int w = 1; w < kXentThreads / 32; ++w) online_merge(M, S, sm[w], ss[w]);
    const float l = M + logf(S);
    lse[r] = l;
    const long long t = target[r];
    loss[r] = (t >= 0 && t < V) ? l - Num<T>::to_f(row[t]) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(kXentThreads)
xent_bwd_kernel(const T* __restrict__ x, long long ld, const long long* __restrict__ target, int V, int cols,
                const float* __restrict__ lse, const float* __restrict__ gout, float scale, T* __restrict__ dx, long long ldd) {
  using X = XVec<T>;
  const long long r = blockIdx.x;
  const T* row = x + r * ld;
  T* drow = dx + r * ldd;
  const long long t = target[r];
  const bool live = t >= 0 && t < V;
  const float g = live ? (gout ? *gout : 1.0f) * scale : 0.f;
  const float l = lse[r];
  const bool vec = (ld % X::N == 0) && (ldd % X::N == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(dx) & 15) == 0);
  int c0 = 0;
  if (vec) {
    const int nv = cols / X::N;
    const X* rv = reinterpret_cast<const X*>(row);
    X* dv = reinterpret_cast<X*>(drow);
    for (int i = threadIdx.x; i < nv; i += kXentThreads) {
      X o;
      if (live) {
        const X a = rv[i];
#pragma unroll
        for (int j = 0; j < X::N; ++j) {
          const int c = i * X::N + j;
          float p = c < V ? __expf(Num<T>::to_f(a.v[j]) - l) : 0.f;
          if (c == t) p -= 1.0f;
          o.v[j] = Num<T>::from_f(p * g);
        }
      } else {
#pragma unroll
        for (int j = 0; j < X::N; ++j) o.v[j] = Num<T>::from_f(0.f);
      }
      dv[i] = o;
    }
    c0 = nv * X::N;
  }
  for (int c = c0 + threadIdx.x; c < cols; c += kXentThreads) {
    float p = (live && c < V) ? __expf(Num<T>::to_f(row[c]) - l) : 0.f;
    if (live && c == t) p -= 1.0f;
    drow[c] = Num<T>::from_f(p * g);
  }
}

}  // namespace lancet

extern "C" {
using namespace lancet;

int lancet_softmax_xent_fwd(const void* logits, long long ld, const long long* target, int rows, int vocab, int dtype,
                            float* loss_rows, float* lse_rows, lancet_stream_t stream) {
  LANCET_REQUIRE(rows >= 0 && vocab >= 1 && ld >= vocab && valid_dtype(dtype), LANCET_ERR_INVALID,
                 "lancet_softmax_xent_fwd: bad rows=%d, vocab=%d, row stride %lld or dtype", rows, vocab, ld);
  if (rows == 0) return LANCET_OK;
  LANCET_REQUIRE(logits && target && loss_rows && lse_rows, LANCET_ERR_NULL, "lancet_softmax_xent_fwd: null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == LANCET_F32)
    xent_fwd_kernel<float><<<rows, kXentThreads, 0, st>>>(static_cast<const float*>(logits), ld, target, vocab, loss_rows, lse_rows);
  else if (dtype == LANCET_F16)
    xent_fwd_kernel<__half><<<rows, kXentThreads, 0, st>>>(static_cast<const __half*>(logits), ld, target, vocab, loss_rows, lse_rows);
  else
    xent_fwd_kernel<__nv_bfloat16><<<rows, kXentThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, target, vocab,
                                                                 loss_rows, lse_rows);
  return launch_status("xent_fwd_kernel");
}

int lancet_softmax_xent_bwd(const void* logits, long long ld, const long long* target, int rows, int vocab, int cols, int dtype,
                            const float* lse_rows, const float* grad_out, float scale, void* dlogits, long long ldd,
                            lancet_stream_t stream) {
  LANCET_REQUIRE(rows >= 0 && vocab >= 1 && cols >= vocab && ld >= cols && ldd >= cols && valid_dtype(dtype), LANCET_ERR_INVALID,
                 "lancet_softmax_xent_bwd: bad rows=%d, vocab=%d, cols=%d, row strides %lld / %lld or dtype", rows, vocab, cols, ld,
                 ldd);
  if (rows == 0) return LANCET_OK;
  LANCET_REQUIRE(logits && target && lse_rows && dlogits, LANCET_ERR_NULL, "lancet_softmax_xent_bwd: null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == LANCET_F32)
    xent_bwd_kernel<float><<<rows, kXentThreads, 0, st>>>(static_cast<const float*>(logits), ld, target, vocab, cols, lse_rows,
                                                         grad_out, scale, static_cast<float*>(dlogits), ldd);
  else if (dtype == LANCET_F16)
    xent_bwd_kernel<__half><<<rows, kXentThreads, 0, st>>>(static_cast<const __half*>(logits), ld, target, vocab, cols, lse_rows,
                                                          grad_out, scale, static_cast<__half*>(dlogits), ldd);
  else
    xent_bwd_kernel<__nv_bfloat16><<<rows, kXentThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, target, vocab,
                                                                 cols, lse_rows, grad_out, scale,
                                                                 static_cast<__nv_bfloat16*>(dlogits), ldd);
  return launch_status("xent_bwd_kernel");
}
}
