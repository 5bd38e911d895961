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
struct XVec;   // 16-byte vector of T (the alignment is what lets the compiler move it with one 128-bit access)
template <>
struct __align__(16) XVec<float> {
  static constexpr int N = 4;
  float v[4];
};
template <>
struct __align__(16) XVec<__half> {
  static constexpr int N = 8;
  __half v[8];
};
template <>
struct __align__(16) XVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __nv_bfloat16 v[8];
};

// Online maximum and sum in the base-2 domain (y = x * log2 e): one vector of N values at a time, so that the running sum
// is rescaled at most once per vector and every value costs one FMA, one ex2 and one add.
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T, int N>
__device__ __forceinline__ void online_add_vec(float& m, float& s, const T* v) {
  float y[N];
#pragma unroll
  for (int j = 0; j < N; ++j) y[j] = Num<T>::to_f(v[j]) * kLog2e;
  float vm = y[0];
#pragma unroll
  for (int j = 1; j < N; ++j) vm = fmaxf(vm, y[j]);
  if (vm > m) {
    s *= ex2f(m - vm);      // m = -inf at the start: ex2(-inf) = 0
    m = vm;
  }
#pragma unroll
  for (int j = 0; j < N; ++j) s += ex2f(y[j] - m);
}
__device__ __forceinline__ void online_add(float& m, float& s, float x) {
  const float y = x * kLog2e;
  if (y > m) {
    s = s * ex2f(m - y) + 1.0f;
    m = y;
  } else {
    s += ex2f(y - m);
  }
}
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) return;
  s = s * ex2f(m - mm) + s2 * ex2f(m2 - mm);
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
    for (; i + 3 * kXentThreads < nv; i += 4 * kXentThreads) {     // four vectors in flight
      const X a = rv[i], b = rv[i + kXentThreads], c = rv[i + 2 * kXentThreads], d = rv[i + 3 * kXentThreads];
      online_add_vec<T, X::N>(m, s, a.v);
      online_add_vec<T, X::N>(m, s, b.v);
      online_add_vec<T, X::N>(m, s, c.v);
      online_add_vec<T, X::N>(m, s, d.v);
    }
    for (; i < nv; i += kXentThreads) {
      const X a = rv[i];
      online_add_vec<T, X::N>(m, s, a.v);
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
    const float l = M * kLn2 + logf(S);      // back to natural logarithms
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
  const long long t64 = target[r];
  const bool live = t64 >= 0 && t64 < V;
  const int t = live ? (int)t64 : -1;
  const float g = live ? (gout ? *gout : 1.0f) * scale : 0.f;
  const float l2 = lse[r] * kLog2e;
  const bool vec = (ld % X::N == 0) && (ldd % X::N == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(dx) & 15) == 0);
  int c0 = 0;
  if (vec) {
    const int nv = cols / X::N;      // vectors of the row, padding included
    const int nfull = V / X::N;      // vectors without a padded column
    const X* rv = reinterpret_cast<const X*>(row);
    X* dv = reinterpret_cast<X*>(drow);
    // p * g for a vector without padding and without the target column: one FMA, one ex2, one multiply per value
    auto grad_vec = [&](const X& a) {
      X o;
#pragma unroll
      for (int j = 0; j < X::N; ++j) o.v[j] = Num<T>::from_f(ex2f(fmaf(Num<T>::to_f(a.v[j]), kLog2e, -l2)) * g);
      return o;
    };
    if (live) {
      // four vectors per thread are loaded before the first exponential or store
      int i = threadIdx.x;
      for (; i + 3 * kXentThreads < nfull; i += 4 * kXentThreads) {
        const X a0 = rv[i], a1 = rv[i + kXentThreads], a2 = rv[i + 2 * kXentThreads], a3 = rv[i + 3 * kXentThreads];
        dv[i] = grad_vec(a0);
        dv[i + kXentThreads] = grad_vec(a1);
        dv[i + 2 * kXentThreads] = grad_vec(a2);
        dv[i + 3 * kXentThreads] = grad_vec(a3);
      }
      for (; i < nfull; i += kXentThreads) dv[i] = grad_vec(rv[i]);
      // the vector that holds the last valid columns, and the all-padding vectors behind it
      for (int i2 = nfull + threadIdx.x; i2 < nv; i2 += kXentThreads) {
        const X a = rv[i2];
        X o;
#pragma unroll
        for (int j = 0; j < X::N; ++j) {
          const int c = i2 * X::N + j;
          o.v[j] = Num<T>::from_f(c < V ? ex2f(fmaf(Num<T>::to_f(a.v[j]), kLog2e, -l2)) * g : 0.f);
        }
        dv[i2] = o;
      }
      __syncthreads();     // the row is written: one thread now takes the one-hot term off the target column
      if (threadIdx.x == 0) drow[t] = Num<T>::from_f((ex2f(fmaf(Num<T>::to_f(row[t]), kLog2e, -l2)) - 1.0f) * g);
    } else {
      X z;
#pragma unroll
      for (int j = 0; j < X::N; ++j) z.v[j] = Num<T>::from_f(0.f);
      for (int i = threadIdx.x; i < nv; i += kXentThreads) dv[i] = z;
    }
    c0 = nv * X::N;
  }
  for (int c = c0 + threadIdx.x; c < cols; c += kXentThreads) {
    float p = (live && c < V) ? ex2f(fmaf(Num<T>::to_f(row[c]), kLog2e, -l2)) : 0.f;
    if (c == t) p -= 1.0f;
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
