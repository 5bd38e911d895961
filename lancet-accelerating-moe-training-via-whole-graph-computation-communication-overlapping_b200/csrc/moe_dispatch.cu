// Dispatch (scatter of token rows into the [E,C,M] expert buffer), combine (gate-weighted
// gather back) and the four gradient kernels of the MoE layer.
//
// Replaces src/op/dialect/cuda/kernels/tutel_moe_dispatch.cu:39-160 and the launchers at
// :461-546 of the reference, which zero the whole expert buffer and then add rows into it
// with scalar atomics.  Here a warp owns a row: it is moved with 16-byte accesses, written
// exactly once, and only rows that no token owns are zero-filled, so the bytes moved are the
// bytes the operator is defined to produce.  All kernels are HBM-bound.
#include "common.cuh"

namespace lancet {

constexpr int kRowThreads = 256;
constexpr int kRowWarps = kRowThreads / 32;

template <typename T, int N>
struct alignas(sizeof(T) * N) Pack {
  T v[N];
};

// idx_loc is laid out [n_chunks][2K][Sp] (Sp = S for a single chunk): token s of the batch is token
// s % Sp of chunk s / Sp.  K2 = 2K rows per chunk.
__device__ __forceinline__ size_t il_index(int s, int Sp, int K2, int row) {
  const int c = s / Sp;
  return ((size_t)c * K2 + row) * Sp + (s - c * Sp);
}

__device__ __forceinline__ bool kept_choice(const int32_t* __restrict__ idx_loc, const int32_t* __restrict__ in_cap,
                                            int j, int s, int Sp, int K2, int C, int E, bool global_loc, long long* row) {
  const int idx = idx_loc[il_index(s, Sp, K2, 2 * j)];
  const int loc = idx_loc[il_index(s, Sp, K2, 2 * j + 1)];
  if (idx < 0 || idx >= E || loc < 0 || loc >= C) return false;
  int used = 0;
  if (in_cap) {
    used = in_cap[idx];
    if (loc >= C - used) return false;
  }
  *row = (long long)idx * C + loc + (global_loc ? used : 0);
  return true;
}

// --------------------------------------------------------------------------------------------
// dispatch: byte mover.  V is the access width (uint4 = 16 B when rows allow it).
// tasks [0,S): token rows; tasks [S, S+E*C): candidate zero rows.
// --------------------------------------------------------------------------------------------
template <typename V, int K>
__global__ void __launch_bounds__(kRowThreads)
dispatch_rows_kernel(const int32_t* __restrict__ idx_loc, const int32_t* __restrict__ in_cap,
                     const int32_t* __restrict__ rows_hi, const int32_t* __restrict__ rows_lo, const V* __restrict__ x,
                     V* __restrict__ out, int S, int Sp, int row_vecs, int C, int E, int global_loc, int zero_tail) {
  constexpr int U = 8;
  chain_enter();
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kRowWarps;
  const long long ntasks = (long long)S + (zero_tail ? (long long)E * C : 0);
  for (long long task = gw; task < ntasks; task += nwarps) {
    if (task < S) {
      const int s = (int)task;
      long long row[K];
      bool keep[K];
      bool any = false;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        keep[j] = kept_choice(idx_loc, in_cap, j, s, Sp, 2 * K, C, E, global_loc != 0, &row[j]);
        any |= keep[j];
      }
      if (!any) continue;
      const V* src = x + (size_t)s * row_vecs;
      for (int base = 0; base < row_vecs; base += 32 * U) {
        V r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = base + u * 32 + lane;
          if (v < row_vecs) r[u] = __ldcs(src + v);
        }
#pragma unroll
        for (int j = 0; j < K; ++j) {
          if (!keep[j]) continue;
          V* dst = out + (size_t)row[j] * row_vecs;
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int v = base + u * 32 + lane;
            if (v < row_vecs) dst[v] = r[u];
          }
        }
      }
    } else {
      const long long r = task - S;
      const int e = (int)(r / C);
      const int c = (int)(r % C);
      int used = rows_hi[e] - (rows_lo ? rows_lo[e] : 0);
      if (c < used) continue;
      V* dst = out + (size_t)r * row_vecs;
      V z;
      memset(&z, 0, sizeof(V));
      for (int v = lane; v < row_vecs; v += 32) dst[v] = z;
    }
  }
}

// --------------------------------------------------------------------------------------------
// combine / encode_dx: out[s] = sum_j g[j,s] * src[row_j]  (g = 1 when gates == nullptr)
// --------------------------------------------------------------------------------------------
template <typename T, int N, int K>
__global__ void __launch_bounds__(kRowThreads)
combine_rows_kernel(const void* __restrict__ gates, int gates_dtype, const int32_t* __restrict__ idx_loc,
                    const T* __restrict__ src, T* __restrict__ out, int S, int Sp, int M, int C, int E) {
  using P = Pack<T, N>;
  chain_enter();
  const int lane = threadIdx.x & 31;
  const int row_vecs = M / N;
  const long long gw = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kRowWarps;
  for (long long s = gw; s < S; s += nwarps) {
    long long row[K];
    bool keep[K];
    float g[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      keep[j] = kept_choice(idx_loc, nullptr, j, (int)s, Sp, 2 * K, C, E, false, &row[j]);
      g[j] = gates ? load_as_float(gates, gates_dtype, il_index((int)s, Sp, K, j)) : 1.0f;
    }
    P* dst = reinterpret_cast<P*>(out + (size_t)s * M);
    constexpr int U = 4;  // independent 16-byte loads in flight per lane and choice
    for (int base = 0; base < row_vecs; base += 32 * U) {
      P p[K][U];
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (!keep[j]) continue;
        const P* srow = reinterpret_cast<const P*>(src + (size_t)row[j] * M);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = base + u * 32 + lane;
          if (v < row_vecs) p[j][u] = srow[v];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = base + u * 32 + lane;
        if (v >= row_vecs) continue;
        float acc[N];
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) {
          if (!keep[j]) continue;
#pragma unroll
          for (int i = 0; i < N; ++i) {
            const float prod = __fmul_rn(g[j], Num<T>::to_f(p[j][u].v[i]));
            acc[i] = (j == 0 || !keep[0]) ? prod : __fadd_rn(acc[i], prod);
          }
        }
        P o;
#pragma unroll
        for (int i = 0; i < N; ++i) o.v[i] = Num<T>::from_f(acc[i]);
        dst[v] = o;
      }
    }
  }
}

// --------------------------------------------------------------------------------------------
// decode_dx: d_expert[row_j] = g[j,s] * dy[s]; rows nobody owns are zero.
// --------------------------------------------------------------------------------------------
template <typename T, int N, int K>
__global__ void __launch_bounds__(kRowThreads)
scatter_scaled_rows_kernel(const void* __restrict__ gates, int gates_dtype, const int32_t* __restrict__ idx_loc,
                           const int32_t* __restrict__ rows_used, const T* __restrict__ dy, T* __restrict__ out, int S,
                           int M, int C, int E, int zero_tail) {
  using P = Pack<T, N>;
  const int lane = threadIdx.x & 31;
  const int row_vecs = M / N;
  const long long gw = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kRowWarps;
  const long long ntasks = (long long)S + (zero_tail ? (long long)E * C : 0);
  for (long long task = gw; task < ntasks; task += nwarps) {
    if (task < S) {
      const int s = (int)task;
      long long row[K];
      bool keep[K];
      float g[K];
      bool any = false;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        keep[j] = kept_choice(idx_loc, nullptr, j, s, S, 2 * K, C, E, false, &row[j]);
        g[j] = load_as_float(gates, gates_dtype, (size_t)j * S + s);
        any |= keep[j];
      }
      if (!any) continue;
      const P* srcp = reinterpret_cast<const P*>(dy + (size_t)s * M);
      for (int v = lane; v < row_vecs; v += 32) {
        const P p = srcp[v];
#pragma unroll
        for (int j = 0; j < K; ++j) {
          if (!keep[j]) continue;
          P o;
#pragma unroll
          for (int i = 0; i < N; ++i) o.v[i] = Num<T>::from_f(__fmul_rn(g[j], Num<T>::to_f(p.v[i])));
          reinterpret_cast<P*>(out + (size_t)row[j] * M)[v] = o;
        }
      }
    } else {
      const long long r = task - S;
      const int e = (int)(r / C);
      const int c = (int)(r % C);
      if (c < rows_used[e]) continue;
      P z;
      memset(&z, 0, sizeof(P));
      P* dst = reinterpret_cast<P*>(out + (size_t)r * M);
      for (int v = lane; v < row_vecs; v += 32) dst[v] = z;
    }
  }
}

// --------------------------------------------------------------------------------------------
// decode_dg: dgate[j,s] = <expert_out[row_j], dy[s]>, accumulated in fp32; one warp per (s, j).
// --------------------------------------------------------------------------------------------
template <typename T, int N>
__global__ void __launch_bounds__(kRowThreads)
rowdot_kernel(const int32_t* __restrict__ idx_loc, int K, const T* __restrict__ dy, const T* __restrict__ eo,
              void* __restrict__ dgates, int gates_dtype, int S, int M, int C, int E) {
  using P = Pack<T, N>;
  const int lane = threadIdx.x & 31;
  const int row_vecs = M / N;
  const long long gw = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kRowWarps;
  const long long ntasks = (long long)S * K;
  for (long long task = gw; task < ntasks; task += nwarps) {
    const int j = (int)(task / S);
    const int s = (int)(task % S);
    long long row;
    float sum = 0.f;
    if (kept_choice(idx_loc, nullptr, j, s, S, 2 * K, C, E, false, &row)) {
      const P* a = reinterpret_cast<const P*>(eo + (size_t)row * M);
      const P* b = reinterpret_cast<const P*>(dy + (size_t)s * M);
      float part[4] = {0.f, 0.f, 0.f, 0.f};
      for (int v = lane; v < row_vecs; v += 32) {
        const P pa = a[v];
        const P pb = b[v];
#pragma unroll
        for (int i = 0; i < N; ++i) part[i & 3] = fmaf(Num<T>::to_f(pa.v[i]), Num<T>::to_f(pb.v[i]), part[i & 3]);
      }
      sum = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    }
    if (lane == 0) store_from_float(dgates, gates_dtype, (size_t)j * S + s, sum);
  }
}

// --------------------------------------------------------------------------------------------
// encode_dg: dense [S,E] gradient of the gate matrix, written once (no memset).
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gate_grad_kernel(const void* __restrict__ dy_gates, int gates_dtype, const int32_t* __restrict__ idx_loc, int K,
                 const void* __restrict__ gate, int gate_dtype, void* __restrict__ dgate, int S, int E) {
  const long long n = (long long)S * E;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int s = (int)(i / E);
    const int e = (int)(i % E);
    float val = 0.f;
    if (K == 1) {
      if (idx_loc[s] == e) val = load_as_float(dy_gates, gates_dtype, s);
    } else {
      const int i0 = idx_loc[s];
      const int i1 = idx_loc[(size_t)2 * S + s];
      if (e == i0 || e == i1) {
        const bool k0 = i0 >= 0 && i0 < E, k1 = i1 >= 0 && i1 < E;
        const float g0 = k0 ? load_as_float(gate, gate_dtype, (size_t)s * E + i0) : 0.f;
        const float g1 = k1 ? load_as_float(gate, gate_dtype, (size_t)s * E + i1) : 0.f;
        const float eps = 1.1920928955078125e-07f;
        const float sum = __fadd_rn(g0, g1);
        const float D = fmaxf(sum, eps);
        const float G0 = __fdiv_rn(g0, D), G1 = __fdiv_rn(g1, D);
        const float d0 = load_as_float(dy_gates, gates_dtype, s);
        const float d1 = load_as_float(dy_gates, gates_dtype, (size_t)S + s);
        const float dot = __fadd_rn(__fmul_rn(d0, G0), __fmul_rn(d1, G1));
        const float dj = (e == i0) ? d0 : d1;
        val = sum > eps ? __fdiv_rn(__fsub_rn(dj, dot), D) : __fdiv_rn(dj, D);
      }
    }
    store_from_float(dgate, gate_dtype, (size_t)i, val);
  }
}

// ---------------------------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------------------------
static int row_grid(long long tasks) {
  long long ctas = (tasks + kRowWarps - 1) / kRowWarps;
  const long long cap = (long long)sm_count() * 8;
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  return (int)ctas;
}

template <typename V>
static int dispatch_launch_v(const int32_t* idx_loc, int k, const int32_t* in_cap, const int32_t* rows_hi,
                             const int32_t* rows_lo, const void* x, void* out, int S, int Sp, size_t row_bytes, int C,
                             int E, int global_loc, int zero_tail, cudaStream_t stream) {
  const int row_vecs = (int)(row_bytes / sizeof(V));
  const long long tasks = (long long)S + (zero_tail ? (long long)E * C : 0);
  const int grid = row_grid(tasks);
  ProfScope prof("dispatch_rows_kernel", stream);
  if (k == 1)
    launch_chained(dispatch_rows_kernel<V, 1>, grid, kRowThreads, 0, stream, idx_loc, in_cap, rows_hi, rows_lo,
                   static_cast<const V*>(x), static_cast<V*>(out), S, Sp > 0 ? Sp : 1, row_vecs, C, E, global_loc, zero_tail);
  else
    launch_chained(dispatch_rows_kernel<V, 2>, grid, kRowThreads, 0, stream, idx_loc, in_cap, rows_hi, rows_lo,
                   static_cast<const V*>(x), static_cast<V*>(out), S, Sp > 0 ? Sp : 1, row_vecs, C, E, global_loc, zero_tail);
  return launch_status("dispatch_rows_kernel");
}

int dispatch_launch(const int32_t* idx_loc, int k, const int32_t* in_cap, const int32_t* rows_hi, const int32_t* rows_lo,
                    const void* x, void* out, int S, int Sp, int M, int C, int E, int dtype, int flags,
                    cudaStream_t stream) {
  const size_t row_bytes = (size_t)M * dtype_bytes(dtype);
  const int global_loc = (flags & LANCET_ENCODE_GLOBAL_LOC) ? 1 : 0;
  int zero_tail = 0;
  if (!(flags & LANCET_ENCODE_NO_ZERO)) {
    if (rows_hi && !global_loc) {
      zero_tail = 1;
    } else {
      LANCET_CUDA(cudaMemsetAsync(out, 0, (size_t)E * C * row_bytes, stream));
    }
  }
  if (S == 0 && !zero_tail) return LANCET_OK;
  if (row_bytes == 0 || (long long)S + (zero_tail ? (long long)E * C : 0) == 0) return LANCET_OK;
  if (row_bytes % 16 == 0 && aligned(x, 16) && aligned(out, 16))
    return dispatch_launch_v<uint4>(idx_loc, k, in_cap, rows_hi, rows_lo, x, out, S, Sp, row_bytes, C, E, global_loc,
                                    zero_tail, stream);
  if (row_bytes % 4 == 0 && aligned(x, 4) && aligned(out, 4))
    return dispatch_launch_v<uint32_t>(idx_loc, k, in_cap, rows_hi, rows_lo, x, out, S, Sp, row_bytes, C, E, global_loc,
                                       zero_tail, stream);
  return dispatch_launch_v<uint16_t>(idx_loc, k, in_cap, rows_hi, rows_lo, x, out, S, Sp, row_bytes, C, E, global_loc,
                                     zero_tail, stream);
}

template <typename T>
static int combine_launch_t(const void* gates, int gates_dtype, const int32_t* idx_loc, int k, const void* src,
                            void* out, int S, int Sp, int M, int C, int E, cudaStream_t stream) {
  constexpr int N = 16 / sizeof(T);
  const bool vec = (M % N == 0) && aligned(src, 16) && aligned(out, 16);
  const int grid = row_grid(S);
  const T* s_ = static_cast<const T*>(src);
  T* o_ = static_cast<T*>(out);
  ProfScope prof("combine_rows_kernel", stream);
  if (vec) {
    if (k == 1)
      launch_chained(combine_rows_kernel<T, N, 1>, grid, kRowThreads, 0, stream, gates, gates_dtype, idx_loc, s_, o_, S, Sp, M, C, E);
    else
      launch_chained(combine_rows_kernel<T, N, 2>, grid, kRowThreads, 0, stream, gates, gates_dtype, idx_loc, s_, o_, S, Sp, M, C, E);
  } else {
    if (k == 1)
      launch_chained(combine_rows_kernel<T, 1, 1>, grid, kRowThreads, 0, stream, gates, gates_dtype, idx_loc, s_, o_, S, Sp, M, C, E);
    else
      launch_chained(combine_rows_kernel<T, 1, 2>, grid, kRowThreads, 0, stream, gates, gates_dtype, idx_loc, s_, o_, S, Sp, M, C, E);
  }
  return launch_status("combine_rows_kernel");
}

int combine_launch(const void* gates, int gates_dtype, const int32_t* idx_loc, int k, const void* src, void* out, int S,
                   int Sp, int M, int C, int E, int dtype, cudaStream_t stream) {
  if (S == 0 || M == 0) return LANCET_OK;
  return LANCET_DISPATCH_DTYPE(dtype, combine_launch_t, gates, gates_dtype, idx_loc, k, src, out, S, Sp, M, C, E, stream);
}

template <typename T>
static int scatter_scaled_launch_t(const void* gates, int gates_dtype, const int32_t* idx_loc, int k,
                                   const int32_t* rows_used, const void* dy, void* out, int S, int M, int C, int E,
                                   cudaStream_t stream) {
  constexpr int N = 16 / sizeof(T);
  const bool vec = (M % N == 0) && aligned(dy, 16) && aligned(out, 16);
  const int zero_tail = rows_used ? 1 : 0;
  if (!zero_tail) LANCET_CUDA(cudaMemsetAsync(out, 0, (size_t)E * C * M * sizeof(T), stream));
  const long long tasks = (long long)S + (zero_tail ? (long long)E * C : 0);
  if (tasks == 0 || M == 0) return LANCET_OK;
  const int grid = row_grid(tasks);
  const T* d_ = static_cast<const T*>(dy);
  T* o_ = static_cast<T*>(out);
#define LANCET_SS(NN, KK)                                                                                         \
  scatter_scaled_rows_kernel<T, NN, KK><<<grid, kRowThreads, 0, stream>>>(gates, gates_dtype, idx_loc, rows_used, d_, \
                                                                          o_, S, M, C, E, zero_tail)
  if (vec) {
    if (k == 1) LANCET_SS(N, 1); else LANCET_SS(N, 2);
  } else {
    if (k == 1) LANCET_SS(1, 1); else LANCET_SS(1, 2);
  }
#undef LANCET_SS
  return launch_status("scatter_scaled_rows_kernel");
}

int scatter_scaled_launch(const void* gates, int gates_dtype, const int32_t* idx_loc, int k, const int32_t* rows_used,
                          const void* dy, void* out, int S, int M, int C, int E, int dtype, cudaStream_t stream) {
  return LANCET_DISPATCH_DTYPE(dtype, scatter_scaled_launch_t, gates, gates_dtype, idx_loc, k, rows_used, dy, out, S, M,
                               C, E, stream);
}

template <typename T>
static int rowdot_launch_t(const int32_t* idx_loc, int k, const void* dy, const void* eo, void* dgates, int gates_dtype,
                           int S, int M, int C, int E, cudaStream_t stream) {
  constexpr int N = 16 / sizeof(T);
  const bool vec = (M % N == 0) && aligned(dy, 16) && aligned(eo, 16);
  const int grid = row_grid((long long)S * k);
  if (vec)
    rowdot_kernel<T, N><<<grid, kRowThreads, 0, stream>>>(idx_loc, k, static_cast<const T*>(dy),
                                                          static_cast<const T*>(eo), dgates, gates_dtype, S, M, C, E);
  else
    rowdot_kernel<T, 1><<<grid, kRowThreads, 0, stream>>>(idx_loc, k, static_cast<const T*>(dy),
                                                          static_cast<const T*>(eo), dgates, gates_dtype, S, M, C, E);
  return launch_status("rowdot_kernel");
}

int rowdot_launch(const int32_t* idx_loc, int k, const void* dy, const void* eo, void* dgates, int gates_dtype, int S,
                  int M, int C, int E, int dtype, cudaStream_t stream) {
  if (S == 0) return LANCET_OK;
  return LANCET_DISPATCH_DTYPE(dtype, rowdot_launch_t, idx_loc, k, dy, eo, dgates, gates_dtype, S, M, C, E, stream);
}

}  // namespace lancet

extern "C" {
using namespace lancet;

#define CHECK_COMMON(fn, S, M, C, E, k, dtype)                                                                     \
  LANCET_REQUIRE((k) == 1 || (k) == 2, LANCET_ERR_INVALID, fn ": k must be 1 or 2, got %d", (k));                  \
  LANCET_REQUIRE((S) >= 0 && (M) >= 0 && (C) >= 0 && (E) > 0, LANCET_ERR_INVALID,                                  \
                 fn ": bad sizes S=%d M=%d C=%d E=%d", (S), (M), (C), (E));                                        \
  LANCET_REQUIRE((long long)(E) * (C) < (1ll << 31), LANCET_ERR_INVALID, fn ": E*C=%lld rows exceed 2^31",          \
                 (long long)(E) * (C));                                                                            \
  LANCET_REQUIRE(valid_dtype(dtype), LANCET_ERR_INVALID, fn ": unknown dtype code %d", (dtype))

int lancet_moe_encode_fwd(const int32_t* idx_loc, int k, const int32_t* in_capused, const int32_t* rows_hi,
                          const int32_t* rows_lo, const void* x, void* dispatched, int S, int M, int C, int E, int dtype,
                          int flags, lancet_stream_t stream) {
  CHECK_COMMON("lancet_moe_encode_fwd", S, M, C, E, k, dtype);
  LANCET_REQUIRE((flags & ~3) == 0, LANCET_ERR_INVALID, "lancet_moe_encode_fwd: unknown flag bits 0x%x", flags);
  LANCET_REQUIRE((S == 0 || (idx_loc && x)) && ((size_t)E * C * M == 0 || dispatched), LANCET_ERR_NULL,
                 "lancet_moe_encode_fwd: null pointer argument");
  LANCET_REQUIRE(!(flags & LANCET_ENCODE_GLOBAL_LOC) || in_capused, LANCET_ERR_NULL,
                 "lancet_moe_encode_fwd: LANCET_ENCODE_GLOBAL_LOC needs in_capused");
  LANCET_REQUIRE(aligned(x, dtype_bytes(dtype)) && aligned(dispatched, dtype_bytes(dtype)), LANCET_ERR_INVALID,
                 "lancet_moe_encode_fwd: data pointers are not aligned to the element size");
  return dispatch_launch(idx_loc, k, in_capused, rows_hi, rows_lo, x, dispatched, S, S, M, C, E, dtype, flags,
                         static_cast<cudaStream_t>(stream));
}

int lancet_moe_zero_tail(void* dispatched, const int32_t* used, int M, int C, int E, int dtype, lancet_stream_t stream) {
  CHECK_COMMON("lancet_moe_zero_tail", 0, M, C, E, 1, dtype);
  LANCET_REQUIRE(used && ((size_t)E * C * M == 0 || dispatched), LANCET_ERR_NULL, "lancet_moe_zero_tail: null pointer argument");
  if ((size_t)E * C * M == 0) return LANCET_OK;
  // token part is empty (S = 0): only the zero-row tasks run
  return dispatch_launch(nullptr, 1, nullptr, used, nullptr, nullptr, dispatched, 0, 1, M, C, E, dtype, 0,
                         static_cast<cudaStream_t>(stream));
}

int lancet_moe_encode(const void* x, const void* gate, int gate_dtype, const int32_t* in_capused, float capacity_factor,
                      int S, int M, int E, int k, int dtype, void* out_gates_s, int gates_dtype, int32_t* out_idx_loc,
                      int32_t* out_capused, uint64_t* out_elems, void* dispatched, void* ws, size_t ws_bytes, int flags,
                      lancet_stream_t stream) {
  LANCET_REQUIRE(E > 0 && (k == 1 || k == 2) && S >= 0, LANCET_ERR_INVALID, "lancet_moe_encode: bad sizes S=%d E=%d k=%d", S, E, k);
  const int C = lancet_moe_capacity(S, E, capacity_factor, k);
  LANCET_REQUIRE(C >= 0, LANCET_ERR_INVALID, "lancet_moe_encode: capacity %d from factor %f is negative", C, capacity_factor);
  LANCET_REQUIRE((flags & ~3) == 0, LANCET_ERR_INVALID, "lancet_moe_encode: unknown flag bits 0x%x", flags);
  const int global_loc = flags & LANCET_ENCODE_GLOBAL_LOC;
  int st = lancet_moe_gate(gate, gate_dtype, S, E, k, in_capused, C, M, out_gates_s, gates_dtype, out_idx_loc,
                           out_capused, out_elems, ws, ws_bytes, global_loc ? LANCET_GATE_GLOBAL_LOC : 0, stream);
  if (st != LANCET_OK) return st;
  if (global_loc)  // locations already include the used capacity: rows of earlier chunks stay untouched
    return lancet_moe_encode_fwd(out_idx_loc, k, nullptr, nullptr, nullptr, x, dispatched, S, M, C, E, dtype,
                                 LANCET_ENCODE_NO_ZERO, stream);
  return lancet_moe_encode_fwd(out_idx_loc, k, in_capused, out_capused, in_capused, x, dispatched, S, M, C, E, dtype,
                               flags, stream);
}

int lancet_moe_decode_fwd(const void* gates_s, int gates_dtype, const int32_t* idx_loc, int k, const void* expert_out,
                          void* out, int S, int M, int C, int E, int dtype, lancet_stream_t stream) {
  CHECK_COMMON("lancet_moe_decode_fwd", S, M, C, E, k, dtype);
  LANCET_REQUIRE(valid_dtype(gates_dtype), LANCET_ERR_INVALID, "lancet_moe_decode_fwd: unknown gates dtype %d", gates_dtype);
  LANCET_REQUIRE(S == 0 || M == 0 || (gates_s && idx_loc && expert_out && out), LANCET_ERR_NULL,
                 "lancet_moe_decode_fwd: null pointer argument");
  return combine_launch(gates_s, gates_dtype, idx_loc, k, expert_out, out, S, S, M, C, E, dtype,
                        static_cast<cudaStream_t>(stream));
}

int lancet_moe_encode_bwd_data(const int32_t* idx_loc, int k, const void* dy_dispatched, void* dx, int S, int M, int C,
                               int E, int dtype, lancet_stream_t stream) {
  CHECK_COMMON("lancet_moe_encode_bwd_data", S, M, C, E, k, dtype);
  LANCET_REQUIRE(S == 0 || M == 0 || (idx_loc && dy_dispatched && dx), LANCET_ERR_NULL,
                 "lancet_moe_encode_bwd_data: null pointer argument");
  return combine_launch(nullptr, LANCET_F32, idx_loc, k, dy_dispatched, dx, S, S, M, C, E, dtype,
                        static_cast<cudaStream_t>(stream));
}

int lancet_moe_encode_bwd_gate(const void* dy_gates_s, int gates_dtype, const int32_t* idx_loc, int k, const void* gate,
                               int gate_dtype, void* dgate, int S, int E, lancet_stream_t stream) {
  LANCET_REQUIRE(k == 1 || k == 2, LANCET_ERR_INVALID, "lancet_moe_encode_bwd_gate: k must be 1 or 2, got %d", k);
  LANCET_REQUIRE(S >= 0 && E > 0, LANCET_ERR_INVALID, "lancet_moe_encode_bwd_gate: bad sizes S=%d E=%d", S, E);
  LANCET_REQUIRE(valid_dtype(gates_dtype) && valid_dtype(gate_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_encode_bwd_gate: unknown dtype code");
  if (S == 0) return LANCET_OK;
  LANCET_REQUIRE(dy_gates_s && idx_loc && dgate && (k == 1 || gate), LANCET_ERR_NULL,
                 "lancet_moe_encode_bwd_gate: null pointer argument");
  const long long n = (long long)S * E;
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  gate_grad_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(dy_gates_s, gates_dtype, idx_loc, k, gate,
                                                                               gate_dtype, dgate, S, E);
  return launch_status("gate_grad_kernel");
}

int lancet_moe_decode_bwd_data(const void* gates_s, int gates_dtype, const int32_t* idx_loc, int k, const void* dy,
                               void* d_expert, const int32_t* rows_used, int S, int M, int C, int E, int dtype,
                               lancet_stream_t stream) {
  CHECK_COMMON("lancet_moe_decode_bwd_data", S, M, C, E, k, dtype);
  LANCET_REQUIRE(valid_dtype(gates_dtype), LANCET_ERR_INVALID, "lancet_moe_decode_bwd_data: unknown gates dtype %d", gates_dtype);
  LANCET_REQUIRE((S == 0 || (gates_s && idx_loc && dy)) && ((size_t)E * C * M == 0 || d_expert), LANCET_ERR_NULL,
                 "lancet_moe_decode_bwd_data: null pointer argument");
  if ((size_t)E * C * M == 0) return LANCET_OK;
  return scatter_scaled_launch(gates_s, gates_dtype, idx_loc, k, rows_used, dy, d_expert, S, M, C, E, dtype,
                               static_cast<cudaStream_t>(stream));
}

int lancet_moe_decode_bwd_gate(const int32_t* idx_loc, int k, const void* dy, const void* expert_out, void* dgates_s,
                               int gates_dtype, int S, int M, int C, int E, int dtype, lancet_stream_t stream) {
  CHECK_COMMON("lancet_moe_decode_bwd_gate", S, M, C, E, k, dtype);
  LANCET_REQUIRE(valid_dtype(gates_dtype), LANCET_ERR_INVALID, "lancet_moe_decode_bwd_gate: unknown gates dtype %d", gates_dtype);
  LANCET_REQUIRE(S == 0 || (idx_loc && dgates_s && (M == 0 || (dy && expert_out))), LANCET_ERR_NULL,
                 "lancet_moe_decode_bwd_gate: null pointer argument");
  return rowdot_launch(idx_loc, k, dy, expert_out, dgates_s, gates_dtype, S, M, C, E, dtype,
                       static_cast<cudaStream_t>(stream));
}
}
