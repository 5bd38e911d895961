// Expert-parallel exchange fused into dispatch and combine over NVLink peer memory.
//
// The reference moves the [E,C,M] expert buffer with an NCCL all-to-all after dispatch and again
// before combine (NCCLAllToAll::Execute, src/op/dialect/nccl/nccl.cc:199-227; layer in
// models/benchmark/pytorch/utils.py:576-634): scatter to a local buffer, copy it through NCCL
// send/recv kernels, read it again on the other side.  Here the scatter itself writes each token
// row into the receive buffer of the GPU that owns the expert (16-byte peer stores through
// NVSwitch), and combine gathers rows straight from the owners' output buffers (peer loads), so
// every row crosses NVLink once and is never staged.  Rank r owns experts [r*LE, (r+1)*LE); its
// receive buffer is [G=W][LE][C][M] with block g written by rank g - exactly the layout the
// all-to-all produces.
//
// Ranks meet at a flag barrier in peer memory.  Every wait is bounded by a time limit after which
// the kernel records which peer was missing in a status word and returns.
#include "common.cuh"

namespace lancet {

constexpr int kMaxPeers = 16;
struct PeerTable {
  void* ptr[kMaxPeers];
};

// 128-thread blocks: one of them still fits beside a resident CTA of the expert GEMM (up to 168 registers x 320
// threads), so the exchange kernels make progress while a GEMM occupies every SM
constexpr int kP2PThreads = 128;
constexpr int kP2PWarps = kP2PThreads / 32;

__device__ __forceinline__ size_t il_index_p2p(int s, int Sp, int K2, int row) {
  const int c = s / Sp;
  return ((size_t)c * K2 + row) * Sp + (s - c * Sp);
}

// tasks [0,S): token rows; tasks [S, S + E*C): candidate zero rows of my block in every owner's buffer.
template <typename V, int K>
__global__ void __launch_bounds__(kP2PThreads)
dispatch_rows_peer_kernel(const int32_t* __restrict__ idx_loc, const int32_t* __restrict__ rows_used,
                          const V* __restrict__ x, PeerTable recv, PeerTable counts, int S, int Sp, int row_vecs, int C,
                          int E, int LE, int my_rank, int zero_tail) {
  constexpr int U = 8;
  chain_enter();
  const int lane = threadIdx.x & 31;
  if (!zero_tail && blockIdx.x == 0 && counts.ptr[0] != nullptr) {
    // tell every owner how many rows of my block it received; it zero-fills the rest locally
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int owner = e / LE, le = e - owner * LE;
      static_cast<int32_t*>(counts.ptr[owner])[my_rank * LE + le] = rows_used[e];
    }
  }
  const long long gw = (long long)blockIdx.x * kP2PWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kP2PWarps;
  const long long ntasks = (long long)S + (zero_tail ? (long long)E * C : 0);
  for (long long task = gw; task < ntasks; task += nwarps) {
    if (task < S) {
      const int s = (int)task;
      V* dst[K];
      bool any = false;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const int idx = idx_loc[il_index_p2p(s, Sp, 2 * K, 2 * j)];
        const int loc = idx_loc[il_index_p2p(s, Sp, 2 * K, 2 * j + 1)];
        dst[j] = nullptr;
        if (idx >= 0 && idx < E && loc >= 0 && loc < C) {
          const int owner = idx / LE, le = idx - owner * LE;
          dst[j] = static_cast<V*>(recv.ptr[owner]) + ((size_t)(my_rank * LE + le) * C + loc) * row_vecs;
          any = true;
        }
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
          if (!dst[j]) continue;
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int v = base + u * 32 + lane;
            if (v < row_vecs) dst[j][v] = r[u];
          }
        }
      }
    } else {
      const long long r = task - S;
      const int e = (int)(r / C);
      const int c = (int)(r % C);
      if (c < rows_used[e]) continue;
      const int owner = e / LE, le = e - owner * LE;
      V* d = static_cast<V*>(recv.ptr[owner]) + ((size_t)(my_rank * LE + le) * C + c) * row_vecs;
      V z;
      memset(&z, 0, sizeof(V));
      for (int v = lane; v < row_vecs; v += 32) d[v] = z;
    }
  }
}

template <typename T, int N>
struct alignas(sizeof(T) * N) PackP {
  T v[N];
};

template <typename T, int N, int K>
__global__ void __launch_bounds__(kP2PThreads)
combine_rows_peer_kernel(const float* __restrict__ gates, const int32_t* __restrict__ idx_loc, PeerTable eo,
                         T* __restrict__ out, int S, int Sp, int M, int C, int E, int LE, int my_rank) {
  using P = PackP<T, N>;
  constexpr int U = 4;
  chain_enter();
  const int lane = threadIdx.x & 31;
  const int row_vecs = M / N;
  const long long gw = (long long)blockIdx.x * kP2PWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kP2PWarps;
  for (long long s = gw; s < S; s += nwarps) {
    const P* srow[K];
    float g[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int idx = idx_loc[il_index_p2p((int)s, Sp, 2 * K, 2 * j)];
      const int loc = idx_loc[il_index_p2p((int)s, Sp, 2 * K, 2 * j + 1)];
      srow[j] = nullptr;
      if (idx >= 0 && idx < E && loc >= 0 && loc < C) {
        const int owner = idx / LE, le = idx - owner * LE;
        srow[j] = reinterpret_cast<const P*>(static_cast<const T*>(eo.ptr[owner]) +
                                             ((size_t)(my_rank * LE + le) * C + loc) * M);
      }
      g[j] = gates ? gates[il_index_p2p((int)s, Sp, K, j)] : 1.0f;
    }
    P* dst = reinterpret_cast<P*>(out + (size_t)s * M);
    for (int base = 0; base < row_vecs; base += 32 * U) {
      P p[K][U];
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (!srow[j]) continue;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = base + u * 32 + lane;
          if (v < row_vecs) p[j][u] = srow[j][v];
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
          if (!srow[j]) continue;
#pragma unroll
          for (int i = 0; i < N; ++i) {
            const float prod = __fmul_rn(g[j], Num<T>::to_f(p[j][u].v[i]));
            acc[i] = (j == 0 || !srow[0]) ? prod : __fadd_rn(acc[i], prod);
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


// Backward of combine, fused with the exchange.  Per token s and choice j kept at (owner, row):
//   d_expert_out[owner][row] = gates[j,s] * dout[s]      (peer store: the transpose of the forward gather)
//   dgates[j,s]             = <expert_out[owner][row], dout[s]>   (peer load, fp32 accumulation)
// One warp per token; the row of dout is read once and used for both.
// PART 0: both halves in one pass (egress and ingress of the link busy at once); 1: only the rows sent to the owners;
// 2: only the gate gradients.  The halves meet the elements in the same order as the joint pass: same bits.
template <typename T, int N, int K, int PART>
__global__ void __launch_bounds__(kP2PThreads)
combine_bwd_peer_kernel(const float* __restrict__ gates, const int32_t* __restrict__ idx_loc, const T* __restrict__ dout,
                        PeerTable d_eo, PeerTable eo, float* __restrict__ dgates, int S, int Sp, int M, int C, int E, int LE,
                        int my_rank) {
  using P = PackP<T, N>;
  chain_enter();
  const int lane = threadIdx.x & 31;
  const int row_vecs = M / N;
  const long long gw = (long long)blockIdx.x * kP2PWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kP2PWarps;
  for (long long s = gw; s < S; s += nwarps) {
    P* drow[K];
    const P* erow[K];
    float g[K], dot[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int idx = idx_loc[il_index_p2p((int)s, Sp, 2 * K, 2 * j)];
      const int loc = idx_loc[il_index_p2p((int)s, Sp, 2 * K, 2 * j + 1)];
      drow[j] = nullptr;
      erow[j] = nullptr;
      dot[j] = 0.f;
      if (idx >= 0 && idx < E && loc >= 0 && loc < C) {
        const int owner = idx / LE, le = idx - owner * LE;
        const size_t off = ((size_t)(my_rank * LE + le) * C + loc) * M;
        drow[j] = reinterpret_cast<P*>(static_cast<T*>(d_eo.ptr[owner]) + off);
        erow[j] = reinterpret_cast<const P*>(static_cast<const T*>(eo.ptr[owner]) + off);
      }
      g[j] = gates[il_index_p2p((int)s, Sp, K, j)];
    }
    const P* src = reinterpret_cast<const P*>(dout + (size_t)s * M);
    // U vectors of the row in flight per lane (a single one left the kernel latency-bound at half the bandwidth);
    // every lane still meets its elements in the same order, so the dot products keep their bits
    constexpr int U = 4;
    for (int base = 0; base < row_vecs; base += 32 * U) {
      P d[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = base + u * 32 + lane;
        if (v < row_vecs) d[u] = src[v];
      }
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (!drow[j]) continue;
        P e[U];
        if (PART != 1) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int v = base + u * 32 + lane;
            if (v < row_vecs) e[u] = erow[j][v];
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = base + u * 32 + lane;
          if (v >= row_vecs) continue;
          P o;
#pragma unroll
          for (int i = 0; i < N; ++i) {
            const float dv = Num<T>::to_f(d[u].v[i]);
            if (PART != 2) o.v[i] = Num<T>::from_f(__fmul_rn(g[j], dv));
            if (PART != 1) dot[j] = fmaf(Num<T>::to_f(e[u].v[i]), dv, dot[j]);
          }
          if (PART != 2) drow[j][v] = o;
        }
      }
    }
    if (PART != 1) {
#pragma unroll
      for (int j = 0; j < K; ++j) {
        float t = dot[j];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
        if (lane == 0) dgates[il_index_p2p((int)s, Sp, K, j)] = t;
      }
    }
  }
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Thread i tells rank i that this rank has arrived (epoch) and waits until rank i has told us.
// flags.ptr[r] is rank r's array of W words; word i of it is written by rank i only.
// With epoch_counter != nullptr the epoch is kept in device memory (previous value + 1, written back by thread 0),
// so that the same launch can be replayed from a CUDA graph.
__global__ void p2p_barrier_kernel(PeerTable flags, int W, int my_rank, unsigned epoch, unsigned long long timeout_ns,
                                   int* __restrict__ status, unsigned* __restrict__ epoch_counter) {
  chain_enter();   // the kernels before this one on the stream have completed: their peer stores are what the flag announces
  const int i = threadIdx.x;
  if (epoch_counter) epoch = *epoch_counter + 1;
  __syncwarp();
  if (i == 0 && epoch_counter) *epoch_counter = epoch;
  if (i >= W) return;
  __threadfence_system();
  unsigned* remote = static_cast<unsigned*>(flags.ptr[i]) + my_rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const unsigned* local = static_cast<const unsigned*>(flags.ptr[my_rank]) + i;
  const unsigned long long t0 = globaltimer_ns();
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
    if ((int)(v - epoch) >= 0) break;
    if (globaltimer_ns() - t0 > timeout_ns) {
      atomicCAS(status, 0, i + 1);  // remember the first peer that did not arrive
      break;
    }
    __nanosleep(64);
  }
  __threadfence_system();
}

// Staged exchange: every rank tells the owners, before the first row travels, how the rows of its block
// will arrive: tables.ptr[owner] is int32 [W][n1][LE], entry (source, c, le) = rows of (source, expert) placed
// by the chunks before c (n1 = n_chunks + 1 entries; the last is the total).
__global__ void publish_chain_kernel(const int32_t* __restrict__ chain, PeerTable tables, int n1, int E, int LE, int my_rank,
                                     int row_begin, int row_end) {
  for (int i = row_begin * E + blockIdx.x * blockDim.x + threadIdx.x; i < row_end * E; i += gridDim.x * blockDim.x) {
    const int c = i / E, e = i - c * E;
    const int owner = e / LE, le = e - owner * LE;
    static_cast<int32_t*>(tables.ptr[owner])[((size_t)my_rank * n1 + c) * LE + le] = chain[i];
  }
}

// Row windows of the pipeline stages on the owner's side.  Stage c may work on the rows of group g = (source, le)
// that have arrived with chunks 0..c and form whole tiles of `align` rows, and must cover every row of the chunks
// before c (their tokens are combined right after stage c): end_c = max(floor(chain[c+1] / align) * align, chain[c]),
// begin_c = the tile that holds end_{c-1} (a tile a stage leaves partial is computed again by the next one, with
// the same values); the last stage ends at the total.
__device__ __forceinline__ int stage_end(const int32_t* col, int LE, int n, int align, int c0, int c1) {
  const int hi = col[(size_t)c1 * LE];
  if (c1 == n) return hi;
  const int lo = col[(size_t)c0 * LE], al = hi / align * align;
  return al > lo ? al : lo;
}
__global__ void stage_windows_kernel(const int32_t* __restrict__ chain, int W, int LE, int n, int align,
                                     int32_t* __restrict__ row_begin, int32_t* __restrict__ row_end,
                                     int32_t* __restrict__ counts) {
  const int G = W * LE, n1 = n + 1;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n * G; i += gridDim.x * blockDim.x) {
    const int c = i / G, g = i - c * G;
    const int src = g / LE, le = g - src * LE;
    const int32_t* col = chain + (size_t)src * n1 * LE + le;
    row_begin[i] = c == 0 ? 0 : stage_end(col, LE, n, align, c - 1, c) / align * align;
    row_end[i] = stage_end(col, LE, n, align, c, c + 1);
    if (c == 0 && counts) counts[g] = col[(size_t)n * LE];
  }
}

// The same for one stage that covers chunks [c0, c1), computable as soon as the chain entries up to c1 are known
// (incremental gating: chunk c is gated, published and sent before chunk c+1 is gated).
__global__ void stage_window_kernel(const int32_t* __restrict__ chain, int W, int LE, int n, int align, int prev_c0, int c0, int c1,
                                    int32_t* __restrict__ row_begin, int32_t* __restrict__ row_end, int32_t* __restrict__ counts) {
  const int G = W * LE, n1 = n + 1;
  for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < G; g += gridDim.x * blockDim.x) {
    const int src = g / LE, le = g - src * LE;
    const int32_t* col = chain + (size_t)src * n1 * LE + le;
    row_begin[g] = c0 == 0 ? 0 : stage_end(col, LE, n, align, prev_c0, c0) / align * align;
    row_end[g] = stage_end(col, LE, n, align, c0, c1);
    if (c1 == n && counts) counts[g] = col[(size_t)n * LE];
  }
}

static int p2p_grid(long long tasks) {
  long long ctas = (tasks + kP2PWarps - 1) / kP2PWarps;
  long long cap = (long long)sm_count() * 16;
  if (exchange_cta_limit() > 0 && exchange_cta_limit() < cap) cap = exchange_cta_limit();
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  return (int)ctas;
}

template <typename T>
static int combine_p2p_t(const float* gates, const int32_t* idx_loc, const PeerTable& t, void* out, int S, int Sp, int M,
                         int C, int E, int LE, int rank, int k, cudaStream_t st) {
  constexpr int N = 16 / sizeof(T);
  ProfScope prof("combine_rows_peer_kernel", st);
  if (k == 1)
    launch_chained(combine_rows_peer_kernel<T, N, 1>, p2p_grid(S), kP2PThreads, 0, st, gates, idx_loc, t, static_cast<T*>(out), S, Sp,
                                                                         M, C, E, LE, rank);
  else
    launch_chained(combine_rows_peer_kernel<T, N, 2>, p2p_grid(S), kP2PThreads, 0, st, gates, idx_loc, t, static_cast<T*>(out), S, Sp,
                                                                         M, C, E, LE, rank);
  return launch_status("combine_rows_peer_kernel");
}


template <typename T>
static int combine_bwd_p2p_t(const float* gates, const int32_t* idx_loc, const void* dout, const PeerTable& td,
                             const PeerTable& te, float* dgates, int S, int Sp, int M, int C, int E, int LE, int rank, int k,
                             int part, cudaStream_t st) {
  constexpr int N = 16 / sizeof(T);
  ProfScope prof("combine_bwd_peer_kernel", st);
#define LANCET_CB(KK, PP)                                                                                                      \
  launch_chained(combine_bwd_peer_kernel<T, N, KK, PP>, p2p_grid(S), kP2PThreads, 0, st, gates, idx_loc,                      \
                 static_cast<const T*>(dout), td, te, dgates, S, Sp, M, C, E, LE, rank)
  if (k == 1) {
    if (part == 0) LANCET_CB(1, 0);
    else if (part == 1) LANCET_CB(1, 1);
    else LANCET_CB(1, 2);
  } else {
    if (part == 0) LANCET_CB(2, 0);
    else if (part == 1) LANCET_CB(2, 1);
    else LANCET_CB(2, 2);
  }
#undef LANCET_CB
  return launch_status("combine_bwd_peer_kernel");
}
}  // namespace lancet

extern "C" {
using namespace lancet;

int lancet_symm_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  LANCET_REQUIRE(ptr && handle64 && bytes > 0, LANCET_ERR_NULL, "lancet_symm_alloc: null argument or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  LANCET_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(LANCET_ERR_CUDA, "lancet_symm_alloc: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return LANCET_OK;
}

int lancet_symm_open(const unsigned char* handle64, void** peer_ptr) {
  LANCET_REQUIRE(handle64 && peer_ptr, LANCET_ERR_NULL, "lancet_symm_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  LANCET_CUDA(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return LANCET_OK;
}

int lancet_symm_close(void* peer_ptr) {
  if (!peer_ptr) return LANCET_OK;
  LANCET_CUDA(cudaIpcCloseMemHandle(peer_ptr));
  return LANCET_OK;
}

int lancet_symm_free(void* ptr) {
  if (!ptr) return LANCET_OK;
  LANCET_CUDA(cudaFree(ptr));
  return LANCET_OK;
}

int lancet_p2p_barrier(void* const* peer_flags, int W, int rank, unsigned epoch, unsigned long long timeout_ns,
                       int32_t* status, lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W, LANCET_ERR_INVALID,
                 "lancet_p2p_barrier: bad world %d / rank %d (at most %d ranks)", W, rank, kMaxPeers);
  LANCET_REQUIRE(peer_flags && status, LANCET_ERR_NULL, "lancet_p2p_barrier: null argument");
  LANCET_REQUIRE(timeout_ns > 0 && timeout_ns <= 60ull * 1000000000ull, LANCET_ERR_INVALID,
                 "lancet_p2p_barrier: the wait limit must be in (0, 60 s]");
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < W ? peer_flags[i] : nullptr;
  for (int i = 0; i < W; ++i) LANCET_REQUIRE(t.ptr[i], LANCET_ERR_NULL, "lancet_p2p_barrier: flag pointer %d is null", i);
  launch_chained(p2p_barrier_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), t, W, rank, epoch, timeout_ns, status,
                 static_cast<unsigned*>(nullptr));
  return launch_status("p2p_barrier_kernel");
}

int lancet_p2p_barrier_counted(void* const* peer_flags, int W, int rank, uint32_t* epoch_counter, unsigned long long timeout_ns,
                               int32_t* status, lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W, LANCET_ERR_INVALID,
                 "lancet_p2p_barrier_counted: bad world %d / rank %d (at most %d ranks)", W, rank, kMaxPeers);
  LANCET_REQUIRE(peer_flags && status && epoch_counter, LANCET_ERR_NULL, "lancet_p2p_barrier_counted: null argument");
  LANCET_REQUIRE(timeout_ns > 0 && timeout_ns <= 60ull * 1000000000ull, LANCET_ERR_INVALID,
                 "lancet_p2p_barrier_counted: the wait limit must be in (0, 60 s]");
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < W ? peer_flags[i] : nullptr;
  for (int i = 0; i < W; ++i) LANCET_REQUIRE(t.ptr[i], LANCET_ERR_NULL, "lancet_p2p_barrier_counted: flag pointer %d is null", i);
  launch_chained(p2p_barrier_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), t, W, rank, 0u, timeout_ns, status, epoch_counter);
  return launch_status("p2p_barrier_kernel");
}

// Reads the status word written by bounded waits (synchronises the stream).
int lancet_p2p_status(const int32_t* status, lancet_stream_t stream) {
  LANCET_REQUIRE(status, LANCET_ERR_NULL, "lancet_p2p_status: null argument");
  int32_t h = 0;
  LANCET_CUDA(cudaMemcpyAsync(&h, status, sizeof(h), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  LANCET_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (h != 0) return fail(LANCET_ERR_TIMEOUT, "a bounded wait ran out: rank %d did not arrive at the barrier", h - 1);
  return LANCET_OK;
}

int lancet_moe_dispatch_chunked_p2p(const void* x, const void* gate, int gate_dtype, float capacity_factor, int S, int M,
                                    int LE, int W, int rank, int k, int n_chunks, int dtype, void* gates_s,
                                    int32_t* idx_loc, int32_t* capused_chain, uint64_t* elems, void* const* peer_recv,
                                    void* const* peer_counts, void* ws, size_t ws_bytes, int flags,
                                    lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W && LE >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: bad world %d / rank %d / local experts %d", W, rank, LE);
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && M >= 0 && valid_dtype(dtype) && valid_dtype(gate_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: bad k=%d, M=%d or dtype", k, M);
  LANCET_REQUIRE((flags & ~LANCET_P2P_NO_REMOTE_ZERO) == 0, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: unknown flag bits 0x%x", flags);
  LANCET_REQUIRE(peer_recv && capused_chain && elems && ws && (S == 0 || (x && gate && gates_s && idx_loc)),
                 LANCET_ERR_NULL, "lancet_moe_dispatch_chunked_p2p: null pointer argument");
  const int E = LE * W;
  const int Sp = S / n_chunks;
  const int C = lancet_moe_capacity(Sp, E, capacity_factor * n_chunks, k);
  LANCET_REQUIRE(C >= 0 && (long long)E * C < (1ll << 31), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: capacity %d out of range", C);
  const size_t row_bytes = (size_t)M * dtype_bytes(dtype);
  LANCET_REQUIRE(row_bytes % 16 == 0 && aligned(x, 16), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: rows must be a multiple of 16 bytes and 16-byte aligned");
  PeerTable t, tc;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < W ? peer_recv[i] : nullptr;
  for (int i = 0; i < kMaxPeers; ++i) tc.ptr[i] = (peer_counts && i < W) ? peer_counts[i] : nullptr;
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(t.ptr[i] && aligned(t.ptr[i], 16), LANCET_ERR_NULL, "lancet_moe_dispatch_chunked_p2p: peer buffer %d is null or unaligned", i);
  if (flags & LANCET_P2P_NO_REMOTE_ZERO)
    for (int i = 0; i < W; ++i)
      LANCET_REQUIRE(tc.ptr[i], LANCET_ERR_NULL, "lancet_moe_dispatch_chunked_p2p: LANCET_P2P_NO_REMOTE_ZERO needs peer_counts (entry %d is null)", i);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LANCET_REQUIRE(E >= k && k * E <= 1024 && (long long)n_chunks * k * E <= 8192, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: k*E=%d or n_chunks*k*E too large", k * E);
  LANCET_REQUIRE(ws_bytes >= gate_workspace_bytes(S, E, k, n_chunks) && aligned(ws, 16), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked_p2p: workspace too small or unaligned");
  int rc = gate_launch(gate, gate_dtype, S, E, k, n_chunks, nullptr, C, M, gates_s, LANCET_F32, idx_loc, capused_chain + E,
                       elems, ws, 1, st, capused_chain);
  if (rc != LANCET_OK) return rc;
  if ((size_t)E * C * M == 0) return LANCET_OK;
  const int zero_tail = (flags & LANCET_P2P_NO_REMOTE_ZERO) ? 0 : 1;
  const long long tasks = (long long)S + (zero_tail ? (long long)E * C : 0);
  const int row_vecs = (int)(row_bytes / 16);
  const int32_t* used = capused_chain + (size_t)n_chunks * E;
  ProfScope prof("dispatch_rows_peer_kernel", st);
  if (k == 1)
    launch_chained(dispatch_rows_peer_kernel<uint4, 1>, p2p_grid(tasks), kP2PThreads, 0, st,
        idx_loc, used, static_cast<const uint4*>(x), t, tc, S, Sp > 0 ? Sp : 1, row_vecs, C, E, LE, rank, zero_tail);
  else
    launch_chained(dispatch_rows_peer_kernel<uint4, 2>, p2p_grid(tasks), kP2PThreads, 0, st,
        idx_loc, used, static_cast<const uint4*>(x), t, tc, S, Sp > 0 ? Sp : 1, row_vecs, C, E, LE, rank, zero_tail);
  return launch_status("dispatch_rows_peer_kernel");
}

int lancet_moe_gate_chunked_p2p(const void* gate, int gate_dtype, float capacity_factor, int S, int M, int LE, int W, int rank,
                                int k, int n_chunks, void* gates_s, int32_t* idx_loc, int32_t* capused_chain, uint64_t* elems,
                                void* const* peer_chain, void* ws, size_t ws_bytes, lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W && LE >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunked_p2p: bad world %d / rank %d / local experts %d", W, rank, LE);
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunked_p2p: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && M >= 0 && valid_dtype(gate_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunked_p2p: bad k=%d, M=%d or dtype", k, M);
  LANCET_REQUIRE(peer_chain && capused_chain && elems && ws && (S == 0 || (gate && gates_s && idx_loc)), LANCET_ERR_NULL,
                 "lancet_moe_gate_chunked_p2p: null pointer argument");
  const int E = LE * W;
  const int Sp = S / n_chunks;
  const int C = lancet_moe_capacity(Sp, E, capacity_factor * n_chunks, k);
  LANCET_REQUIRE(C >= 0 && (long long)E * C < (1ll << 31), LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunked_p2p: capacity %d out of range", C);
  LANCET_REQUIRE(E >= k && k * E <= 1024 && (long long)n_chunks * k * E <= 8192, LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunked_p2p: k*E=%d or n_chunks*k*E too large", k * E);
  LANCET_REQUIRE(ws_bytes >= gate_workspace_bytes(S, E, k, n_chunks) && aligned(ws, 16), LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunked_p2p: workspace too small or unaligned");
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < W ? peer_chain[i] : nullptr;
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(t.ptr[i] && aligned(t.ptr[i], 4), LANCET_ERR_NULL, "lancet_moe_gate_chunked_p2p: chain table %d is null or unaligned", i);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = gate_launch(gate, gate_dtype, S, E, k, n_chunks, nullptr, C, M, gates_s, LANCET_F32, idx_loc, capused_chain + E,
                       elems, ws, 1, st, capused_chain);
  if (rc != LANCET_OK) return rc;
  const int n1 = n_chunks + 1;
  publish_chain_kernel<<<1, 256, 0, st>>>(capused_chain, t, n1, E, LE, rank, 0, n1);
  return launch_status("publish_chain_kernel");
}

int lancet_moe_gate_chunks_p2p(const void* gate_rows, int gate_dtype, float capacity_factor, int S, int M, int LE, int W, int rank,
                               int k, int n_chunks, int chunk_begin, int chunk_end, void* gates_s, int32_t* idx_loc,
                               int32_t* capused_chain, uint64_t* elems, void* const* peer_chain, void* ws, size_t ws_bytes,
                               lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W && LE >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunks_p2p: bad world %d / rank %d / local experts %d", W, rank, LE);
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunks_p2p: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE(chunk_begin >= 0 && chunk_begin < chunk_end && chunk_end <= n_chunks, LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunks_p2p: bad chunk range [%d, %d) of %d", chunk_begin, chunk_end, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && M >= 0 && valid_dtype(gate_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunks_p2p: bad k=%d, M=%d or dtype", k, M);
  LANCET_REQUIRE(peer_chain && capused_chain && elems && ws && (S == 0 || (gate_rows && gates_s && idx_loc)), LANCET_ERR_NULL,
                 "lancet_moe_gate_chunks_p2p: null pointer argument");
  const int E = LE * W;
  const int Sp = S / n_chunks;
  const int nsub = chunk_end - chunk_begin;
  const int C = lancet_moe_capacity(Sp, E, capacity_factor * n_chunks, k);
  LANCET_REQUIRE(C >= 0 && (long long)E * C < (1ll << 31), LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunks_p2p: capacity %d out of range", C);
  LANCET_REQUIRE(E >= k && k * E <= 1024 && (long long)n_chunks * k * E <= 8192, LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunks_p2p: k*E=%d or n_chunks*k*E too large", k * E);
  LANCET_REQUIRE(ws_bytes >= gate_workspace_bytes(nsub * Sp, E, k, nsub) && aligned(ws, 16), LANCET_ERR_INVALID,
                 "lancet_moe_gate_chunks_p2p: workspace too small or unaligned");
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < W ? peer_chain[i] : nullptr;
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(t.ptr[i] && aligned(t.ptr[i], 4), LANCET_ERR_NULL, "lancet_moe_gate_chunks_p2p: chain table %d is null or unaligned", i);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the chunks see the capacity used by the chunks before them: row chunk_begin of the chain (row 0 = zeros, written here)
  const int32_t* in_cap = chunk_begin == 0 ? nullptr : capused_chain + (size_t)chunk_begin * E;
  float* gs = static_cast<float*>(gates_s) + (size_t)chunk_begin * k * Sp;
  int rc = gate_launch(gate_rows, gate_dtype, nsub * Sp, E, k, nsub, in_cap, C, M, gs, LANCET_F32,
                       idx_loc + (size_t)chunk_begin * 2 * k * Sp, capused_chain + (size_t)(chunk_begin + 1) * E,
                       elems + (size_t)chunk_begin * E, ws, 1, st, chunk_begin == 0 ? capused_chain : nullptr);
  if (rc != LANCET_OK) return rc;
  publish_chain_kernel<<<1, 256, 0, st>>>(capused_chain, t, n_chunks + 1, E, LE, rank, chunk_begin == 0 ? 0 : chunk_begin + 1,
                                          chunk_end + 1);
  return launch_status("publish_chain_kernel");
}

int lancet_moe_stage_window(const int32_t* chain, int W, int LE, int n_chunks, int row_align, int prev_chunk_begin, int chunk_begin,
                            int chunk_end, int32_t* row_begin, int32_t* row_end, int32_t* counts, lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && LE >= 1 && n_chunks >= 1 && row_align >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_stage_window: bad world %d / local experts %d / chunks %d / alignment %d", W, LE, n_chunks, row_align);
  LANCET_REQUIRE(chunk_begin >= 0 && chunk_begin < chunk_end && chunk_end <= n_chunks, LANCET_ERR_INVALID,
                 "lancet_moe_stage_window: bad chunk range [%d, %d) of %d", chunk_begin, chunk_end, n_chunks);
  LANCET_REQUIRE(chunk_begin == 0 || (prev_chunk_begin >= 0 && prev_chunk_begin < chunk_begin), LANCET_ERR_INVALID,
                 "lancet_moe_stage_window: the previous stage must start before chunk %d (got %d)", chunk_begin, prev_chunk_begin);
  LANCET_REQUIRE(chain && row_begin && row_end, LANCET_ERR_NULL, "lancet_moe_stage_window: null pointer argument");
  const int G = W * LE;
  stage_window_kernel<<<(G + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      chain, W, LE, n_chunks, row_align, prev_chunk_begin, chunk_begin, chunk_end, row_begin, row_end, counts);
  return launch_status("stage_window_kernel");
}

int lancet_moe_dispatch_rows_p2p(const void* x, const int32_t* idx_loc, int S, int M, int C, int LE, int W, int rank, int k,
                                 int n_chunks, int chunk_begin, int chunk_end, int dtype, void* const* peer_recv,
                                 lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W && LE >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_rows_p2p: bad world %d / rank %d / local experts %d", W, rank, LE);
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_rows_p2p: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE(chunk_begin >= 0 && chunk_begin <= chunk_end && chunk_end <= n_chunks, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_rows_p2p: bad chunk range [%d, %d) of %d", chunk_begin, chunk_end, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && M >= 0 && C >= 0 && valid_dtype(dtype), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_rows_p2p: bad k=%d, M=%d, C=%d or dtype", k, M, C);
  const int E = LE * W, Sp = S / n_chunks;
  LANCET_REQUIRE((long long)E * C < (1ll << 31), LANCET_ERR_INVALID, "lancet_moe_dispatch_rows_p2p: capacity %d out of range", C);
  const long long tokens = (long long)(chunk_end - chunk_begin) * Sp;
  if (tokens == 0 || M == 0 || C == 0) return LANCET_OK;
  LANCET_REQUIRE(x && idx_loc && peer_recv, LANCET_ERR_NULL, "lancet_moe_dispatch_rows_p2p: null pointer argument");
  const size_t row_bytes = (size_t)M * dtype_bytes(dtype);
  LANCET_REQUIRE(row_bytes % 16 == 0 && aligned(x, 16), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_rows_p2p: rows must be a multiple of 16 bytes and 16-byte aligned");
  PeerTable t, none;
  for (int i = 0; i < kMaxPeers; ++i) {
    t.ptr[i] = i < W ? peer_recv[i] : nullptr;
    none.ptr[i] = nullptr;
  }
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(t.ptr[i] && aligned(t.ptr[i], 16), LANCET_ERR_NULL, "lancet_moe_dispatch_rows_p2p: peer buffer %d is null or unaligned", i);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int row_vecs = (int)(row_bytes / 16);
  const uint4* xs = static_cast<const uint4*>(x) + (size_t)chunk_begin * Sp * row_vecs;
  const int32_t* il = idx_loc + (size_t)chunk_begin * 2 * k * Sp;
  ProfScope prof("dispatch_rows_peer_kernel", st);
  if (k == 1)
    launch_chained(dispatch_rows_peer_kernel<uint4, 1>, p2p_grid(tokens), kP2PThreads, 0, st, il, nullptr, xs, t, none, (int)tokens, Sp,
                                                                                 row_vecs, C, E, LE, rank, 0);
  else
    launch_chained(dispatch_rows_peer_kernel<uint4, 2>, p2p_grid(tokens), kP2PThreads, 0, st, il, nullptr, xs, t, none, (int)tokens, Sp,
                                                                                 row_vecs, C, E, LE, rank, 0);
  return launch_status("dispatch_rows_peer_kernel");
}

int lancet_moe_stage_windows(const int32_t* chain, int W, int LE, int n_chunks, int row_align, int32_t* row_begin,
                             int32_t* row_end, int32_t* counts, lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && LE >= 1 && n_chunks >= 1 && row_align >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_stage_windows: bad world %d / local experts %d / chunks %d / alignment %d", W, LE, n_chunks, row_align);
  LANCET_REQUIRE(chain && row_begin && row_end, LANCET_ERR_NULL, "lancet_moe_stage_windows: null pointer argument");
  const int total = n_chunks * W * LE;
  stage_windows_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(chain, W, LE, n_chunks, row_align,
                                                                                          row_begin, row_end, counts);
  return launch_status("stage_windows_kernel");
}

int lancet_moe_combine_chunked_p2p(void* const* peer_expert_out, const void* gates_s, const int32_t* idx_loc, int S, int M,
                                   int C, int LE, int W, int rank, int k, int n_chunks, int dtype, void* out,
                                   lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W && LE >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_combine_chunked_p2p: bad world %d / rank %d / local experts %d", W, rank, LE);
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_combine_chunked_p2p: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && M >= 0 && C >= 0 && valid_dtype(dtype), LANCET_ERR_INVALID,
                 "lancet_moe_combine_chunked_p2p: bad k=%d, M=%d, C=%d or dtype", k, M, C);
  if (S == 0 || M == 0) return LANCET_OK;
  LANCET_REQUIRE(peer_expert_out && idx_loc && out, LANCET_ERR_NULL, "lancet_moe_combine_chunked_p2p: null pointer argument");
  LANCET_REQUIRE(((size_t)M * dtype_bytes(dtype)) % 16 == 0 && aligned(out, 16), LANCET_ERR_INVALID,
                 "lancet_moe_combine_chunked_p2p: rows must be a multiple of 16 bytes and 16-byte aligned");
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < W ? peer_expert_out[i] : nullptr;
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(t.ptr[i] && aligned(t.ptr[i], 16), LANCET_ERR_NULL, "lancet_moe_combine_chunked_p2p: peer buffer %d is null or unaligned", i);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = LE * W, Sp = S / n_chunks;
  const float* g = static_cast<const float*>(gates_s);
  if (dtype == LANCET_F32) return combine_p2p_t<float>(g, idx_loc, t, out, S, Sp, M, C, E, LE, rank, k, st);
  if (dtype == LANCET_F16) return combine_p2p_t<__half>(g, idx_loc, t, out, S, Sp, M, C, E, LE, rank, k, st);
  return combine_p2p_t<__nv_bfloat16>(g, idx_loc, t, out, S, Sp, M, C, E, LE, rank, k, st);
}

int lancet_moe_combine_bwd_part_p2p(const void* dout, const void* gates_s, const int32_t* idx_loc, void* const* peer_d_expert_out,
                                    void* const* peer_expert_out, void* dgates_s, int S, int M, int C, int LE, int W, int rank,
                                    int k, int n_chunks, int dtype, int part, lancet_stream_t stream) {
  LANCET_REQUIRE(part >= 0 && part <= 2, LANCET_ERR_INVALID, "lancet_moe_combine_bwd_part_p2p: part %d is not 0, 1 or 2", part);
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeers && rank >= 0 && rank < W && LE >= 1, LANCET_ERR_INVALID,
                 "lancet_moe_combine_bwd_p2p: bad world %d / rank %d / local experts %d", W, rank, LE);
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_combine_bwd_p2p: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && M >= 0 && C >= 0 && valid_dtype(dtype), LANCET_ERR_INVALID,
                 "lancet_moe_combine_bwd_p2p: bad k=%d, M=%d, C=%d or dtype", k, M, C);
  if (S == 0 || M == 0) return LANCET_OK;
  LANCET_REQUIRE(dout && gates_s && idx_loc && peer_d_expert_out && peer_expert_out && dgates_s, LANCET_ERR_NULL,
                 "lancet_moe_combine_bwd_p2p: null pointer argument");
  LANCET_REQUIRE(((size_t)M * dtype_bytes(dtype)) % 16 == 0 && aligned(dout, 16), LANCET_ERR_INVALID,
                 "lancet_moe_combine_bwd_p2p: rows must be a multiple of 16 bytes and 16-byte aligned");
  PeerTable td, te;
  for (int i = 0; i < kMaxPeers; ++i) {
    td.ptr[i] = i < W ? peer_d_expert_out[i] : nullptr;
    te.ptr[i] = i < W ? peer_expert_out[i] : nullptr;
  }
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(td.ptr[i] && te.ptr[i] && aligned(td.ptr[i], 16) && aligned(te.ptr[i], 16), LANCET_ERR_NULL,
                   "lancet_moe_combine_bwd_p2p: peer buffer %d is null or unaligned", i);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = LE * W, Sp = S / n_chunks;
  const float* g = static_cast<const float*>(gates_s);
  float* dg = static_cast<float*>(dgates_s);
  if (dtype == LANCET_F32) return combine_bwd_p2p_t<float>(g, idx_loc, dout, td, te, dg, S, Sp, M, C, E, LE, rank, k, part, st);
  if (dtype == LANCET_F16) return combine_bwd_p2p_t<__half>(g, idx_loc, dout, td, te, dg, S, Sp, M, C, E, LE, rank, k, part, st);
  return combine_bwd_p2p_t<__nv_bfloat16>(g, idx_loc, dout, td, te, dg, S, Sp, M, C, E, LE, rank, k, part, st);
}

int lancet_moe_combine_bwd_p2p(const void* dout, const void* gates_s, const int32_t* idx_loc, void* const* peer_d_expert_out,
                               void* const* peer_expert_out, void* dgates_s, int S, int M, int C, int LE, int W, int rank, int k,
                               int n_chunks, int dtype, lancet_stream_t stream) {
  return lancet_moe_combine_bwd_part_p2p(dout, gates_s, idx_loc, peer_d_expert_out, peer_expert_out, dgates_s, S, M, C, LE, W, rank,
                                         k, n_chunks, dtype, 0, stream);
}
}
