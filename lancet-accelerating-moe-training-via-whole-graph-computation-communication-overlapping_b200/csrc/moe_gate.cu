// Top-k gating with capacity slot assignment.
//
// Replaces the reference's argmax / one_hot / sum(gate*mask) helper kernels and its
// gen_location_kernel (src/op/dialect/cuda/moe.cc:177-250, :366-380;
// src/op/dialect/cuda/kernels/tutel_moe_dispatch.cu:164-212), which walk all S tokens with
// one block per expert.  Here the token axis is tiled over the whole GPU:
//
//   pass 1 (gate_select_kernel): one thread per token picks its k experts (first maximum
//     wins), ranks the token among the tile's tokens of the same expert with a warp
//     match/ballot and a per-warp count table in shared memory, and writes the tile's
//     per-expert histogram to the workspace.
//   pass 1b (gate_scan_tiles_kernel, only for many tiles): turns the histograms into
//     exclusive prefixes over tiles.
//   pass 2 (gate_assign_kernel): location = (first choices of all tokens, for the second
//     choice) + prefix over earlier tiles + rank in tile; capacity test; drops; the k=2
//     normalisation; per-expert used capacity and element counts.
//
// The order of tokens inside an expert is the token order, so the result is identical to the
// serial cumulative sum of the reference.
#include <mutex>

#include "common.cuh"

namespace lancet {

constexpr int kGateTile = 256;       // tokens per CTA
constexpr int kGateWarps = kGateTile / 32;
constexpr int kSelfScanMaxTiles = 256;  // beyond this pass 1b is used
constexpr int kMaxChainInts = 8192;     // n_chunks * k * E ints of shared memory in pass 2

// The token axis may be split into n_chunks contiguous chunks of Sp tokens that are gated as a
// chain: chunk c sees the capacity used by chunks < c (the reference's partitioned moe_encode,
// src/pass/dist_optimization/partition_exprs.cc:1709-1795).  All chunks are processed by the same
// launches; a tile never straddles two chunks.  Layouts: idx_loc [n][2K][Sp], gates [n][K][Sp].

__device__ __forceinline__ float gate_at(const void* g, int dtype, size_t i) { return load_as_float(g, dtype, i); }

template <int K>
__global__ void __launch_bounds__(kGateTile)
gate_select_kernel(const void* __restrict__ gate, int gate_dtype, int Sp, int E, int tiles_per_chunk,
                   float* __restrict__ raw_gates, int32_t* __restrict__ idx_loc, int* __restrict__ hist) {
  extern __shared__ int warp_cnt[];  // [kGateWarps][K*E]
  chain_enter();
  const int KE = K * E;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = blockIdx.x / tiles_per_chunk;
  const int sc = (blockIdx.x % tiles_per_chunk) * kGateTile + tid;  // token inside the chunk
  const bool valid = sc < Sp;
  for (int i = tid; i < kGateWarps * KE; i += kGateTile) warp_cnt[i] = 0;
  __syncthreads();

  int e_sel[K];
  float g_sel[K];
#pragma unroll
  for (int j = 0; j < K; ++j) { e_sel[j] = -1; g_sel[j] = 0.f; }
  if (valid) {
    float b1 = -INFINITY, b2 = -INFINITY;
    int i1 = 0, i2 = 0;
    const size_t row = ((size_t)chunk * Sp + sc) * E;
    if (gate_dtype == LANCET_F32 && (E & 3) == 0 && (reinterpret_cast<uintptr_t>(gate) & 15) == 0) {
      const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(gate) + row);
      for (int e4 = 0; e4 < E / 4; ++e4) {
        float4 v = p[e4];
        float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int e = e4 * 4 + q;
          if (vv[q] > b1) { b2 = b1; i2 = i1; b1 = vv[q]; i1 = e; }
          else if (vv[q] > b2) { b2 = vv[q]; i2 = e; }
        }
      }
    } else if (gate_dtype == LANCET_F32 && (E & 1) == 0 && (reinterpret_cast<uintptr_t>(gate) & 7) == 0) {
      const float2* p = reinterpret_cast<const float2*>(static_cast<const float*>(gate) + row);
      for (int e2 = 0; e2 < E / 2; ++e2) {
        float2 v = p[e2];
        float vv[2] = {v.x, v.y};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int e = e2 * 2 + q;
          if (vv[q] > b1) { b2 = b1; i2 = i1; b1 = vv[q]; i1 = e; }
          else if (vv[q] > b2) { b2 = vv[q]; i2 = e; }
        }
      }
    } else {
      for (int e = 0; e < E; ++e) {
        const float v = gate_at(gate, gate_dtype, row + e);
        if (v > b1) { b2 = b1; i2 = i1; b1 = v; i1 = e; }
        else if (v > b2) { b2 = v; i2 = e; }
      }
    }
    // b1/b2 hold the selected values except in the degenerate all -inf row, where the element is re-read
    e_sel[0] = i1;
    g_sel[0] = (b1 > -INFINITY) ? b1 : gate_at(gate, gate_dtype, row + i1);
    if (K == 2) {
      e_sel[K - 1] = i2;
      g_sel[K - 1] = (b2 > -INFINITY) ? b2 : gate_at(gate, gate_dtype, row + i2);
    }
  }
  int rank_in_warp[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const unsigned peers = __match_any_sync(0xffffffffu, e_sel[j]);
    rank_in_warp[j] = __popc(peers & ((1u << lane) - 1u));
    if (e_sel[j] >= 0 && rank_in_warp[j] == 0) warp_cnt[warp * KE + j * E + e_sel[j]] = __popc(peers);
  }
  __syncthreads();
  if (valid) {
    const size_t il_base = (size_t)chunk * 2 * K * Sp + sc;
    const size_t g_base = (size_t)chunk * K * Sp + sc;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      int r = rank_in_warp[j];
      for (int w = 0; w < warp; ++w) r += warp_cnt[w * KE + j * E + e_sel[j]];
      idx_loc[il_base + (size_t)(2 * j) * Sp] = e_sel[j];
      idx_loc[il_base + (size_t)(2 * j + 1) * Sp] = r;
      raw_gates[g_base + (size_t)j * Sp] = g_sel[j];
    }
  }
  for (int c = tid; c < KE; c += kGateTile) {
    int t = 0;
#pragma unroll
    for (int w = 0; w < kGateWarps; ++w) t += warp_cnt[w * KE + c];
    hist[(size_t)blockIdx.x * KE + c] = t;
  }
}

// One CTA per (column, chunk): exclusive scan of that column over the tiles of the chunk.
__global__ void __launch_bounds__(256) gate_scan_tiles_kernel(int* __restrict__ hist, int* __restrict__ total,
                                                              int tiles_per_chunk, int KE) {
  __shared__ int warp_sum[8];
  __shared__ int carry_s;
  const int c = blockIdx.x, chunk = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* h = hist + (size_t)chunk * tiles_per_chunk * KE;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < tiles_per_chunk; base += 256) {
    const int t = base + tid;
    const int v = t < tiles_per_chunk ? h[(size_t)t * KE + c] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += n;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < warp; ++w) woff += warp_sum[w];
    const int carry = carry_s;
    if (t < tiles_per_chunk) h[(size_t)t * KE + c] = carry + woff + incl - v;
    __syncthreads();
    if (tid == 255) carry_s = carry + woff + incl;
    __syncthreads();
  }
  if (tid == 0) total[(size_t)chunk * KE + c] = carry_s;
}

template <int K>
__global__ void __launch_bounds__(kGateTile)
gate_assign_kernel(int Sp, int E, int C, int M, int n_chunks, int tiles_per_chunk, int prescanned, int global_loc,
                   const int* __restrict__ hist, const int* __restrict__ total_in,
                   const int32_t* __restrict__ in_capused, const float* __restrict__ raw_gates,
                   int32_t* __restrict__ idx_loc, void* __restrict__ gates_out, int gates_dtype,
                   int32_t* __restrict__ out_capused, uint64_t* __restrict__ out_elems, int32_t* __restrict__ chain_row0) {
  extern __shared__ int sm[];  // pre[KE], used[E], tot[n_chunks][KE]
  chain_enter();
  const int KE = K * E;
  int* pre = sm;
  int* used_s = sm + KE;
  int* tot = sm + KE + E;
  const int tid = threadIdx.x;
  const int chunk = blockIdx.x / tiles_per_chunk;
  const int tile = blockIdx.x % tiles_per_chunk;
  // the CTA of the last chunk's first tile also writes the capacity chain of every chunk
  const bool writes_chain = (chunk == n_chunks - 1 && tile == 0);
  const int chunks_needed = chunk + 1;
  if (prescanned) {
    for (int c = tid; c < KE; c += kGateTile) pre[c] = hist[((size_t)chunk * tiles_per_chunk + tile) * KE + c];
    for (int i = tid; i < chunks_needed * KE; i += kGateTile) tot[i] = total_in[i];
    __syncthreads();
  } else {
    for (int i = tid; i < KE + E + chunks_needed * KE; i += kGateTile) sm[i] = 0;
    __syncthreads();
    // threads (group, column): every group sums a strided subset of the tiles of chunks <= chunk
    int cols = 1;
    while (cols < KE) cols <<= 1;
    if (cols > kGateTile) cols = kGateTile;
    const int groups = kGateTile / cols;
    const int grp = tid / cols;
    const int ntiles = chunks_needed * tiles_per_chunk;
    const int my_first = chunk * tiles_per_chunk;
    for (int c = tid % cols; c < KE; c += cols) {
      int p = 0;
      for (int t = grp; t < ntiles; t += groups) {
        const int h = hist[(size_t)t * KE + c];
        if (h) atomicAdd(&tot[(t / tiles_per_chunk) * KE + c], h);
        if (t >= my_first && t < my_first + tile) p += h;
      }
      if (p) atomicAdd(&pre[c], p);
    }
    __syncthreads();
  }
  // capacity used before this chunk: the chain min(used + n, C) over the earlier chunks
  for (int ex = tid; ex < E; ex += kGateTile) {
    int used = in_capused ? in_capused[ex] : 0;
    if (writes_chain && chain_row0) chain_row0[ex] = used;  // row 0 of a [n+1][E] capacity chain
    for (int c = 0; c < chunk; ++c) {
      int n = 0;
#pragma unroll
      for (int j = 0; j < K; ++j) n += tot[c * KE + j * E + ex];
      if (writes_chain) {
        int oc = used + n;
        if (oc > C) oc = C;
        out_capused[(size_t)c * E + ex] = oc;
        out_elems[(size_t)c * E + ex] = (uint64_t)((long long)(oc - used) * (long long)M);
      }
      used = used + n > C ? C : used + n;
    }
    used_s[ex] = used;
    if (writes_chain) {
      int n = 0;
#pragma unroll
      for (int j = 0; j < K; ++j) n += tot[chunk * KE + j * E + ex];
      int oc = used + n;
      if (oc > C) oc = C;
      out_capused[(size_t)chunk * E + ex] = oc;
      out_elems[(size_t)chunk * E + ex] = (uint64_t)((long long)(oc - used) * (long long)M);
    }
  }
  __syncthreads();
  const int sc = tile * kGateTile + tid;
  if (sc < Sp) {
    const size_t il_base = (size_t)chunk * 2 * K * Sp + sc;
    const size_t g_base = (size_t)chunk * K * Sp + sc;
    const int* tot_c = tot + chunk * KE;
    int e[K], loc[K];
    bool keep[K];
    float g[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      e[j] = idx_loc[il_base + (size_t)(2 * j) * Sp];
      int l = idx_loc[il_base + (size_t)(2 * j + 1) * Sp] + pre[j * E + e[j]];
      for (int jj = 0; jj < j; ++jj) l += tot_c[jj * E + e[j]];
      loc[j] = l;
      const int used = used_s[e[j]];
      keep[j] = l < C - used;
      g[j] = raw_gates[g_base + (size_t)j * Sp];
      idx_loc[il_base + (size_t)(2 * j) * Sp] = keep[j] ? e[j] : -1;
      idx_loc[il_base + (size_t)(2 * j + 1) * Sp] = global_loc ? l + used : l;
    }
    if (K == 1) {
      store_from_float(gates_out, gates_dtype, g_base, g[0]);
    } else {
      const float m0 = keep[0] ? g[0] : 0.f;
      const float m1 = keep[K - 1] ? g[K - 1] : 0.f;
      const float denom = fmaxf(__fadd_rn(m0, m1), 1.1920928955078125e-07f);
      store_from_float(gates_out, gates_dtype, g_base, __fdiv_rn(m0, denom));
      store_from_float(gates_out, gates_dtype, g_base + Sp, __fdiv_rn(m1, denom));
    }
  }
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct GateLayout {
  int Sp, tiles_per_chunk, tiles;
  size_t raw_off, hist_off, total_off, bytes;
};

static GateLayout gate_layout(int S, int E, int k, int n_chunks) {
  GateLayout L;
  L.Sp = S / n_chunks;
  L.tiles_per_chunk = (L.Sp + kGateTile - 1) / kGateTile;
  if (L.tiles_per_chunk < 1) L.tiles_per_chunk = 1;
  L.tiles = L.tiles_per_chunk * n_chunks;
  size_t off = 0;
  L.raw_off = off;   off += align_up((size_t)k * (S > 0 ? S : 1) * sizeof(float), 256);
  L.hist_off = off;  off += align_up((size_t)L.tiles * k * E * sizeof(int), 256);
  L.total_off = off; off += align_up((size_t)n_chunks * k * E * sizeof(int), 256);
  L.bytes = off;
  return L;
}

size_t gate_workspace_bytes(int S, int E, int k, int n_chunks) { return gate_layout(S, E, k, n_chunks).bytes; }

int gate_launch(const void* gate, int gate_dtype, int S, int E, int k, int n_chunks, const int32_t* in_capused, int C,
                int M, void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused,
                uint64_t* out_elems, void* ws, int global_loc, cudaStream_t stream, int32_t* chain_row0) {
  const GateLayout L = gate_layout(S, E, k, n_chunks);
  char* w = static_cast<char*>(ws);
  float* raw = reinterpret_cast<float*>(w + L.raw_off);
  int* hist = reinterpret_cast<int*>(w + L.hist_off);
  int* total = reinterpret_cast<int*>(w + L.total_off);
  const int KE = k * E;
  const size_t smem1 = (size_t)kGateWarps * KE * sizeof(int);
  const size_t smem2 = (size_t)(KE + E + (size_t)n_chunks * KE) * sizeof(int);
  // with S == 0 the select pass still runs (every thread is out of range) so that the histograms are zero
  if (k == 1)
    launch_chained(gate_select_kernel<1>, L.tiles, kGateTile, smem1, stream, gate, gate_dtype, L.Sp, E, L.tiles_per_chunk, raw,
                   out_idx_loc, hist);
  else
    launch_chained(gate_select_kernel<2>, L.tiles, kGateTile, smem1, stream, gate, gate_dtype, L.Sp, E, L.tiles_per_chunk, raw,
                   out_idx_loc, hist);
  if (int st = launch_status("gate_select_kernel")) return st;
  const int prescanned = L.tiles > kSelfScanMaxTiles ? 1 : 0;
  if (prescanned) {
    gate_scan_tiles_kernel<<<dim3(KE, n_chunks), 256, 0, stream>>>(hist, total, L.tiles_per_chunk, KE);
    if (int st = launch_status("gate_scan_tiles_kernel")) return st;
  }
  if (k == 1)
    launch_chained(gate_assign_kernel<1>, L.tiles, kGateTile, smem2, stream, L.Sp, E, C, M, n_chunks, L.tiles_per_chunk,
                   prescanned, global_loc, hist, total, in_capused, raw, out_idx_loc, out_gates_s, gates_dtype, out_capused,
                   out_elems, chain_row0);
  else
    launch_chained(gate_assign_kernel<2>, L.tiles, kGateTile, smem2, stream, L.Sp, E, C, M, n_chunks, L.tiles_per_chunk,
                   prescanned, global_loc, hist, total, in_capused, raw, out_idx_loc, out_gates_s, gates_dtype, out_capused,
                   out_elems, chain_row0);
  return launch_status("gate_assign_kernel");
}

}  // namespace lancet

extern "C" {

size_t lancet_moe_gate_workspace_bytes(int S, int E, int k) {
  if (S < 0 || E <= 0 || k < 1 || k > 2) return 0;
  return lancet::gate_workspace_bytes(S, E, k, 1);
}

size_t lancet_moe_gate_chained_workspace_bytes(int S, int E, int k, int n_chunks) {
  if (S < 0 || E <= 0 || k < 1 || k > 2 || n_chunks < 1 || S % n_chunks != 0) return 0;
  return lancet::gate_workspace_bytes(S, E, k, n_chunks);
}

int lancet_moe_gate_chained(const void* gate, int gate_dtype, int S, int E, int k, int n_chunks,
                            const int32_t* in_capused, int C, int M, void* out_gates_s, int gates_dtype,
                            int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems, void* ws, size_t ws_bytes,
                            int flags, lancet_stream_t stream) {
  using namespace lancet;
  LANCET_REQUIRE(k == 1 || k == 2, LANCET_ERR_INVALID, "lancet_moe_gate: k must be 1 or 2, got %d", k);
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_gate: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE(E >= k && k * E <= 1024 && C >= 0 && M >= 0, LANCET_ERR_INVALID,
                 "lancet_moe_gate: bad sizes S=%d E=%d C=%d M=%d (need S>=0, k<=E, k*E<=1024)", S, E, C, M);
  LANCET_REQUIRE((long long)n_chunks * k * E <= kMaxChainInts, LANCET_ERR_INVALID,
                 "lancet_moe_gate: n_chunks*k*E = %lld exceeds %d", (long long)n_chunks * k * E, kMaxChainInts);
  LANCET_REQUIRE((flags & ~LANCET_GATE_GLOBAL_LOC) == 0, LANCET_ERR_INVALID, "lancet_moe_gate: unknown flag bits 0x%x", flags);
  LANCET_REQUIRE(valid_dtype(gate_dtype) && valid_dtype(gates_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_gate: unknown dtype code (gate %d, gates_s %d)", gate_dtype, gates_dtype);
  LANCET_REQUIRE((S == 0 || (gate && out_gates_s && out_idx_loc)) && out_capused && out_elems && ws, LANCET_ERR_NULL,
                 "lancet_moe_gate: null pointer argument");
  LANCET_REQUIRE(ws_bytes >= gate_workspace_bytes(S, E, k, n_chunks), LANCET_ERR_INVALID,
                 "lancet_moe_gate: workspace of %zu bytes is smaller than the %zu needed", ws_bytes,
                 gate_workspace_bytes(S, E, k, n_chunks));
  LANCET_REQUIRE(aligned(ws, 16) && aligned(gate, dtype_bytes(gate_dtype)), LANCET_ERR_INVALID,
                 "lancet_moe_gate: workspace must be 16-byte aligned");
  return gate_launch(gate, gate_dtype, S, E, k, n_chunks, in_capused, C, M, out_gates_s, gates_dtype, out_idx_loc,
                     out_capused, out_elems, ws, (flags & LANCET_GATE_GLOBAL_LOC) ? 1 : 0,
                     static_cast<cudaStream_t>(stream), nullptr);
}

int lancet_moe_gate(const void* gate, int gate_dtype, int S, int E, int k, const int32_t* in_capused, int C, int M,
                    void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems,
                    void* ws, size_t ws_bytes, int flags, lancet_stream_t stream) {
  return lancet_moe_gate_chained(gate, gate_dtype, S, E, k, 1, in_capused, C, M, out_gates_s, gates_dtype, out_idx_loc,
                                 out_capused, out_elems, ws, ws_bytes, flags, stream);
}

// ---------------------------------------------------------------------------------------------
// Gating without a caller-supplied workspace.
//
// Some hosts of this library cannot hand it scratch memory and cannot let it allocate either: an
// executor that has already given all device memory to its own pool (a raw cudaMalloc would fail
// or fragment it), an operator bound after that executor planned its workspaces, or a step loop
// in which cudaMalloc's device-wide synchronisation would stall work running on other streams.
// For them the gating scratch lives in a fixed array inside the library image.  Every GPU that
// loads the library holds these kLancetStaticGateBytes until the process exits.
// ---------------------------------------------------------------------------------------------
constexpr size_t kLancetStaticGateBytes = 4u << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_static_gate_scratch[kLancetStaticGateBytes];

namespace {
// Device address of g_static_gate_scratch per device.  In host code the symbol itself is only a
// stand-in, so the address is looked up once per device (with that device current) and cached.
void* g_static_gate_ptr[64] = {nullptr};
std::mutex g_static_gate_mu;

int static_gate_scratch(void** out) {
  int dev = -1;
  LANCET_CUDA(cudaGetDevice(&dev));
  LANCET_REQUIRE(dev >= 0 && dev < 64, LANCET_ERR_UNSUPPORTED, "lancet_moe_gate_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_static_gate_mu);
  if (g_static_gate_ptr[dev] == nullptr) {
    void* p = nullptr;
    LANCET_CUDA(cudaGetSymbolAddress(&p, g_static_gate_scratch));
    LANCET_REQUIRE(p != nullptr, LANCET_ERR_CUDA, "lancet_moe_gate_static: no device address for the scratch array");
    g_static_gate_ptr[dev] = p;
  }
  *out = g_static_gate_ptr[dev];
  return LANCET_OK;
}
}  // namespace

size_t lancet_moe_gate_static_max_bytes(void) { return kLancetStaticGateBytes; }

int lancet_moe_gate_static(const void* gate, int gate_dtype, int S, int E, int k, const int32_t* in_capused, int C, int M,
                           void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused,
                           uint64_t* out_elems, int flags, lancet_stream_t stream) {
  using namespace lancet;
  LANCET_REQUIRE(k == 1 || k == 2, LANCET_ERR_INVALID, "lancet_moe_gate_static: k must be 1 or 2, got %d", k);
  LANCET_REQUIRE(S >= 0 && E >= k && k * E <= 1024, LANCET_ERR_INVALID,
                 "lancet_moe_gate_static: bad sizes S=%d E=%d k=%d (need S>=0, k<=E, k*E<=1024)", S, E, k);
  const size_t need = gate_workspace_bytes(S, E, k, 1);
  LANCET_REQUIRE(need <= kLancetStaticGateBytes, LANCET_ERR_INVALID,
                 "lancet_moe_gate_static: S=%d E=%d k=%d needs %zu bytes of scratch, the built-in array holds %zu; "
                 "use lancet_moe_gate with a caller workspace",
                 S, E, k, need, kLancetStaticGateBytes);
  void* scratch = nullptr;
  if (int rc = static_gate_scratch(&scratch)) return rc;
  // Nothing in the scratch has to start at zero: every word the kernels read (raw gate values,
  // tile histograms, tile totals) is written earlier in the same call, so stale contents of the
  // previous call are harmless and no clearing pass is needed.
  return lancet_moe_gate(gate, gate_dtype, S, E, k, in_capused, C, M, out_gates_s, gates_dtype, out_idx_loc,
                         out_capused, out_elems, scratch, kLancetStaticGateBytes, flags, stream);
}
}
