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
#include "common.cuh"

namespace lancet {

constexpr int kGateTile = 256;       // tokens per CTA
constexpr int kGateWarps = kGateTile / 32;
constexpr int kSelfScanMaxTiles = 256;  // beyond this pass 1b is used

struct GateWs {
  int* hist;    // [tiles][k*E]  per-tile counts (pass 1), exclusive prefix after pass 1b
  int* total;   // [k*E]         totals over all tiles (only written by pass 1b)
};

__device__ __forceinline__ float gate_at(const void* g, int dtype, size_t i) { return load_as_float(g, dtype, i); }

template <int K>
__global__ void __launch_bounds__(kGateTile)
gate_select_kernel(const void* __restrict__ gate, int gate_dtype, int S, int E, float* __restrict__ raw_gates,
                   int32_t* __restrict__ idx_loc, int* __restrict__ hist) {
  extern __shared__ int warp_cnt[];  // [kGateWarps][K*E]
  const int KE = K * E;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int s = blockIdx.x * kGateTile + tid;
  for (int i = tid; i < kGateWarps * KE; i += kGateTile) warp_cnt[i] = 0;
  __syncthreads();

  int e_sel[K];
  float g_sel[K];
#pragma unroll
  for (int j = 0; j < K; ++j) { e_sel[j] = -1; g_sel[j] = 0.f; }
  if (s < S) {
    float b1 = -INFINITY, b2 = -INFINITY;
    int i1 = 0, i2 = 0;
    const size_t row = (size_t)s * E;
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
    } else {
      for (int e = 0; e < E; ++e) {
        const float v = gate_at(gate, gate_dtype, row + e);
        if (v > b1) { b2 = b1; i2 = i1; b1 = v; i1 = e; }
        else if (v > b2) { b2 = v; i2 = e; }
      }
    }
    e_sel[0] = i1;
    g_sel[0] = gate_at(gate, gate_dtype, row + i1);
    if (K == 2) {
      e_sel[K - 1] = i2;
      g_sel[K - 1] = gate_at(gate, gate_dtype, row + i2);
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
  if (s < S) {
#pragma unroll
    for (int j = 0; j < K; ++j) {
      int r = rank_in_warp[j];
      for (int w = 0; w < warp; ++w) r += warp_cnt[w * KE + j * E + e_sel[j]];
      idx_loc[(size_t)(2 * j) * S + s] = e_sel[j];
      idx_loc[(size_t)(2 * j + 1) * S + s] = r;
      raw_gates[(size_t)j * S + s] = g_sel[j];
    }
  }
  for (int c = tid; c < KE; c += kGateTile) {
    int t = 0;
#pragma unroll
    for (int w = 0; w < kGateWarps; ++w) t += warp_cnt[w * KE + c];
    hist[(size_t)blockIdx.x * KE + c] = t;
  }
}

// One CTA per (choice, expert) column: exclusive scan of that column over the tiles.
__global__ void __launch_bounds__(256) gate_scan_tiles_kernel(int* __restrict__ hist, int* __restrict__ total, int tiles,
                                                              int KE) {
  __shared__ int warp_sum[8];
  __shared__ int carry_s;
  const int c = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < tiles; base += 256) {
    const int t = base + tid;
    const int v = t < tiles ? hist[(size_t)t * KE + c] : 0;
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
    if (t < tiles) hist[(size_t)t * KE + c] = carry + woff + incl - v;
    __syncthreads();
    if (tid == 255) carry_s = carry + woff + incl;
    __syncthreads();
  }
  if (tid == 0) total[c] = carry_s;
}

template <int K>
__global__ void __launch_bounds__(kGateTile)
gate_assign_kernel(int S, int E, int C, int M, int tiles, int prescanned, const int* __restrict__ hist,
                   const int* __restrict__ total_in, const int32_t* __restrict__ in_capused,
                   const float* __restrict__ raw_gates, int32_t* __restrict__ idx_loc, void* __restrict__ gates_out,
                   int gates_dtype, int32_t* __restrict__ out_capused, uint64_t* __restrict__ out_elems) {
  extern __shared__ int sm[];  // pre[K*E], tot[K*E]
  const int KE = K * E;
  int* pre = sm;
  int* tot = sm + KE;
  const int tid = threadIdx.x;
  const int tile = blockIdx.x;
  if (prescanned) {
    for (int c = tid; c < KE; c += kGateTile) {
      pre[c] = hist[(size_t)tile * KE + c];
      tot[c] = total_in[c];
    }
    __syncthreads();
  } else {
    for (int c = tid; c < 2 * KE; c += kGateTile) sm[c] = 0;
    __syncthreads();
    // threads (group, column): every group sums a strided subset of the tiles
    int cols = 1;
    while (cols < KE) cols <<= 1;
    if (cols > kGateTile) cols = kGateTile;
    const int groups = kGateTile / cols;
    const int grp = tid / cols;
    for (int c = tid % cols; c < KE; c += cols) {
      int p = 0, t_all = 0;
      for (int t = grp; t < tiles; t += groups) {
        const int h = hist[(size_t)t * KE + c];
        t_all += h;
        if (t < tile) p += h;
      }
      if (p) atomicAdd(&pre[c], p);
      if (t_all) atomicAdd(&tot[c], t_all);
    }
    __syncthreads();
  }
  const int s = tile * kGateTile + tid;
  if (s < S) {
    int e[K], loc[K];
    bool keep[K];
    float g[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      e[j] = idx_loc[(size_t)(2 * j) * S + s];
      int l = idx_loc[(size_t)(2 * j + 1) * S + s] + pre[j * E + e[j]];
      for (int jj = 0; jj < j; ++jj) l += tot[jj * E + e[j]];
      loc[j] = l;
      const int used = in_capused ? in_capused[e[j]] : 0;
      keep[j] = l < C - used;
      g[j] = raw_gates[(size_t)j * S + s];
      idx_loc[(size_t)(2 * j) * S + s] = keep[j] ? e[j] : -1;
      idx_loc[(size_t)(2 * j + 1) * S + s] = l;
    }
    if (K == 1) {
      store_from_float(gates_out, gates_dtype, s, g[0]);
    } else {
      const float m0 = keep[0] ? g[0] : 0.f;
      const float m1 = keep[K - 1] ? g[K - 1] : 0.f;
      const float denom = fmaxf(__fadd_rn(m0, m1), 1.1920928955078125e-07f);
      store_from_float(gates_out, gates_dtype, s, __fdiv_rn(m0, denom));
      store_from_float(gates_out, gates_dtype, (size_t)S + s, __fdiv_rn(m1, denom));
    }
  }
  if (tile == 0) {
    for (int ex = tid; ex < E; ex += kGateTile) {
      int n = 0;
#pragma unroll
      for (int j = 0; j < K; ++j) n += tot[j * E + ex];
      const int used = in_capused ? in_capused[ex] : 0;
      int oc = used + n;
      if (oc > C) oc = C;
      out_capused[ex] = oc;
      out_elems[ex] = (uint64_t)((long long)(oc - used) * (long long)M);
    }
  }
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t gate_workspace_bytes(int S, int E, int k) {
  const size_t tiles = (size_t)(S + kGateTile - 1) / kGateTile;
  size_t raw = align_up((size_t)k * (S > 0 ? S : 1) * sizeof(float), 256);
  size_t hist = align_up((tiles > 0 ? tiles : 1) * k * E * sizeof(int), 256);
  size_t total = align_up((size_t)k * E * sizeof(int), 256);
  return raw + hist + total;
}

int gate_launch(const void* gate, int gate_dtype, int S, int E, int k, const int32_t* in_capused, int C, int M,
                void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems,
                void* ws, cudaStream_t stream) {
  const int tiles = (S + kGateTile - 1) / kGateTile;
  char* w = static_cast<char*>(ws);
  float* raw = reinterpret_cast<float*>(w);
  w += align_up((size_t)k * (S > 0 ? S : 1) * sizeof(float), 256);
  int* hist = reinterpret_cast<int*>(w);
  w += align_up((size_t)(tiles > 0 ? tiles : 1) * k * E * sizeof(int), 256);
  int* total = reinterpret_cast<int*>(w);
  const int KE = k * E;
  if (tiles == 0) {
    // no tokens: only the capacity outputs are defined
    LANCET_CUDA(cudaMemsetAsync(hist, 0, (size_t)KE * sizeof(int), stream));
  }
  const size_t smem1 = (size_t)kGateWarps * KE * sizeof(int);
  const size_t smem2 = (size_t)2 * KE * sizeof(int);
  if (tiles > 0) {
    if (k == 1)
      gate_select_kernel<1><<<tiles, kGateTile, smem1, stream>>>(gate, gate_dtype, S, E, raw, out_idx_loc, hist);
    else
      gate_select_kernel<2><<<tiles, kGateTile, smem1, stream>>>(gate, gate_dtype, S, E, raw, out_idx_loc, hist);
    if (int st = launch_status("gate_select_kernel")) return st;
  }
  const int prescanned = tiles > kSelfScanMaxTiles ? 1 : 0;
  if (prescanned) {
    gate_scan_tiles_kernel<<<KE, 256, 0, stream>>>(hist, total, tiles, KE);
    if (int st = launch_status("gate_scan_tiles_kernel")) return st;
  }
  const int grid2 = tiles > 0 ? tiles : 1;
  const int tiles_arg = tiles > 0 ? tiles : 1;
  if (k == 1)
    gate_assign_kernel<1><<<grid2, kGateTile, smem2, stream>>>(S, E, C, M, tiles_arg, prescanned, hist, total, in_capused,
                                                               raw, out_idx_loc, out_gates_s, gates_dtype, out_capused,
                                                               out_elems);
  else
    gate_assign_kernel<2><<<grid2, kGateTile, smem2, stream>>>(S, E, C, M, tiles_arg, prescanned, hist, total, in_capused,
                                                               raw, out_idx_loc, out_gates_s, gates_dtype, out_capused,
                                                               out_elems);
  return launch_status("gate_assign_kernel");
}

}  // namespace lancet

extern "C" {

size_t lancet_moe_gate_workspace_bytes(int S, int E, int k) {
  if (S < 0 || E <= 0 || k < 1 || k > 2) return 0;
  return lancet::gate_workspace_bytes(S, E, k);
}

int lancet_moe_gate(const void* gate, int gate_dtype, int S, int E, int k, const int32_t* in_capused, int C, int M,
                    void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems,
                    void* ws, size_t ws_bytes, lancet_stream_t stream) {
  using namespace lancet;
  LANCET_REQUIRE(k == 1 || k == 2, LANCET_ERR_INVALID, "lancet_moe_gate: k must be 1 or 2, got %d", k);
  LANCET_REQUIRE(S >= 0 && E >= k && k * E <= 1024 && C >= 0 && M >= 0, LANCET_ERR_INVALID,
                 "lancet_moe_gate: bad sizes S=%d E=%d C=%d M=%d (need S>=0, k<=E, k*E<=1024)", S, E, C, M);
  LANCET_REQUIRE(valid_dtype(gate_dtype) && valid_dtype(gates_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_gate: unknown dtype code (gate %d, gates_s %d)", gate_dtype, gates_dtype);
  LANCET_REQUIRE((S == 0 || (gate && out_gates_s && out_idx_loc)) && out_capused && out_elems && ws, LANCET_ERR_NULL,
                 "lancet_moe_gate: null pointer argument");
  LANCET_REQUIRE(ws_bytes >= gate_workspace_bytes(S, E, k), LANCET_ERR_INVALID,
                 "lancet_moe_gate: workspace of %zu bytes is smaller than the %zu needed", ws_bytes,
                 gate_workspace_bytes(S, E, k));
  LANCET_REQUIRE(aligned(ws, 16) && aligned(gate, dtype_bytes(gate_dtype)), LANCET_ERR_INVALID,
                 "lancet_moe_gate: workspace must be 16-byte aligned");
  return gate_launch(gate, gate_dtype, S, E, k, in_capused, C, M, out_gates_s, gates_dtype, out_idx_loc, out_capused,
                     out_elems, ws, static_cast<cudaStream_t>(stream));
}
}
