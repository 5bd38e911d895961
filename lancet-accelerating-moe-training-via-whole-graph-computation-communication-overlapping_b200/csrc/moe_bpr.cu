// Batch-prioritized routing (moe_encode_batch_prioritized).
//
// Replaces the TVM argsort plus gen_location_bpr_kernel of the reference
// (src/op/dialect/cuda/moe.cc:415-729; kernels/tutel_moe_dispatch.cu:259-363): over ALL S_orig tokens
// of the batch, each expert keeps its C highest-gate tokens (ties: lower token index first; the
// reference leaves ties to TVM's argsort); the tokens of partition `partition_id` then get their
// locations by counting the kept tokens of the same expert before them in the partition; dropped
// tokens get (-1, -1).
//
// No global sort is needed: tokens are bucketed per expert in token order (reusing the gating
// passes); one block per expert then finds the gate value of its C-th best token with a radix select
// (four 8-bit rounds) and hands out the locations with block-wide prefix counts, all in about five
// passes over the bucket, so the cost grows linearly with the batch.
#include "common.cuh"

namespace lancet {

__global__ void __launch_bounds__(256)
bpr_bucket_kernel(const int32_t* __restrict__ il_all, const float* __restrict__ gates_all, const int32_t* __restrict__ n_e,
                  int S, int E, float* __restrict__ list_gate, int32_t* __restrict__ list_tok, int32_t* __restrict__ list_exp,
                  int32_t* __restrict__ e_off_out) {
  extern __shared__ int off[];  // exclusive offsets of the expert buckets
  if (threadIdx.x == 0) {
    int a = 0;
    for (int e = 0; e < E; ++e) { off[e] = a; a += n_e[e]; }
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e < E; e += blockDim.x) e_off_out[e] = off[e];
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gridDim.x * blockDim.x) {
    const int e = il_all[s];
    const int pos = off[e] + il_all[S + s];
    list_gate[pos] = gates_all[s];
    list_tok[pos] = s;
    list_exp[pos] = e;
  }
}

// Order-preserving map of a float onto an unsigned integer (larger gate = larger key); -0 counts as +0.
__device__ __forceinline__ uint32_t bpr_key(float g) {
  if (g == 0.0f) g = 0.0f;
  const uint32_t b = __float_as_uint(g);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

constexpr int kBprThreads = 1024;

// Inclusive block scan of one int per thread (1024 threads); returns the inclusive prefix, *total = block sum.
__device__ __forceinline__ int bpr_block_scan(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  __syncthreads();   // warp_sums may still be read from the previous call
  if (lane == 31) warp_sums[warp] = x;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += y;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  *total = warp_sums[31];
  return x + (warp > 0 ? warp_sums[warp - 1] : 0);
}

// One block per expert.  Its bucket (the tokens that chose it, in token order) keeps the C tokens with the largest
// gate, an equal gate earlier in the batch first:
//   1. radix select, four rounds of 8 bits over the order-preserving keys, finds the key T of the C-th kept token and
//      how many tokens with exactly that key are kept (the first `need_eq` of them in token order);
//   2. one pass in token order decides keep = key > T, or key == T and fewer than need_eq equal keys came before, and
//      gives every kept token of partition `partition_id` its location = kept tokens of the partition before it.
// Work per bucket is about five passes over its tokens (the earlier form compared every pair of tokens of a bucket).
__global__ void __launch_bounds__(kBprThreads)
bpr_select_locate_kernel(const float* __restrict__ list_gate, const int32_t* __restrict__ list_tok,
                         const int32_t* __restrict__ e_off, const int32_t* __restrict__ n_e, int Sp, int part_off, int C, int M,
                         void* __restrict__ gates_out, int gates_dtype, int32_t* __restrict__ idx_loc,
                         int32_t* __restrict__ out_capused, uint64_t* __restrict__ out_elems) {
  __shared__ int hist[256];
  __shared__ int warp_sums[32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  const int e = blockIdx.x;
  const int b = e_off[e], n = n_e[e];
  const float* g = list_gate + b;
  const int32_t* tok = list_tok + b;
  // ---- 1. threshold key ----
  uint32_t T = 0;           // keys >= T ... all kept when the bucket is not over capacity
  int need_eq = n;          // how many tokens with key == T are kept
  bool select = n > C;
  if (select && C == 0) {
    T = 0xffffffffu;
    need_eq = 0;
    select = false;
  }
  if (select) {
    if (threadIdx.x == 0) { s_prefix = 0; s_need = C; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int i = threadIdx.x; i < 256; i += kBprThreads) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = threadIdx.x; i < n; i += kBprThreads) {
        const uint32_t k = bpr_key(g[i]);
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int need = s_need, d = 255;
        for (; d > 0; --d) {              // from the largest digit down: where does the need-th token fall
          if (hist[d] >= need) break;
          need -= hist[d];
        }
        s_prefix = prefix | ((uint32_t)d << shift);
        s_need = need;
      }
      __syncthreads();
    }
    T = s_prefix;
    need_eq = s_need;
  }
  // ---- 2. keep decisions and locations, in token order ----
  int carry_eq = 0, carry_loc = 0;
  for (int base = 0; base < n; base += kBprThreads) {
    const int i = base + threadIdx.x;
    const bool valid = i < n;
    uint32_t k = 0;
    int t = 0;
    float gv = 0.f;
    if (valid) {
      gv = g[i];
      k = bpr_key(gv);
      t = tok[i];
    }
    const bool is_eq = valid && k == T;
    int tot_eq;
    const int eq_incl = bpr_block_scan(is_eq ? 1 : 0, warp_sums, &tot_eq);
    const bool keep = valid && (k > T || (is_eq && carry_eq + eq_incl - 1 < need_eq));
    const bool in_part = valid && t >= part_off && t < part_off + Sp;
    int tot_loc;
    const int loc_incl = bpr_block_scan((keep && in_part) ? 1 : 0, warp_sums, &tot_loc);
    if (in_part) {
      const int s = t - part_off;
      const bool mine = keep;
      idx_loc[s] = mine ? e : -1;
      idx_loc[Sp + s] = mine ? carry_loc + loc_incl - 1 : -1;
      store_from_float(gates_out, gates_dtype, s, gv);
    }
    carry_eq += tot_eq;
    carry_loc += tot_loc;
  }
  if (threadIdx.x == 0) {
    const int cnt = carry_loc > C ? C : carry_loc;
    out_capused[e] = cnt;
    out_elems[e] = (uint64_t)cnt * (uint64_t)M;
  }
}

struct BprLayout {
  size_t gates, il, ne, elems, lgate, ltok, lexp, eoff, keep, gate_ws, total;
};

static BprLayout bpr_layout(int S, int E) {
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  BprLayout L;
  const size_t s = (size_t)(S > 0 ? S : 1);
  size_t o = 0;
  L.gates = o; o += up(s * 4);
  L.il = o;    o += up(2 * s * 4);
  L.ne = o;    o += up((size_t)E * 4);
  L.elems = o; o += up((size_t)E * 8);
  L.lgate = o; o += up(s * 4);
  L.ltok = o;  o += up(s * 4);
  L.lexp = o;  o += up(s * 4);
  L.eoff = o;  o += up((size_t)E * 4);
  L.keep = o;  o += up(s);
  L.gate_ws = o; o += up(gate_workspace_bytes(S, E, 1, 1));
  L.total = o;
  return L;
}

}  // namespace lancet

extern "C" {
using namespace lancet;

size_t lancet_moe_gate_bpr_workspace_bytes(int S_orig, int E) {
  if (S_orig < 0 || E < 1 || E > 1024) return 0;
  return bpr_layout(S_orig, E).total;
}

int lancet_moe_gate_bpr(const void* gate, int gate_dtype, int S_orig, int E, int n_partitions, int partition_id, int C, int M,
                        void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems,
                        void* ws, size_t ws_bytes, lancet_stream_t stream) {
  LANCET_REQUIRE(S_orig >= 0 && E >= 1 && E <= 1024 && C >= 0 && M >= 0, LANCET_ERR_INVALID,
                 "lancet_moe_gate_bpr: bad sizes S=%d E=%d C=%d M=%d", S_orig, E, C, M);
  LANCET_REQUIRE(n_partitions >= 1 && partition_id >= 0 && partition_id < n_partitions && S_orig % n_partitions == 0,
                 LANCET_ERR_INVALID, "lancet_moe_gate_bpr: bad partition %d of %d for %d tokens", partition_id, n_partitions, S_orig);
  LANCET_REQUIRE(valid_dtype(gate_dtype) && valid_dtype(gates_dtype), LANCET_ERR_INVALID, "lancet_moe_gate_bpr: unknown dtype code");
  LANCET_REQUIRE(out_capused && out_elems && ws && (S_orig == 0 || (gate && out_gates_s && out_idx_loc)), LANCET_ERR_NULL,
                 "lancet_moe_gate_bpr: null pointer argument");
  const BprLayout L = bpr_layout(S_orig, E);
  LANCET_REQUIRE(ws_bytes >= L.total && aligned(ws, 16), LANCET_ERR_INVALID,
                 "lancet_moe_gate_bpr: workspace of %zu bytes is smaller than the %zu needed (or unaligned)", ws_bytes, L.total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* w = static_cast<char*>(ws);
  float* gates_all = reinterpret_cast<float*>(w + L.gates);
  int32_t* il_all = reinterpret_cast<int32_t*>(w + L.il);
  int32_t* n_e = reinterpret_cast<int32_t*>(w + L.ne);
  uint64_t* el = reinterpret_cast<uint64_t*>(w + L.elems);
  LANCET_CUDA(cudaMemsetAsync(out_capused, 0, (size_t)E * sizeof(int32_t), st));
  LANCET_CUDA(cudaMemsetAsync(out_elems, 0, (size_t)E * sizeof(uint64_t), st));
  if (S_orig == 0) return LANCET_OK;
  // bucket positions: the plain gating pass with an unlimited capacity gives, per token, its expert and its
  // position among the tokens of that expert; the "used capacity" output is the bucket size n_e
  int rc = gate_launch(gate, gate_dtype, S_orig, E, 1, 1, nullptr, 1 << 30, 0, gates_all, LANCET_F32, il_all, n_e, el,
                       w + L.gate_ws, 0, st);
  if (rc != LANCET_OK) return rc;
  float* lgate = reinterpret_cast<float*>(w + L.lgate);
  int32_t* ltok = reinterpret_cast<int32_t*>(w + L.ltok);
  int32_t* lexp = reinterpret_cast<int32_t*>(w + L.lexp);
  int32_t* eoff = reinterpret_cast<int32_t*>(w + L.eoff);
  long long blocks = ((long long)S_orig + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  bpr_bucket_kernel<<<(int)blocks, 256, (size_t)E * sizeof(int), st>>>(il_all, gates_all, n_e, S_orig, E, lgate, ltok, lexp, eoff);
  if (int s = launch_status("bpr_bucket_kernel")) return s;
  const int Sp = S_orig / n_partitions;
  bpr_select_locate_kernel<<<E, kBprThreads, 0, st>>>(lgate, ltok, eoff, n_e, Sp, Sp * partition_id, C, M, out_gates_s, gates_dtype,
                                                      out_idx_loc, out_capused, out_elems);
  return launch_status("bpr_select_locate_kernel");
}

int lancet_moe_encode_bpr(const void* x, const void* gate, int gate_dtype, int n_partitions, int partition_id,
                          float capacity_factor, int S_orig, int M, int E, int dtype, void* out_gates_s, int gates_dtype,
                          int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems, void* dispatched, void* ws,
                          size_t ws_bytes, lancet_stream_t stream) {
  LANCET_REQUIRE(n_partitions >= 1 && S_orig >= 0 && S_orig % n_partitions == 0 && E >= 1 && valid_dtype(dtype), LANCET_ERR_INVALID,
                 "lancet_moe_encode_bpr: bad sizes S=%d partitions=%d E=%d or dtype", S_orig, n_partitions, E);
  const int Sp = S_orig / n_partitions;
  // capacity from the per-partition token count: src/op/dialect/cuda/moe.cc:433-438 of the reference
  const int C = lancet_moe_capacity(Sp, E, capacity_factor, 1);
  LANCET_REQUIRE(C >= 0, LANCET_ERR_INVALID, "lancet_moe_encode_bpr: negative capacity");
  int rc = lancet_moe_gate_bpr(gate, gate_dtype, S_orig, E, n_partitions, partition_id, C, M, out_gates_s, gates_dtype,
                               out_idx_loc, out_capused, out_elems, ws, ws_bytes, stream);
  if (rc != LANCET_OK) return rc;
  const char* xp = static_cast<const char*>(x) + (size_t)partition_id * Sp * M * dtype_bytes(dtype);
  return lancet_moe_encode_fwd(out_idx_loc, 1, nullptr, out_capused, nullptr, xp, dispatched, Sp, M, C, E, dtype, 0, stream);
}
}
