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
// passes), every token counts the tokens of its own bucket that beat it, and a second count over the
// bucket gives the final location.  The work is sum_e n_e^2 comparisons (n_e tokens chose expert e),
// about S_orig^2 / E for balanced routing, served from L1/L2; this favours the batch sizes the
// reference uses this gate with (10^4 tokens).
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

// keep[pos] = 1 when fewer than C tokens of the same bucket have priority over this one.
__global__ void __launch_bounds__(256)
bpr_rank_kernel(const float* __restrict__ list_gate, const int32_t* __restrict__ list_exp, const int32_t* __restrict__ e_off,
                const int32_t* __restrict__ n_e, int S, int C, unsigned char* __restrict__ keep) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < S; i += gridDim.x * blockDim.x) {
    const int e = list_exp[i];
    const int b = e_off[e], n = n_e[e];
    const float g = list_gate[i];
    int rank = 0;
    // inside a bucket, list order is token order: an equal gate earlier in the list wins the tie
    for (int j = b; j < i; ++j) rank += (list_gate[j] >= g) ? 1 : 0;
    for (int j = i + 1; j < b + n; ++j) rank += (list_gate[j] > g) ? 1 : 0;
    keep[i] = rank < C ? 1 : 0;
  }
}

__global__ void __launch_bounds__(256)
bpr_locate_kernel(const float* __restrict__ list_gate, const int32_t* __restrict__ list_tok, const int32_t* __restrict__ list_exp,
                  const int32_t* __restrict__ e_off, const int32_t* __restrict__ n_e, const unsigned char* __restrict__ keep,
                  int S_orig, int Sp, int part_off, int C, int M, void* __restrict__ gates_out, int gates_dtype,
                  int32_t* __restrict__ idx_loc, int32_t* __restrict__ out_capused, uint64_t* __restrict__ out_elems) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < S_orig; i += gridDim.x * blockDim.x) {
    const int e = list_exp[i];
    const int b = e_off[e];
    const int tok = list_tok[i];
    const bool in_part = tok >= part_off && tok < part_off + Sp;
    const bool last = (i == b + n_e[e] - 1);
    if (!in_part && !last) continue;
    int before = 0;
    for (int j = b; j < i; ++j) {
      const int t = list_tok[j];
      before += (keep[j] && t >= part_off && t < part_off + Sp) ? 1 : 0;
    }
    const bool mine = keep[i] && in_part;
    if (in_part) {
      const int s = tok - part_off;
      idx_loc[s] = mine ? e : -1;
      idx_loc[Sp + s] = mine ? before : -1;
      store_from_float(gates_out, gates_dtype, s, list_gate[i]);
    }
    if (last) {  // the last token of a bucket knows the bucket's kept count in this partition
      int cnt = before + (mine ? 1 : 0);
      if (cnt > C) cnt = C;
      out_capused[e] = cnt;
      out_elems[e] = (uint64_t)cnt * (uint64_t)M;
    }
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
  unsigned char* keep = reinterpret_cast<unsigned char*>(w + L.keep);
  long long blocks = ((long long)S_orig + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  bpr_bucket_kernel<<<(int)blocks, 256, (size_t)E * sizeof(int), st>>>(il_all, gates_all, n_e, S_orig, E, lgate, ltok, lexp, eoff);
  if (int s = launch_status("bpr_bucket_kernel")) return s;
  bpr_rank_kernel<<<(int)blocks, 256, 0, st>>>(lgate, lexp, eoff, n_e, S_orig, C, keep);
  if (int s = launch_status("bpr_rank_kernel")) return s;
  const int Sp = S_orig / n_partitions;
  bpr_locate_kernel<<<(int)blocks, 256, 0, st>>>(lgate, ltok, lexp, eoff, n_e, keep, S_orig, Sp, Sp * partition_id, C, M,
                                                 out_gates_s, gates_dtype, out_idx_loc, out_capused, out_elems);
  return launch_status("bpr_locate_kernel");
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
