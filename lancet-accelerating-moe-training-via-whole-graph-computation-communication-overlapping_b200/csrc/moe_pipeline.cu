// Chunked MoE dispatch / combine: the static form of the reference's partitioned encode.
//
// The reference's scheduler splits `moe_encode` into n chained calls on S/n tokens with capacity
// factor cf*n (PartitionMoEEncode, src/pass/dist_optimization/partition_exprs.cc:1709-1795), gives
// every partition its own full-size [E,C,M] buffer and re-compacts them afterwards with
// moe_merge_masks / moe_redispatch (src/op/dialect/cuda/moe.cc:731-1073).  Here all chunks write
// into ONE [E,C,M] buffer at row used_capacity[e] + location, so nothing has to be merged or
// re-compacted, and one host call enqueues the whole chain.
#include "common.cuh"

extern "C" {
using namespace lancet;

size_t lancet_moe_dispatch_chunked_workspace_bytes(int S, int E, int k, int n_chunks) {
  return lancet_moe_gate_chained_workspace_bytes(S, E, k, n_chunks);
}

int lancet_moe_dispatch_chunked(const void* x, const void* gate, int gate_dtype, float capacity_factor, int S, int M,
                                int E, int k, int n_chunks, int dtype, void* gates_s, int gates_dtype, int32_t* idx_loc,
                                int32_t* capused_chain, uint64_t* elems, void* dispatched, void* ws, size_t ws_bytes,
                                lancet_stream_t stream) {
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && E >= k && M >= 0, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked: bad sizes E=%d k=%d M=%d (need k in {1,2}, E >= k)", E, k, M);
  LANCET_REQUIRE(valid_dtype(dtype) && valid_dtype(gate_dtype) && valid_dtype(gates_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked: unknown dtype code");
  LANCET_REQUIRE(capused_chain && elems && ws && (S == 0 || (x && gate && gates_s && idx_loc)), LANCET_ERR_NULL,
                 "lancet_moe_dispatch_chunked: null pointer argument");
  const int Sp = S / n_chunks;
  const int C = lancet_moe_capacity(Sp, E, capacity_factor * n_chunks, k);
  LANCET_REQUIRE(C >= 0, LANCET_ERR_INVALID, "lancet_moe_dispatch_chunked: negative capacity");
  LANCET_REQUIRE((long long)E * C < (1ll << 31), LANCET_ERR_INVALID, "lancet_moe_dispatch_chunked: E*C exceeds 2^31 rows");
  LANCET_REQUIRE((size_t)E * C * M == 0 || dispatched, LANCET_ERR_NULL, "lancet_moe_dispatch_chunked: null expert buffer");
  LANCET_REQUIRE(aligned(x, dtype_bytes(dtype)) && aligned(dispatched, dtype_bytes(dtype)), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked: data pointers are not aligned to the element size");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LANCET_REQUIRE(k * E <= 1024 && (long long)n_chunks * k * E <= 8192, LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked: k*E=%d or n_chunks*k*E too large", k * E);
  LANCET_REQUIRE(ws_bytes >= gate_workspace_bytes(S, E, k, n_chunks) && aligned(ws, 16), LANCET_ERR_INVALID,
                 "lancet_moe_dispatch_chunked: workspace too small or unaligned");
  // one gating pass over all chunks (chain of used capacities starting from zero; the pass also writes row 0
  // of the chain), locations = rows of the shared buffer
  int rc = gate_launch(gate, gate_dtype, S, E, k, n_chunks, nullptr, C, M, gates_s, gates_dtype, idx_loc, capused_chain + E,
                       elems, ws, 1, st, capused_chain);
  if (rc != LANCET_OK) return rc;
  if ((size_t)E * C * M == 0) return LANCET_OK;
  // one scatter over all tokens; rows past the final used capacity are zero-filled by the same launch
  return dispatch_launch(idx_loc, k, nullptr, capused_chain + (size_t)n_chunks * E, nullptr, x, dispatched, S, Sp, M, C, E,
                         dtype, 0, st);
}

int lancet_moe_scatter_chunked(const void* x, const int32_t* idx_loc, const int32_t* capused_chain, void* dispatched, int S,
                               int M, int C, int E, int k, int n_chunks, int dtype, lancet_stream_t stream) {
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_scatter_chunked: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && E >= k && M >= 0 && C >= 0 && (long long)E * C < (1ll << 31) && valid_dtype(dtype),
                 LANCET_ERR_INVALID, "lancet_moe_scatter_chunked: bad sizes E=%d k=%d M=%d C=%d or dtype", E, k, M, C);
  if ((size_t)E * C * M == 0) return LANCET_OK;
  LANCET_REQUIRE(capused_chain && dispatched && (S == 0 || (x && idx_loc)), LANCET_ERR_NULL,
                 "lancet_moe_scatter_chunked: null pointer argument");
  LANCET_REQUIRE(aligned(x, dtype_bytes(dtype)) && aligned(dispatched, dtype_bytes(dtype)), LANCET_ERR_INVALID,
                 "lancet_moe_scatter_chunked: data pointers are not aligned to the element size");
  return dispatch_launch(idx_loc, k, nullptr, capused_chain + (size_t)n_chunks * E, nullptr, x, dispatched, S, S / n_chunks, M, C,
                         E, dtype, 0, static_cast<cudaStream_t>(stream));
}

int lancet_moe_combine_chunked(const void* expert_out, const void* gates_s, int gates_dtype, const int32_t* idx_loc,
                               int S, int M, int C, int E, int k, int n_chunks, int dtype, void* out,
                               lancet_stream_t stream) {
  LANCET_REQUIRE(n_chunks >= 1 && S >= 0 && S % n_chunks == 0, LANCET_ERR_INVALID,
                 "lancet_moe_combine_chunked: S=%d is not divisible into %d chunks", S, n_chunks);
  LANCET_REQUIRE((k == 1 || k == 2) && M >= 0 && C >= 0 && E > 0 && (long long)E * C < (1ll << 31), LANCET_ERR_INVALID,
                 "lancet_moe_combine_chunked: bad sizes k=%d M=%d C=%d E=%d", k, M, C, E);
  LANCET_REQUIRE(valid_dtype(dtype) && valid_dtype(gates_dtype), LANCET_ERR_INVALID,
                 "lancet_moe_combine_chunked: unknown dtype code");
  LANCET_REQUIRE(S == 0 || M == 0 || (expert_out && gates_s && idx_loc && out), LANCET_ERR_NULL,
                 "lancet_moe_combine_chunked: null pointer argument");
  return combine_launch(gates_s, gates_dtype, idx_loc, k, expert_out, out, S, S / n_chunks, M, C, E, dtype,
                        static_cast<cudaStream_t>(stream));
}
}
