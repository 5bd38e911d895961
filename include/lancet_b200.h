/*
 * lancet_b200.h - C ABI of the B200-native MoE data-parallel hot path.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes, returns an int
 * status (0 = ok) and only enqueues work on the stream it is given: nothing here allocates
 * device memory or synchronises the device.  Outputs and workspaces are owned by the
 * caller (in RAF: by the executor, see include/raf/op.h:55-91 and src/requests.h:17-52 of
 * the reference).  Arguments are validated before anything is launched; an invalid call
 * launches nothing and `lancet_last_error()` describes the reason.
 *
 * Each declaration cites the reference interface it replaces (path inside the reference
 * project : line).
 *
 * Conventions: S tokens, E experts, M model dim, C capacity rows per expert, k choices per
 * token (1 or 2).  `idx_loc` is int32 [2k, S]: rows (2j, 2j+1) are the expert index (-1 when
 * dropped) and the location of choice j; for k = 1 this is the reference's
 * `indices_locations[2, S]`.  `gates_s` is [k, S].
 */
#ifndef LANCET_B200_H_
#define LANCET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* lancet_stream_t; /* a cudaStream_t */
typedef void* lancet_comm_t;   /* an opaque communicator made by lancet_comm_init_rank */

enum { LANCET_F32 = 0, LANCET_F16 = 1, LANCET_BF16 = 2 };

enum {
  LANCET_OK = 0,
  LANCET_ERR_INVALID = 1,     /* bad shape, dtype, size, alignment or flag */
  LANCET_ERR_NULL = 2,        /* a required pointer is null */
  LANCET_ERR_CUDA = 3,        /* a CUDA runtime call or launch failed */
  LANCET_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out (peer never arrived) */
  LANCET_ERR_COMM = 5,        /* NCCL missing or an NCCL call failed */
  LANCET_ERR_UNSUPPORTED = 6
};

/* flag of lancet_moe_gate: locations are written as in_capused[e] + location, i.e. rows of one
 * buffer shared by all chunks of a chained, partitioned encode (what the reference obtains later
 * with moe_merge_masks, src/op/dialect/cuda/kernels/tutel_moe_dispatch.cu:214-255) */
enum { LANCET_GATE_GLOBAL_LOC = 1 };

/* flags of lancet_moe_encode_fwd / lancet_moe_encode.  With LANCET_ENCODE_GLOBAL_LOC,
 * lancet_moe_encode gates with LANCET_GATE_GLOBAL_LOC and zeroes nothing (finish the chain with
 * lancet_moe_zero_tail); lancet_moe_encode_fwd adds in_capused[e] to local locations. */
enum {
  LANCET_ENCODE_GLOBAL_LOC = 1, /* write row in_capused[e] + loc (one shared buffer for chained chunks) */
  LANCET_ENCODE_NO_ZERO = 2     /* do not zero rows that no token owns */
};

const char* lancet_last_error(void);      /* thread-local text of the last failure */
const char* lancet_version(void);
int lancet_abi_version(void);
/* Number of kernels this library has launched in this process (all threads). */
unsigned long long lancet_launch_count(void);
/* Per-kernel timing for benchmarks: between begin and end every launch of a kernel whose name
 * contains `kernel_substr` is bracketed by a CUDA event pair on its own stream; end waits for
 * them and returns the summed duration and the number of launches.  Not for concurrent use. */
int lancet_profile_begin(const char* kernel_substr);
int lancet_profile_end(double* total_ms, long long* launches);

/* C = (int)(cf * ((k*S + E - 1) / E)).  Replaces the inline formula of
 * src/op/declare/moe.cc:46 and src/op/dialect/cuda/moe.cc:110 (k = 1). */
int lancet_moe_capacity(int S, int E, float capacity_factor, int k);

/* ---- gating with capacity slot assignment -------------------------------------------------
 * Replaces the three TVM helper kernels of MoeEncode (src/op/dialect/cuda/moe.cc:177-250,
 * :366-371: argmax, one_hot, sum(gate*mask)) and launch_gen_location
 * (src/op/dialect/cuda/kernels/kernel_util.cuh:59, tutel_moe_dispatch.cu:164-212, :548-553).
 * gate [S,E] in gate_dtype; in_capused [E] may be null (= zeros).  Outputs: gates_s [k,S] in
 * gates_dtype, idx_loc [2k,S], out_capused [E], out_elems [E] (elements sent per expert).
 * ws: lancet_moe_gate_workspace_bytes(S,E,k) bytes of scratch, 16-byte aligned. */
size_t lancet_moe_gate_workspace_bytes(int S, int E, int k);
int lancet_moe_gate(const void* gate, int gate_dtype, int S, int E, int k, const int32_t* in_capused,
                    int C, int M, void* out_gates_s, int gates_dtype, int32_t* out_idx_loc,
                    int32_t* out_capused, uint64_t* out_elems, void* ws, size_t ws_bytes, int flags,
                    lancet_stream_t stream);

/* Gating of n_chunks chained chunks in one pass (the partitioned moe_encode chain of
 * src/pass/dist_optimization/partition_exprs.cc:1709-1795): chunk c of Sp = S/n_chunks tokens sees
 * the capacity used by chunks < c.  Layouts: gate [S,E]; gates_s [n][k][Sp]; idx_loc [n][2k][Sp];
 * out_capused [n][E] (after each chunk); out_elems [n][E].  Results equal n chained
 * lancet_moe_gate calls. */
size_t lancet_moe_gate_chained_workspace_bytes(int S, int E, int k, int n_chunks);
int lancet_moe_gate_chained(const void* gate, int gate_dtype, int S, int E, int k, int n_chunks,
                            const int32_t* in_capused, int C, int M, void* out_gates_s, int gates_dtype,
                            int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems, void* ws,
                            size_t ws_bytes, int flags, lancet_stream_t stream);

/* Gating for callers that can neither pass a workspace nor allocate one: lancet_moe_gate with its
 * scratch in a fixed 4 MiB array inside the library (lancet_moe_gate_static_max_bytes()), which
 * every GPU that loads the library holds until the process exits.  It has no counterpart in the
 * reference, whose executor always supplies workspaces.  It is meant for hosts whose memory pool
 * already owns the whole device, for operators bound after workspaces were planned, and for step
 * loops that must not take cudaMalloc's device-wide synchronisation.  Allocates nothing.  Sizes
 * whose scratch exceeds the array (roughly k*S*4 bytes plus k*E*4 per 256 tokens) are rejected with
 * LANCET_ERR_INVALID.  The first call on each device looks up the array's device address; make
 * that call outside any stream capture.  All calls on a device share the array: two calls whose
 * kernels overlap on the GPU (different streams) race; calls on one stream are safe. */
size_t lancet_moe_gate_static_max_bytes(void);
int lancet_moe_gate_static(const void* gate, int gate_dtype, int S, int E, int k, const int32_t* in_capused,
                           int C, int M, void* out_gates_s, int gates_dtype, int32_t* out_idx_loc,
                           int32_t* out_capused, uint64_t* out_elems, int flags, lancet_stream_t stream);

/* ---- dispatch: scatter token rows into the [E,C,M] expert buffer ---------------------------
 * Replaces launch_encode_forward (kernel_util.cuh:36-39; tutel_moe_dispatch.cu:61-86, :461-484).
 * rows_hi/rows_lo (both nullable, int32 [E]): when rows_hi is given, expert e owns rows
 * [0, rows_hi[e] - rows_lo[e]) and only the rows past that are zeroed (no full-buffer memset);
 * when null the whole buffer is zeroed first, as the reference does. */
int lancet_moe_encode_fwd(const int32_t* idx_loc, int k, const int32_t* in_capused, const int32_t* rows_hi,
                          const int32_t* rows_lo, const void* x, void* dispatched, int S, int M, int C, int E,
                          int dtype, int flags, lancet_stream_t stream);

/* Zero rows [used[e], C) of every expert (finishes a LANCET_ENCODE_GLOBAL_LOC chain). */
int lancet_moe_zero_tail(void* dispatched, const int32_t* used, int M, int C, int E, int dtype,
                         lancet_stream_t stream);

/* The whole `raf.op.cuda.moe_encode` op (src/op/dialect/cuda/moe.cc:351-396; outputs as
 * src/op/declare/moe.cc:48-57): gating, then dispatch.  C is computed from capacity_factor. */
int lancet_moe_encode(const void* x, const void* gate, int gate_dtype, const int32_t* in_capused,
                      float capacity_factor, int S, int M, int E, int k, int dtype, void* out_gates_s,
                      int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems,
                      void* dispatched, void* ws, size_t ws_bytes, int flags, lancet_stream_t stream);

/* ---- combine and the four gradient ops -----------------------------------------------------
 * launch_decode_forward (kernel_util.cuh:44-45; tutel_moe_dispatch.cu:110-116, :511-518). */
int lancet_moe_decode_fwd(const void* gates_s, int gates_dtype, const int32_t* idx_loc, int k,
                          const void* expert_out, void* out, int S, int M, int C, int E, int dtype,
                          lancet_stream_t stream);
/* launch_encode_backward_data (kernel_util.cuh:40-41; tutel_moe_dispatch.cu:88-94, :486-493). */
int lancet_moe_encode_bwd_data(const int32_t* idx_loc, int k, const void* dy_dispatched, void* dx, int S,
                               int M, int C, int E, int dtype, lancet_stream_t stream);
/* launch_encode_backward_gate (kernel_util.cuh:42-43; tutel_moe_dispatch.cu:96-108, :498-506).
 * gate is read only for k = 2 (Jacobian of the normalisation). */
int lancet_moe_encode_bwd_gate(const void* dy_gates_s, int gates_dtype, const int32_t* idx_loc, int k,
                               const void* gate, int gate_dtype, void* dgate, int S, int E,
                               lancet_stream_t stream);
/* launch_decode_backward_data (kernel_util.cuh:46-47; tutel_moe_dispatch.cu:118-124, :523-531).
 * rows_used nullable: as rows_hi above. */
int lancet_moe_decode_bwd_data(const void* gates_s, int gates_dtype, const int32_t* idx_loc, int k,
                               const void* dy, void* d_expert, const int32_t* rows_used, int S, int M, int C,
                               int E, int dtype, lancet_stream_t stream);
/* launch_decode_backward_gate (kernel_util.cuh:48-49; tutel_moe_dispatch.cu:126-160, :536-543). */
int lancet_moe_decode_bwd_gate(const int32_t* idx_loc, int k, const void* dy, const void* expert_out,
                               void* dgates_s, int gates_dtype, int S, int M, int C, int E, int dtype,
                               lancet_stream_t stream);

/* ---- chunked dispatch / combine (static form of the reference's partitioned encode) ------------
 * Replaces the chain moe_encode x n -> moe_merge_masks -> moe_redispatch that the reference's
 * scheduler emits (src/pass/dist_optimization/partition_exprs.cc:1709-1795, :474-594).  S tokens are
 * split into n_chunks contiguous chunks of Sp = S/n_chunks; chunk i is gated with capacity factor
 * capacity_factor*n_chunks and the used capacity of chunks < i, and its rows go straight to their
 * final place in the single [E,C,M] buffer, C = lancet_moe_capacity(Sp, E, cf*n_chunks, k).
 * Outputs per chunk: gates_s [n][k][Sp], idx_loc [n][2k][Sp] (locations are rows of the shared
 * buffer), elems [n][E]; capused_chain [n+1][E] (row 0 is zeroed here, row i+1 = after chunk i). */
size_t lancet_moe_dispatch_chunked_workspace_bytes(int S, int E, int k, int n_chunks);
int lancet_moe_dispatch_chunked(const void* x, const void* gate, int gate_dtype, float capacity_factor, int S,
                                int M, int E, int k, int n_chunks, int dtype, void* gates_s, int gates_dtype,
                                int32_t* idx_loc, int32_t* capused_chain, uint64_t* elems, void* dispatched,
                                void* ws, size_t ws_bytes, lancet_stream_t stream);
/* Combine for outputs of lancet_moe_dispatch_chunked: out [S,M]. */
/* The scatter of lancet_moe_dispatch_chunked alone, for a table that is already gated (idx_loc [n][2k][Sp] with
 * shared-buffer rows, capused_chain [n+1][E] as that call wrote them): moves another [S,M] tensor with the same routing,
 * the role of a second launch_encode_forward on the same indices_locations (kernel_util.cuh:36-39). */
int lancet_moe_scatter_chunked(const void* x, const int32_t* idx_loc, const int32_t* capused_chain, void* dispatched,
                               int S, int M, int C, int E, int k, int n_chunks, int dtype, lancet_stream_t stream);
int lancet_moe_combine_chunked(const void* expert_out, const void* gates_s, int gates_dtype,
                               const int32_t* idx_loc, int S, int M, int C, int E, int k, int n_chunks, int dtype,
                               void* out, lancet_stream_t stream);

/* ---- batch-prioritized routing -------------------------------------------------------------------
 * Replaces launch_gen_location_bpr and the argsort in front of it (kernel_util.cuh:67;
 * src/op/dialect/cuda/moe.cc:415-729; tutel_moe_dispatch.cu:259-363).  gate is [S_orig,E] for the whole
 * batch; the outputs describe partition `partition_id` of n_partitions (Sp = S_orig/n_partitions
 * tokens): gates_s [Sp], idx_loc [2,Sp] with (-1,-1) for dropped tokens, out_capused / out_elems [E].
 * Each expert keeps its C highest-gate tokens of the whole batch; ties go to the lower token index.
 * One block per expert selects the C-th best gate with a radix select and assigns locations with prefix counts:
 * the cost grows linearly with S_orig (about five passes over each expert's tokens), any S_orig is accepted.
 * lancet_moe_encode_bpr is the whole `raf.op.cuda.moe_encode_batch_prioritized` op: capacity
 * (int)(cf * ceil(Sp / E)), gating, then dispatch of the partition's rows of x [S_orig, M]. */
size_t lancet_moe_gate_bpr_workspace_bytes(int S_orig, int E);
int lancet_moe_gate_bpr(const void* gate, int gate_dtype, int S_orig, int E, int n_partitions, int partition_id, int C,
                        int M, void* out_gates_s, int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused,
                        uint64_t* out_elems, void* ws, size_t ws_bytes, lancet_stream_t stream);
int lancet_moe_encode_bpr(const void* x, const void* gate, int gate_dtype, int n_partitions, int partition_id,
                          float capacity_factor, int S_orig, int M, int E, int dtype, void* out_gates_s,
                          int gates_dtype, int32_t* out_idx_loc, int32_t* out_capused, uint64_t* out_elems,
                          void* dispatched, void* ws, size_t ws_bytes, lancet_stream_t stream);

/* ---- re-compaction operators of graphs partitioned the reference's way --------------------------
 * idx_locs / datas / recv_counts are HOST arrays of n_partitions device pointers (at most 16).
 * ws: lancet_moe_partition_workspace_bytes(n_partitions, E) bytes.
 * lancet_moe_merge_masks replaces launch_merge_masks (kernel_util.cuh:61-62; tutel_moe_dispatch.cu:214-255):
 *   idx_locs[p] is [2,S]; out [2, n*S]; locations of partition p are shifted by the tokens kept for
 *   the same expert in partitions < p; dropped tokens become (-1,-1).
 * lancet_moe_redispatch replaces launch_redispatch (kernel_util.cuh:50-52; tutel_moe_dispatch.cu:365-408):
 *   datas[p] is [E,C,M]; out [E,C,M] holds, per expert, the kept rows of all partitions one after the
 *   other; rows past the merged count are zero (the reference leaves them unwritten).
 * lancet_moe_redispatch_expert_input replaces launch_redispatch_expert_input (kernel_util.cuh:53-55;
 *   tutel_moe_dispatch.cu:436-459): datas[p] is [C,G,M], recv_counts[p] uint64 [G*LE] (elements); column
 *   g of out [C,G,M] is the concatenation over p of the first recv_counts[p][g*LE+le]*scale elements of
 *   column g of datas[p]; the rest is zero. */
size_t lancet_moe_partition_workspace_bytes(int n_partitions, int E);
int lancet_moe_merge_masks(const int32_t* const* idx_locs, int n_partitions, int S, int E, int32_t* out, void* ws,
                           size_t ws_bytes, lancet_stream_t stream);
int lancet_moe_redispatch(const void* const* datas, const int32_t* const* idx_locs, int n_partitions, int S, int M,
                          int C, int E, int dtype, void* out, void* ws, size_t ws_bytes, lancet_stream_t stream);
int lancet_moe_redispatch_expert_input(const void* const* datas, const uint64_t* const* recv_counts, int n_partitions,
                                       int local_expert_id, int n_local_experts, int C, int G, int M,
                                       int recv_cnts_scale, int dtype, void* out, lancet_stream_t stream);

/* ---- expert-parallel exchange fused into dispatch / combine over NVLink peer memory ------------
 * Replaces `moe_encode -> _all_to_all` and `_all_to_all -> moe_decode` of the MoE layer
 * (NCCLAllToAll::Execute, src/op/dialect/nccl/nccl.cc:199-227; layer wiring in
 * models/benchmark/pytorch/utils.py:576-634).  Rank r of W owns experts [r*LE, (r+1)*LE).  Every
 * rank exposes a receive buffer [W][LE][C][M] (what the all-to-all would deliver: block g comes
 * from rank g); peer_recv / peer_expert_out are HOST arrays of the W device addresses of those
 * buffers as mapped into this process (own buffer at index `rank`).
 *
 * lancet_symm_alloc/open/close/free: device buffers that other processes on the node can map
 * (set-up time only; these do allocate).  Replaces the communicator bootstrap of
 * src/distributed/cuda/nccl_communicator.cc:27-60 for the peer-memory path; the 64-byte handle is
 * exchanged by the caller (any host channel). */
int lancet_symm_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int lancet_symm_open(const unsigned char* handle64, void** peer_ptr);
int lancet_symm_close(void* peer_ptr);
int lancet_symm_free(void* ptr);

/* Flag barrier between the W ranks on `stream`.  peer_flags[r] = rank r's array of W 32-bit words
 * (zero-initialised, symmetric memory); epoch must grow by one per barrier on every rank.  A rank
 * that waits longer than timeout_ns records the missing peer in *status (device int32, zero when
 * healthy) and returns; lancet_p2p_status() turns a non-zero word into LANCET_ERR_TIMEOUT. */
int lancet_p2p_barrier(void* const* peer_flags, int W, int rank, unsigned epoch, unsigned long long timeout_ns,
                       int32_t* status, lancet_stream_t stream);
/* Same barrier with the epoch kept in device memory (*epoch_counter, zero-initialised, owned by this rank):
 * every launch uses the stored value + 1 and writes it back, so the launch can be replayed from a CUDA graph. */
int lancet_p2p_barrier_counted(void* const* peer_flags, int W, int rank, uint32_t* epoch_counter,
                               unsigned long long timeout_ns, int32_t* status, lancet_stream_t stream);
int lancet_p2p_status(const int32_t* status, lancet_stream_t stream);

/* LANCET_P2P_NO_REMOTE_ZERO: do not send zero rows over NVLink; instead the row count of every
 * (source rank, local expert) block is written to the owner's peer_counts array (int32 [W*LE]) and
 * the owner zero-fills its tails after the barrier: lancet_moe_zero_tail(recv, counts, M, C, W*LE). */
enum { LANCET_P2P_NO_REMOTE_ZERO = 1 };
/* As lancet_moe_dispatch_chunked with E = LE*W, but rows go straight into the owners' receive
 * buffers.  gates_s is float32 [n][k][Sp].  peer_counts may be null without the flag. */
int lancet_moe_dispatch_chunked_p2p(const void* x, const void* gate, int gate_dtype, float capacity_factor, int S,
                                    int M, int LE, int W, int rank, int k, int n_chunks, int dtype, void* gates_s,
                                    int32_t* idx_loc, int32_t* capused_chain, uint64_t* elems,
                                    void* const* peer_recv, void* const* peer_counts, void* ws, size_t ws_bytes,
                                    int flags, lancet_stream_t stream);
/* Staged form of the call above, for running the exchange of chunk c+1 under the expert GEMMs of chunk c
 * (the reference's chunk pipeline: src/pass/dist_optimization/partition_exprs.cc:1745-1757 partitions
 * moe_encode / _all_to_all / experts, lancet_optimization.cc schedules them on two streams).
 * 1. lancet_moe_gate_chunked_p2p gates all chunks and writes the chained row counts capused_chain
 *    [n+1][E] into every owner's table peer_chain[owner] = int32 [W][n+1][LE] (block `rank`), so that the
 *    owner knows before any row arrives where each chunk's rows of every block will lie.
 * 2. lancet_moe_dispatch_rows_p2p scatters the rows of chunks [chunk_begin, chunk_end) (x [S][M] and
 *    idx_loc [n][2k][Sp] are the whole arrays); follow each stage with lancet_p2p_barrier.
 * 3. lancet_moe_stage_windows (on the owner, after the first barrier) turns its chain table into the row
 *    windows of every stage, row_begin / row_end int32 [n][W*LE] (row_align = 128 for the grouped GEMM):
 *    stage c ends at max(floor(chain[c+1] / row_align) * row_align, chain[c]), i.e. it covers the whole tiles that
 *    have arrived with chunks 0..c and in any case every row of the chunks before c, whose tokens are combined
 *    right after it; it begins at the tile that holds the previous stage's end (a tile left partial is computed
 *    again, with the same values); the last stage ends at the total.  counts (nullable, int32 [W*LE])
 *    receives the totals.
 * Combine, its backward and the dispatch backward run per chunk through the existing calls on sub-arrays
 * (gates_s + c*k*Sp, idx_loc + c*2k*Sp, out + c*Sp*M, S = Sp, n_chunks = 1). */
int lancet_moe_gate_chunked_p2p(const void* gate, int gate_dtype, float capacity_factor, int S, int M, int LE, int W,
                                int rank, int k, int n_chunks, void* gates_s, int32_t* idx_loc,
                                int32_t* capused_chain, uint64_t* elems, void* const* peer_chain, void* ws,
                                size_t ws_bytes, lancet_stream_t stream);
int lancet_moe_dispatch_rows_p2p(const void* x, const int32_t* idx_loc, int S, int M, int C, int LE, int W, int rank,
                                 int k, int n_chunks, int chunk_begin, int chunk_end, int dtype,
                                 void* const* peer_recv, lancet_stream_t stream);
/* Incremental form of steps 1 and 3, for pipelines that also split the operators IN FRONT of the layer into token
 * chunks (the reference's forward partition of non-MoE operators, partition_exprs.cc:1709-1795 with the range search
 * of lancet_optimization.cc:1203-1345): the gate probabilities of chunk c+1 do not exist yet when chunk c travels.
 * lancet_moe_gate_chunks_p2p gates chunks [chunk_begin, chunk_end) from gate_rows = their rows only
 * ([(chunk_end-chunk_begin)*Sp][E]), starting from row chunk_begin of capused_chain (the chunks must be gated in
 * order), writes the usual slices of gates_s / idx_loc / capused_chain / elems and publishes the new chain rows to
 * the owners.  lancet_moe_stage_window gives the row window of ONE stage covering those chunks (row_begin / row_end
 * int32 [W*LE]; prev_chunk_begin = first chunk of the stage before it, ignored for the first stage) as soon as its
 * barrier has been passed; counts is written when chunk_end == n_chunks.
 * Results are identical to the all-at-once calls. */
int lancet_moe_gate_chunks_p2p(const void* gate_rows, int gate_dtype, float capacity_factor, int S, int M, int LE, int W,
                               int rank, int k, int n_chunks, int chunk_begin, int chunk_end, void* gates_s,
                               int32_t* idx_loc, int32_t* capused_chain, uint64_t* elems, void* const* peer_chain,
                               void* ws, size_t ws_bytes, lancet_stream_t stream);
int lancet_moe_stage_window(const int32_t* chain, int W, int LE, int n_chunks, int row_align, int prev_chunk_begin,
                            int chunk_begin, int chunk_end, int32_t* row_begin, int32_t* row_end, int32_t* counts,
                            lancet_stream_t stream);
int lancet_moe_stage_windows(const int32_t* chain, int W, int LE, int n_chunks, int row_align, int32_t* row_begin,
                             int32_t* row_end, int32_t* counts, lancet_stream_t stream);
/* As lancet_moe_combine_chunked, gathering rows from the owners' expert output buffers.  With
 * gates_s == NULL every kept row has weight 1: the data gradient of dispatch (moe_encode_dx,
 * src/op/dialect/cuda/moe.cc:1108-1133) fused with the returning all-to-all. */
int lancet_moe_combine_chunked_p2p(void* const* peer_expert_out, const void* gates_s, const int32_t* idx_loc, int S,
                                   int M, int C, int LE, int W, int rank, int k, int n_chunks, int dtype, void* out,
                                   lancet_stream_t stream);

/* ---- `_all_to_all` / `_all_to_allv` as stand-alone operators ------------------------------------
 * NCCL transport: replaces NCCLAllToAll::Execute (src/op/dialect/nccl/nccl.cc:199-227): W grouped
 * ncclSend/ncclRecv pairs of bytes_per_rank bytes on `stream`; any device buffers.  The
 * communicator replaces src/distributed/cuda/nccl_communicator.cc:27-60: rank 0 makes the 128-byte
 * id, the caller broadcasts it over its own host channel (the reference uses MPI). */
int lancet_comm_unique_id(unsigned char* id128);
int lancet_comm_init_rank(const unsigned char* id128, int world, int rank, lancet_comm_t* comm);
int lancet_comm_destroy(lancet_comm_t comm);
int lancet_all_to_all(const void* send, void* recv, size_t bytes_per_rank, lancet_comm_t comm,
                      lancet_stream_t stream);
/* Same, taking the whole tensor size: splits it evenly over the communicator's ranks and fails with
 * the reference's message when it does not divide (nccl.cc:213). */
int lancet_all_to_all_evenly(const void* send, void* recv, size_t total_bytes, lancet_comm_t comm,
                             lancet_stream_t stream);
/* Tuple form of `_all_to_all` (nccl.cc:228-277): n_tensors (at most 16) tensors of nbytes[i] bytes are
 * exchanged in ONE grouped all-to-all: a kernel packs the per-rank slices into in_ws, the result lands in
 * out_ws and a kernel unpacks it into recvs[i].  in_ws and out_ws: sum(nbytes) bytes each. */
int lancet_all_to_all_tuple(const void* const* sends, void* const* recvs, const size_t* nbytes, int n_tensors,
                            void* in_ws, void* out_ws, size_t ws_bytes, lancet_comm_t comm, lancet_stream_t stream);
/* Count-aware all-to-all over NCCL, replaces NCCLAllToAllv::Execute (nccl.cc:357-431) for buffers that are not in
 * symmetric memory: send / recv are [W][n_chunks][chunk_elems]; the counts (device uint64 [W*n_chunks]) are
 * exchanged on the device, whole chunks travel, and a kernel clears everything past recv_counts[i*n_chunks+j]
 * elements of every received chunk - the same result as the reference without its host round trip (:388-390). */
int lancet_all_to_allv(const void* send, void* recv, const uint64_t* send_counts, uint64_t* recv_counts, int n_chunks,
                       size_t elem_size, size_t chunk_elems, lancet_comm_t comm, lancet_stream_t stream);
/* Peer-memory transport for receive buffers in symmetric memory: one kernel stores chunk i of
 * `send` into block `rank` of peer_recv[i].  Follow with lancet_p2p_barrier before reading. */
int lancet_all_to_all_p2p(const void* send, void* const* peer_recv, size_t bytes_per_rank, int W, int rank,
                          lancet_stream_t stream);
/* Count-aware all-to-all, replaces NCCLAllToAllv::Execute (nccl.cc:357-431) without its host
 * round trip: send is [W][n_chunks][chunk_elems]; for (peer i, chunk j) only the first
 * send_counts[i*n_chunks+j] elements (device uint64) travel, the rest of the destination chunk is
 * zero; the destination's recv_counts[rank*n_chunks+j] (uint64, peer_recv_counts[i]) receives the
 * count.  Follow with lancet_p2p_barrier. */
int lancet_all_to_allv_p2p(const void* send, void* const* peer_recv, const uint64_t* send_counts,
                           void* const* peer_recv_counts, int n_chunks, size_t elem_size, size_t chunk_elems,
                           int W, int rank, lancet_stream_t stream);

/* ---- expert FFN grouped GEMM (tcgen05 tensor cores, TMEM accumulators, TMA operand tiles) -------
 * Replaces the cuBLAS calls of the expert layers: GemmImpl (src/op/dialect/cublas/matmul.cc:30-78),
 * SparseExpertMatmulNtImpl (:211-303) and the per-expert loop of Experts.forward
 * (models/benchmark/pytorch/utils.py:546-562).  D[g] = act(A[g] * B[g % LE]^T + bias[g % LE]) for
 * g in [0, groups): A [groups][C][K], B [LE][N][K] (nn.Linear layout), D [groups][C][N], all bf16 or
 * fp16 with fp32 accumulation; bias [LE][N] and preact (copy of the pre-activation, [groups][C][N])
 * nullable.  counts (nullable, device int32 [groups]): only the first counts[g] rows of group g are
 * computed; rows from counts[g] up to the end of the last 128-row tile that holds a live row are
 * written as zeros, later rows are not touched.  act: 0 none, 1 relu, 2 gelu (erf), 3 gelu (tanh).
 * N % 256 == 0, K % 8 == 0; A, B and bias 16-byte aligned, D and preact 32-byte aligned (32-byte stores).
 * status: device int32, zero when healthy; a bounded wait that gave up stores its site there
 * (read it with lancet_p2p_status). */
int lancet_grouped_gemm_nt(const void* A, const void* B, void* D, const void* bias, void* preact, int groups,
                           int LE, int C, int N, int K, const int32_t* counts, int act, int dtype,
                           int32_t* status, lancet_stream_t stream);
/* Data gradient of the layer above (the reference's dX = matmul_nt(dy, w), src/op/grad/gemm.cc:31-36,
 * with w stored [N_out][K_in] so that the contraction runs over its rows):
 * D[g] = (A[g] * B[g % LE]) .* act'(preact[g]);  A [groups][C][K], B [LE][K][N] (N contiguous),
 * D and preact [groups][C][N]; preact is required when act != 0.  K % 64 == 0, N % 256 == 0. */
int lancet_grouped_gemm_nn(const void* A, const void* B, void* D, const void* preact, int groups, int LE, int C,
                           int N, int K, const int32_t* counts, int act, int dtype, int32_t* status,
                           lancet_stream_t stream);
/* Row-window forms of the two calls above for a pipelined exchange: group g is computed on rows
 * [row_begin[g] rounded down to a multiple of 128, row_end[g]) only (device int32 [groups] each, row_begin
 * nullable = 0); rows outside the window are not touched, except that rows from row_end[g] to the end of its
 * 128-row tile are written as zeros.  Row results do not depend on the windows they are computed in.
 * No reference counterpart: the reference runs one cuBLAS call per partition
 * (src/pass/dist_optimization/partition_exprs.cc:1745-1757 splits the expert matmuls with the tokens). */
int lancet_grouped_gemm_nt_window(const void* A, const void* B, void* D, const void* bias, void* preact, int groups,
                                  int LE, int C, int N, int K, const int32_t* row_begin, const int32_t* row_end,
                                  int act, int dtype, int32_t* status, lancet_stream_t stream);
int lancet_grouped_gemm_nn_window(const void* A, const void* B, void* D, const void* preact, int groups, int LE,
                                  int C, int N, int K, const int32_t* row_begin, const int32_t* row_end, int act,
                                  int dtype, int32_t* status, lancet_stream_t stream);
/* `sparse_expert_matmul_nt` (SparseExpertMatmulNtImpl, src/op/dialect/cublas/matmul.cc:144-326; schema
 * scripts/src_codegen/def_schema.py:711-718): data [C][G][M] (capacity-major, the G source ranks interleaved),
 * weight [N][M], out [C][G][N] = data * weight^T for the rows every source really sent:
 * rows_g = nelements_per_gpu[offset + g * stride] * scale / M (device uint64, the element counts `_all_to_allv`
 * returns), clamped to C.  Rows past rows_g are written as zeros (the count-aware path the reference sketches in
 * :221-247 and :289 but ships disabled: as shipped it multiplies the padded rows too, which gives the same output
 * when the padding is zero).  bf16 / fp16, N % 256 == 0, M % 8 == 0; the operands are read in place through a
 * 3-D tensor map, nothing is compacted.  ws: lancet_sparse_expert_matmul_nt_workspace_bytes(G) bytes, 16-byte
 * aligned (row counts and the status word of the bounded waits). */
size_t lancet_sparse_expert_matmul_nt_workspace_bytes(int G);
int lancet_sparse_expert_matmul_nt(const void* data, const void* weight, void* out, const uint64_t* nelements_per_gpu,
                                   int nelements_offset, int nelements_stride, int nelements_scale, int C, int G, int M,
                                   int N, int dtype, void* ws, size_t ws_bytes, lancet_stream_t stream);
/* Weight gradient (the reference's dW = matmul_tn(a, dy), src/op/grad/gemm.cc:31-36), summed over the
 * source ranks of an expert: D[e] = sum over groups g with g % LE == e of A[g][:counts[g]]^T * B[g][:counts[g]];
 * A [groups][C][Mout], B [groups][C][N], D [LE][Mout][N].  Rows from counts[g] to the next multiple
 * of 64 (or to C) must be zero in A or B and finite in both (the forms above leave their outputs that way;
 * dispatch zero-fills the expert input).  Mout % 128 == 0, N % 256 == 0. */
int lancet_grouped_gemm_tn(const void* A, const void* B, void* D, int groups, int LE, int C, int Mout, int N,
                           const int32_t* counts, int dtype, int32_t* status, lancet_stream_t stream);
/* Backward of combine fused with the exchange (moe_decode_dx + moe_decode_dg + _all_to_all of the
 * reference, src/op/dialect/cuda/moe.cc:1345-1375, :1431-1461): for every kept choice the row
 * gates * dout[s] is stored into the owner's d_expert_out buffer [W][LE][C][M] and
 * dgates_s [n][k][Sp] (float32) receives <expert_out row, dout[s]>.  Rows nobody owns are left to
 * the owner (zero-fill with lancet_moe_zero_tail and the row counts of the forward pass). */
int lancet_moe_combine_bwd_p2p(const void* dout, const void* gates_s, const int32_t* idx_loc,
                               void* const* peer_d_expert_out, void* const* peer_expert_out, void* dgates_s, int S,
                               int M, int C, int LE, int W, int rank, int k, int n_chunks, int dtype,
                               lancet_stream_t stream);
/* The two halves of lancet_moe_combine_bwd_p2p as separate launches, for schedules that start the expert GEMMs as soon
 * as the rows have been sent and compute the gate gradients beside them: part 1 = moe_decode_dx + _all_to_all
 * (src/op/dialect/cuda/moe.cc:1345-1375; stores to the owners only, dgates_s is not touched), part 2 = moe_decode_dg
 * (:1431-1461; loads of the owners' expert outputs only, peer_d_expert_out is not touched), part 0 = both in one pass.
 * Same bits as the joint pass.  A caller of part 2 must not pass the step's last flag barrier before that launch has
 * finished: the owners overwrite expert_out in their next forward pass. */
int lancet_moe_combine_bwd_part_p2p(const void* dout, const void* gates_s, const int32_t* idx_loc,
                                    void* const* peer_d_expert_out, void* const* peer_expert_out, void* dgates_s, int S,
                                    int M, int C, int LE, int W, int rank, int k, int n_chunks, int dtype, int part,
                                    lancet_stream_t stream);
/* Layer normalisation over the last axis (raf.op.layer_norm / layer_norm_dx of the reference, src/op/declare/nn.cc; one of the
 * non-MoE operators next to the MoE layer that the reference's forward partition splits into token chunks,
 * src/pass/dist_optimization/partition_exprs.cc:1709-1795).  x [rows][M] float32, M a multiple of 128 up to 2048 in
 * {128,256,512,768,1024,1536,2048}; y in out_dtype (float32, or the 16-bit type the next GEMM reads: no cast pass);
 * mean, rstd [rows] float32 are kept for the backward pass.  A row's result depends on that row only. */
int lancet_layer_norm_fwd(const float* x, const float* gamma, const float* beta, void* y, int out_dtype, float* mean, float* rstd,
                          int rows, int M, float eps, lancet_stream_t stream);
/* dx [rows][M] float32, dgamma, dbeta [M] float32 from dy [rows][M] in dy_dtype; ws: lancet_layer_norm_workspace_bytes(rows, M)
 * bytes (partial column sums; they are added in a fixed order: reproducible). */
size_t lancet_layer_norm_workspace_bytes(int rows, int M);
int lancet_layer_norm_bwd(const float* x, const void* dy, int dy_dtype, const float* gamma, const float* mean, const float* rstd,
                          float* dx, float* dgamma, float* dbeta, int rows, int M, void* ws, size_t ws_bytes,
                          lancet_stream_t stream);
/* Softmax cross-entropy of the language-model head over a padded vocabulary; replaces the log_softmax + nll_loss pair the
 * reference's benchmark models end in (models/benchmark/raf/raf_bencher.py:84; raf.op.nll_loss and nll_loss_dpred,
 * src/op/declare/loss.cc:55-92) without materialising float32 logits or log-probabilities.
 * logits [rows][ld] (ld >= vocab elements between rows; columns >= vocab are padding and never read), target [rows] int64
 * (negative or >= vocab = ignored row), loss_rows[r] = logsumexp(row r) - logits[r][target[r]] (0 for ignored rows), lse_rows[r] kept for
 * the backward pass. */
int lancet_softmax_xent_fwd(const void* logits, long long ld, const long long* target, int rows, int vocab, int dtype,
                            float* loss_rows, float* lse_rows, lancet_stream_t stream);
/* dlogits[r][j] = (softmax(row r)[j] - [j == target[r]]) * (*grad_out) * scale for j < vocab; 0 for vocab <= j < cols and in
 * ignored rows.  grad_out is a float32 scalar in device memory (nullptr = 1): no host round trip; scale is the host-side
 * reduction factor (1 / number of live rows for a mean).  dlogits [rows][ldd] has the logits' type. */
int lancet_softmax_xent_bwd(const void* logits, long long ld, const long long* target, int rows, int vocab, int cols, int dtype,
                            const float* lse_rows, const float* grad_out, float scale, void* dlogits, long long ldd,
                            lancet_stream_t stream);
/* Bias gradient of an expert layer: db[e][:] = sum over the groups of expert e and their live rows of
 * dY[g][r][:]  (dY [groups][C][N], db [LE][N]); the reference gets it from the autodiff of nn.Linear's
 * bias add (a `sum` over rows).  ws: lancet_grouped_bias_grad_workspace_bytes(LE, N) bytes. */
size_t lancet_grouped_bias_grad_workspace_bytes(int LE, int N);
int lancet_grouped_bias_grad(const void* dY, void* db, int groups, int LE, int C, int N, const int32_t* counts,
                             int dtype, void* ws, size_t ws_bytes, lancet_stream_t stream);

/* ---- gate projection -----------------------------------------------------------------------------
 * probs [S,E] float32 = softmax(h [S,M] * wg [E,M]^T): the Linear(bias = False) + softmax in front of moe_encode
 * (Gate module, models/benchmark/pytorch/utils.py:565-573; TopKGate.forward, docker/resources/sharded_moe.py:370-390),
 * which the reference leaves to library GEMM and softmax operators.  One warp per token in a fixed order, fp32
 * accumulation: a token's probabilities do not depend on how the tokens are split into calls, which is what lets a
 * chunked pipeline reproduce the unchunked routing bit for bit.  E <= 64.  The backward form returns
 * dlogits [S,E] float32 (for the weight gradient dlogits^T * h, left to the caller) and dh [S,M] in `dtype`. */
int lancet_gate_softmax(const void* h, int dtype, const float* wg, float* probs, int S, int M, int E,
                        lancet_stream_t stream);
int lancet_gate_softmax_bwd(const float* probs, const float* dprobs, const float* wg, float* dlogits, void* dh,
                            int dtype, int S, int M, int E, lancet_stream_t stream);

/* ---- scheduling knobs and a plain copy ----------------------------------------------------------
 * No counterpart in the reference, whose kernels take whatever grid the library picks.  The static
 * schedule that stands in for the reference's overlap pass (src/pass/dist_optimization/lancet_optimization.cc)
 * runs an exchange stage beside an expert GEMM; both would otherwise ask for every SM and time-slice.
 * exchange_ctas caps the grid of the peer-memory exchange kernels, gemm_ctas the persistent grid of the
 * grouped GEMM (0 = no cap).  Process-wide; change it between steps, not while launches are being issued
 * from another thread. */
int lancet_set_cta_limits(int exchange_ctas, int gemm_ctas);
/* Grouped GEMM form, for A/B timing (same results bit for bit).  Bit 0: 1 (default) = two CTAs of a cluster share a
 * 256 x 256 tile (tcgen05 cta_group::2) whenever the shape allows it, 0 = always the single-CTA 128 x 256 form.
 * Bit 1: 0 (default) = the tile walk visits all (source, expert) groups of one expert before the next expert's, so
 * that an expert's weights stay in L2; 1 = groups in index order. */
int lancet_set_gemm_paired(int mode);
/* The short dependent kernels of the dispatch path (gate selection, slot assignment, scatter, combine) are launched with
 * programmatic stream serialization: the next kernel's CTAs become resident while the previous kernel drains and wait, as
 * their first instruction, until it has completed.  Results do not change; 0 switches to plain launches (A/B timing).
 * No counterpart in the reference (one TVM/CUDA launch per operator, src/op/dialect/cuda/moe.cc:364-395). */
int lancet_set_chained_launch(int on);
/* cudaMemcpyAsync(dst, src, bytes) with the kind inferred from the pointers; dst or src may be a peer
 * mapping from lancet_symm_open (copy-engine transfer over NVLink; the bandwidth yardstick of bench.py). */
int lancet_peer_copy(void* dst, const void* src, size_t bytes, lancet_stream_t stream);

/* ---- LANS optimizer ---------------------------------------------------------------------------
 * Replaces multi_tensor_lans_cuda (kernel_util.cuh:26-34; multi_tensor_lans.cu:401-450) and the
 * host side of LansImpl::Execute (src/op/dialect/cuda/lans.cc:92-148).  g/p/m/v are HOST arrays of
 * n_tensors device pointers (float32 tensors, updated in place except g), numels a host array.
 * `step` is the 1-based step count as a host integer (the reference reads it back from the
 * device, lans.cc:102-107); bias corrections are computed from it on the host (lans.cc:108-117).
 * ws: lancet_lans_workspace_bytes() bytes, 16-byte aligned, kept by the caller between steps.
 * With LANCET_LANS_TABLES_READY the tensor table uploaded by an earlier call with the same
 * pointers, sizes and workspace is reused and the call is launch-only. */
enum { LANCET_LANS_TABLES_READY = 1 };
size_t lancet_lans_workspace_bytes(int n_tensors, const int64_t* numels);
int lancet_lans(void* ws, size_t ws_bytes, int n_tensors, const int64_t* numels, void* const* g, void* const* p,
                void* const* m, void* const* v, int dtype, int step, float lr, float beta1, float beta2, float eps,
                int bias_correction, float weight_decay, int grad_averaging, int mode, int normalize_grad, int flags,
                lancet_stream_t stream);
/* The same step with the step count left where the reference's op receives it: a float32 scalar in DEVICE
 * memory (`step` tensor of raf.op.lans, read as (int)value).  The reference copies it to the host and waits
 * (lans.cc:102-107: CopyTo(cpu) = a device-wide synchronisation per optimizer step); here a one-thread kernel
 * derives the bias corrections (lans.cc:108-113) on the stream and the call stays asynchronous.
 * Only use LANCET_LANS_TABLES_READY with a workspace nobody else writes between the calls. */
int lancet_lans_dev_step(void* ws, size_t ws_bytes, int n_tensors, const int64_t* numels, void* const* g, void* const* p,
                         void* const* m, void* const* v, int dtype, const float* step_dev, float lr, float beta1, float beta2,
                         float eps, int bias_correction, float weight_decay, int grad_averaging, int mode,
                         int normalize_grad, int flags, lancet_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LANCET_B200_H_ */
