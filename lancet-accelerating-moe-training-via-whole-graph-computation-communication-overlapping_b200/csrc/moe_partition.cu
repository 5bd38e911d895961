// Re-compaction operators of a partitioned MoE layer: moe_merge_masks, moe_redispatch and
// moe_redispatch_expert_input.
//
// The reference's scheduler emits them after n chained moe_encode calls whose partitions each own a
// full-size buffer (src/pass/dist_optimization/partition_exprs.cc:474-594); its kernels use one block
// per expert (or per source rank) and a pinned host pointer table copied to the device on every call
// (src/op/dialect/cuda/moe.cc:731-1073, kernels/tutel_moe_dispatch.cu:214-255, :365-459).  Here the
// pointer table travels as a kernel argument, the per-partition counts are one histogram pass over
// all partitions, and rows are moved by a warp each with 16-byte accesses.  (The chunked dispatch of
// this library never needs these operators; they exist for graphs that were partitioned the
// reference's way.)
#include "common.cuh"

namespace lancet {

constexpr int kMaxParts = 16;
struct PartTable {
  const void* ptr[kMaxParts];
};

// counts[p][e] = number of tokens of partition p kept for expert e.
__global__ void __launch_bounds__(256)
partition_hist_kernel(PartTable idx_locs, int S, int E, int* __restrict__ counts) {
  extern __shared__ int h[];
  const int p = blockIdx.y;
  for (int i = threadIdx.x; i < E; i += blockDim.x) h[i] = 0;
  __syncthreads();
  const int32_t* idx = static_cast<const int32_t*>(idx_locs.ptr[p]);
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gridDim.x * blockDim.x) {
    const int e = idx[s];
    if (e >= 0 && e < E) atomicAdd(&h[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (h[i]) atomicAdd(&counts[p * E + i], h[i]);
}

__global__ void __launch_bounds__(256)
merge_masks_kernel(PartTable idx_locs, int n, int S, int E, const int* __restrict__ counts, int32_t* __restrict__ out) {
  const int p = blockIdx.y;
  const int32_t* il = static_cast<const int32_t*>(idx_locs.ptr[p]);
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gridDim.x * blockDim.x) {
    const int e = il[s];
    int o_idx = -1, o_loc = -1;
    if (e >= 0 && e < E) {
      int base = 0;
      for (int q = 0; q < p; ++q) base += counts[q * E + e];
      o_idx = e;
      o_loc = il[S + s] + base;
    }
    out[(size_t)p * S + s] = o_idx;
    out[(size_t)n * S + (size_t)p * S + s] = o_loc;
  }
}

// One warp per output row (e, r): copy from the partition that owns it, or zero.
template <typename V>
__global__ void __launch_bounds__(256)
redispatch_kernel(PartTable datas, int n, int E, int C, int row_vecs, const int* __restrict__ counts, V* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const long long nw = (long long)gridDim.x * 8;
  for (long long row = gw; row < (long long)E * C; row += nw) {
    const int e = (int)(row / C), r = (int)(row % C);
    int base = 0, p = 0;
    for (; p < n; ++p) {
      const int c = counts[p * E + e];
      if (r < base + c) break;
      base += c;
    }
    V* dst = out + (size_t)row * row_vecs;
    if (p < n) {
      const V* src = static_cast<const V*>(datas.ptr[p]) + ((size_t)e * C + (r - base)) * row_vecs;
      for (int v = lane; v < row_vecs; v += 32) dst[v] = src[v];
    } else {
      V z;
      memset(&z, 0, sizeof(V));
      for (int v = lane; v < row_vecs; v += 32) dst[v] = z;
    }
  }
}

// [C,G,M] layout: column g of the output is the concatenation, partition after partition, of the first
// recv_counts[p][g*LE + le] * scale elements of column g of partition p (elements counted along (c, m)).
template <typename T>
__global__ void __launch_bounds__(256)
redispatch_expert_input_kernel(PartTable datas, PartTable recv_counts, int n, int le, int LE, int C, int G, int M,
                               int scale, T* __restrict__ out) {
  const long long per_col = (long long)C * M;
  const long long total = per_col * G;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i % M);
    const int g = (int)((i / M) % G);
    const int c = (int)(i / ((long long)M * G));
    const long long q = (long long)c * M + m;  // position inside column g
    long long base = 0;
    int p = 0;
    for (; p < n; ++p) {
      long long cnt = (long long)static_cast<const unsigned long long*>(recv_counts.ptr[p])[g * LE + le] * scale;
      if (cnt > per_col) cnt = per_col;
      if (q < base + cnt) break;
      base += cnt;
    }
    T v = Num<T>::from_f(0.f);
    if (p < n) {
      const long long qs = q - base;
      v = static_cast<const T*>(datas.ptr[p])[((qs / M) * G + g) * M + (qs % M)];
    }
    out[i] = v;
  }
}

static int fill_table(PartTable* t, const void* const* ptrs, int n, const char* fn) {
  LANCET_REQUIRE(n >= 1 && n <= kMaxParts, LANCET_ERR_INVALID, "%s: 1 to %d partitions are supported, got %d", fn, kMaxParts, n);
  LANCET_REQUIRE(ptrs, LANCET_ERR_NULL, "%s: null pointer table", fn);
  for (int i = 0; i < kMaxParts; ++i) t->ptr[i] = nullptr;
  for (int i = 0; i < n; ++i) {
    LANCET_REQUIRE(ptrs[i], LANCET_ERR_NULL, "%s: partition %d is null", fn, i);
    t->ptr[i] = ptrs[i];
  }
  return LANCET_OK;
}

static int grid_for(long long items, int per_block) {
  long long b = (items + per_block - 1) / per_block;
  const long long cap = (long long)sm_count() * 8;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

static int run_hist(const PartTable& t, int n, int S, int E, int* counts, cudaStream_t st) {
  LANCET_CUDA(cudaMemsetAsync(counts, 0, (size_t)n * E * sizeof(int), st));
  if (S == 0) return LANCET_OK;
  int bx = grid_for(S, 256);
  if (bx > 64) bx = 64;
  partition_hist_kernel<<<dim3(bx, n), 256, (size_t)E * sizeof(int), st>>>(t, S, E, counts);
  return launch_status("partition_hist_kernel");
}

}  // namespace lancet

extern "C" {
using namespace lancet;

size_t lancet_moe_partition_workspace_bytes(int n_partitions, int E) {
  if (n_partitions < 1 || E < 1) return 0;
  return ((size_t)n_partitions * E * sizeof(int) + 255) / 256 * 256;
}

int lancet_moe_merge_masks(const int32_t* const* idx_locs, int n_partitions, int S, int E, int32_t* out, void* ws,
                           size_t ws_bytes, lancet_stream_t stream) {
  PartTable t;
  if (int rc = fill_table(&t, reinterpret_cast<const void* const*>(idx_locs), n_partitions, "lancet_moe_merge_masks")) return rc;
  LANCET_REQUIRE(S >= 0 && E >= 1 && E <= 8192, LANCET_ERR_INVALID, "lancet_moe_merge_masks: bad sizes S=%d E=%d", S, E);
  LANCET_REQUIRE(ws && ws_bytes >= lancet_moe_partition_workspace_bytes(n_partitions, E), LANCET_ERR_INVALID,
                 "lancet_moe_merge_masks: workspace missing or too small");
  if (S == 0) return LANCET_OK;
  LANCET_REQUIRE(out, LANCET_ERR_NULL, "lancet_moe_merge_masks: null output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* counts = static_cast<int*>(ws);
  if (int rc = run_hist(t, n_partitions, S, E, counts, st)) return rc;
  int bx = grid_for(S, 256);
  merge_masks_kernel<<<dim3(bx, n_partitions), 256, 0, st>>>(t, n_partitions, S, E, counts, out);
  return launch_status("merge_masks_kernel");
}

int lancet_moe_redispatch(const void* const* datas, const int32_t* const* idx_locs, int n_partitions, int S, int M, int C,
                          int E, int dtype, void* out, void* ws, size_t ws_bytes, lancet_stream_t stream) {
  PartTable td, ti;
  if (int rc = fill_table(&td, datas, n_partitions, "lancet_moe_redispatch")) return rc;
  if (int rc = fill_table(&ti, reinterpret_cast<const void* const*>(idx_locs), n_partitions, "lancet_moe_redispatch")) return rc;
  LANCET_REQUIRE(S >= 0 && M >= 0 && C >= 0 && E >= 1 && E <= 8192 && valid_dtype(dtype), LANCET_ERR_INVALID,
                 "lancet_moe_redispatch: bad sizes S=%d M=%d C=%d E=%d or dtype", S, M, C, E);
  LANCET_REQUIRE(ws && ws_bytes >= lancet_moe_partition_workspace_bytes(n_partitions, E), LANCET_ERR_INVALID,
                 "lancet_moe_redispatch: workspace missing or too small");
  if ((size_t)E * C * M == 0) return LANCET_OK;
  LANCET_REQUIRE(out, LANCET_ERR_NULL, "lancet_moe_redispatch: null output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* counts = static_cast<int*>(ws);
  if (int rc = run_hist(ti, n_partitions, S, E, counts, st)) return rc;
  const size_t row_bytes = (size_t)M * dtype_bytes(dtype);
  bool a16 = row_bytes % 16 == 0 && aligned(out, 16);
  for (int i = 0; i < n_partitions; ++i) a16 = a16 && aligned(datas[i], 16);
  const int grid = grid_for((long long)E * C, 8);
  if (a16)
    redispatch_kernel<uint4><<<grid, 256, 0, st>>>(td, n_partitions, E, C, (int)(row_bytes / 16), counts, static_cast<uint4*>(out));
  else
    redispatch_kernel<uint16_t><<<grid, 256, 0, st>>>(td, n_partitions, E, C, (int)(row_bytes / 2), counts,
                                                      static_cast<uint16_t*>(out));
  return launch_status("redispatch_kernel");
}

int lancet_moe_redispatch_expert_input(const void* const* datas, const uint64_t* const* recv_counts, int n_partitions,
                                       int local_expert_id, int n_local_experts, int C, int G, int M, int recv_cnts_scale,
                                       int dtype, void* out, lancet_stream_t stream) {
  PartTable td, tc;
  if (int rc = fill_table(&td, datas, n_partitions, "lancet_moe_redispatch_expert_input")) return rc;
  if (int rc = fill_table(&tc, reinterpret_cast<const void* const*>(recv_counts), n_partitions, "lancet_moe_redispatch_expert_input")) return rc;
  LANCET_REQUIRE(C >= 0 && G >= 1 && M >= 0 && n_local_experts >= 1 && local_expert_id >= 0 && local_expert_id < n_local_experts &&
                     recv_cnts_scale >= 1 && valid_dtype(dtype),
                 LANCET_ERR_INVALID, "lancet_moe_redispatch_expert_input: bad sizes or dtype");
  const long long total = (long long)C * G * M;
  if (total == 0) return LANCET_OK;
  LANCET_REQUIRE(out, LANCET_ERR_NULL, "lancet_moe_redispatch_expert_input: null output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(total, 256 * 4);
#define LANCET_REI(T)                                                                                              \
  redispatch_expert_input_kernel<T><<<grid, 256, 0, st>>>(td, tc, n_partitions, local_expert_id, n_local_experts, C, G, M, \
                                                          recv_cnts_scale, static_cast<T*>(out))
  if (dtype == LANCET_F32) LANCET_REI(float);
  else if (dtype == LANCET_F16) LANCET_REI(__half);
  else LANCET_REI(__nv_bfloat16);
#undef LANCET_REI
  return launch_status("redispatch_expert_input_kernel");
}
}
