// `_all_to_all` and `_all_to_allv` as stand-alone operators.
//
// Two transports behind the same semantics (out chunk i <- rank i's chunk `rank`, equal split of the
// flattened tensor; NCCLAllToAll::Execute, src/op/dialect/nccl/nccl.cc:199-227 of the reference):
//  * NCCL: grouped ncclSend/ncclRecv pairs exactly as the reference issues them; works on any
//    caller-owned buffers.  NCCL is loaded with dlopen at first use, so the library itself has no
//    link-time dependency on it.
//  * peer memory: when the receive buffers live in symmetric memory (lancet_symm_alloc), one copy
//    kernel stores every chunk straight into its destination GPU; ranks then meet at
//    lancet_p2p_barrier.  The count-aware variant ships only the first send_counts elements of each
//    chunk and the counts themselves, without the device-to-host copy and stream synchronisation of
//    NCCLAllToAllv::Execute (nccl.cc:357-431, host sync at :388-390).
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "common.cuh"

namespace lancet {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommCount)(const ncclComm_t, int*) = nullptr;
  ncclResult_t (*CommUserRank)(const ncclComm_t, int*) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

static NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) return;
#define LOAD(field, sym)                                                  \
  api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, sym)); \
  if (!api.field) return;
    LOAD(GetUniqueId, "ncclGetUniqueId");
    LOAD(CommInitRank, "ncclCommInitRank");
    LOAD(CommDestroy, "ncclCommDestroy");
    LOAD(CommCount, "ncclCommCount");
    LOAD(CommUserRank, "ncclCommUserRank");
    LOAD(GroupStart, "ncclGroupStart");
    LOAD(GroupEnd, "ncclGroupEnd");
    LOAD(Send, "ncclSend");
    LOAD(Recv, "ncclRecv");
    LOAD(GetErrorString, "ncclGetErrorString");
#undef LOAD
    api.ok = true;
  });
  return api;
}

#define LANCET_NCCL(expr)                                                                              \
  do {                                                                                                 \
    ncclResult_t _r = (expr);                                                                          \
    if (_r != ncclSuccess)                                                                             \
      return ::lancet::fail(LANCET_ERR_COMM, "%s failed: %s", #expr, ::lancet::nccl().GetErrorString(_r)); \
  } while (0)

constexpr int kMaxPeersA2A = 16;
struct PeerTableA {
  void* ptr[kMaxPeersA2A];
};

// Copy chunk `dst` of my send buffer into block `my_rank` of rank dst's receive buffer.  A warp moves 4 KB
// pieces (8 independent 16-byte loads per lane, then 8 stores, like the fused dispatch kernel); consecutive
// pieces go to different destinations so that all links are busy all the time.
__global__ void __launch_bounds__(256)
a2a_store_kernel(const uint4* __restrict__ send, PeerTableA recv, size_t vecs_per_rank, int W, int my_rank) {
  constexpr int U = 8;
  const int lane = threadIdx.x & 31;
  const size_t pieces_per_rank = (vecs_per_rank + 32 * U - 1) / (32 * U);
  const size_t tasks = pieces_per_rank * W;
  const size_t gw = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const size_t nw = (size_t)gridDim.x * 8;
  for (size_t t = gw; t < tasks; t += nw) {
    const int dst = (int)((t + my_rank) % W);          // start at a different peer on every rank
    const size_t base = (t / W) * (32 * U);
    const uint4* s = send + (size_t)dst * vecs_per_rank + base;
    uint4* d = static_cast<uint4*>(recv.ptr[dst]) + (size_t)my_rank * vecs_per_rank + base;
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = (size_t)u * 32 + lane;
      if (base + v < vecs_per_rank) r[u] = __ldcs(s + v);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = (size_t)u * 32 + lane;
      if (base + v < vecs_per_rank) d[v] = r[u];
    }
  }
}

// Count-aware variant: for destination dst and chunk j only the first send_counts[dst*n_chunks+j]
// elements travel; the rest of the destination chunk is zero-filled; the count is stored into
// recv_counts[my_rank*n_chunks + j] on the destination.  grid = (blocks, n_chunks, W).
__global__ void __launch_bounds__(256)
a2av_store_kernel(const unsigned char* __restrict__ send, PeerTableA recv, PeerTableA recv_counts,
                  const unsigned long long* __restrict__ send_counts, int n_chunks, size_t chunk_bytes, int elem_size,
                  int my_rank) {
  const int dst = blockIdx.z, j = blockIdx.y;
  unsigned long long cnt = send_counts[(size_t)dst * n_chunks + j];
  size_t live = (size_t)cnt * elem_size;
  if (live > chunk_bytes) live = chunk_bytes;
  const size_t src_off = ((size_t)dst * n_chunks + j) * chunk_bytes;
  const size_t dst_off = ((size_t)my_rank * n_chunks + j) * chunk_bytes;
  const unsigned char* s = send + src_off;
  unsigned char* d = static_cast<unsigned char*>(recv.ptr[dst]) + dst_off;
  if (blockIdx.x == 0 && threadIdx.x == 0)
    static_cast<unsigned long long*>(recv_counts.ptr[dst])[(size_t)my_rank * n_chunks + j] = cnt;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // chunk_bytes and both bases are multiples of 16: move whole 16-byte words, zero the tail words
  const size_t live_vecs = live / 16, vecs = chunk_bytes / 16;
  const uint4* s4 = reinterpret_cast<const uint4*>(s);
  uint4* d4 = reinterpret_cast<uint4*>(d);
  for (size_t i = tid; i < live_vecs; i += stride) d4[i] = __ldcs(s4 + i);
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (size_t i = live_vecs + tid; i < vecs; i += stride) {
    if (i == live_vecs && (live & 15)) {
      // word that holds the boundary: live bytes then zeros
      uint4 w = s4[i];
      unsigned char* wb = reinterpret_cast<unsigned char*>(&w);
      for (int b = (int)(live & 15); b < 16; ++b) wb[b] = 0;
      d4[i] = w;
    } else {
      d4[i] = z;
    }
  }
}

// NCCL transport of the count-aware exchange: whole chunks travel, then everything past the received count is
// cleared in place.  grid = (blocks, n_chunks, W).
__global__ void __launch_bounds__(256)
a2av_mask_kernel(unsigned char* __restrict__ recv, const unsigned long long* __restrict__ recv_counts, int n_chunks,
                 size_t chunk_bytes, int elem_size) {
  const int src = blockIdx.z, j = blockIdx.y;
  size_t live = (size_t)recv_counts[(size_t)src * n_chunks + j] * elem_size;
  if (live > chunk_bytes) live = chunk_bytes;
  uint4* d4 = reinterpret_cast<uint4*>(recv + ((size_t)src * n_chunks + j) * chunk_bytes);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t live_vecs = live / 16, vecs = chunk_bytes / 16;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (size_t i = live_vecs + tid; i < vecs; i += stride) {
    if (i == live_vecs && (live & 15)) {
      uint4 w = d4[i];
      unsigned char* wb = reinterpret_cast<unsigned char*>(&w);
      for (int b = (int)(live & 15); b < 16; ++b) wb[b] = 0;
      d4[i] = w;
    } else {
      d4[i] = z;
    }
  }
}

}  // namespace lancet

extern "C" {
using namespace lancet;

int lancet_comm_unique_id(unsigned char* id128) {
  LANCET_REQUIRE(id128, LANCET_ERR_NULL, "lancet_comm_unique_id: null argument");
  LANCET_REQUIRE(nccl().ok, LANCET_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
  ncclUniqueId id;
  LANCET_NCCL(nccl().GetUniqueId(&id));
  memcpy(id128, &id, 128);
  return LANCET_OK;
}

int lancet_comm_init_rank(const unsigned char* id128, int world, int rank, lancet_comm_t* comm) {
  LANCET_REQUIRE(id128 && comm, LANCET_ERR_NULL, "lancet_comm_init_rank: null argument");
  LANCET_REQUIRE(world >= 1 && rank >= 0 && rank < world, LANCET_ERR_INVALID, "lancet_comm_init_rank: bad world %d / rank %d", world, rank);
  LANCET_REQUIRE(nccl().ok, LANCET_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  ncclComm_t c = nullptr;
  LANCET_NCCL(nccl().CommInitRank(&c, world, id, rank));
  *comm = c;
  return LANCET_OK;
}

int lancet_comm_destroy(lancet_comm_t comm) {
  if (!comm) return LANCET_OK;
  LANCET_REQUIRE(nccl().ok, LANCET_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  LANCET_NCCL(nccl().CommDestroy(static_cast<ncclComm_t>(comm)));
  return LANCET_OK;
}

int lancet_all_to_all(const void* send, void* recv, size_t bytes_per_rank, lancet_comm_t comm, lancet_stream_t stream) {
  LANCET_REQUIRE(comm, LANCET_ERR_NULL, "lancet_all_to_all: null communicator");
  LANCET_REQUIRE(nccl().ok, LANCET_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  if (bytes_per_rank == 0) return LANCET_OK;  // nccl.cc:220: nothing is issued for an empty tensor
  LANCET_REQUIRE(send && recv, LANCET_ERR_NULL, "lancet_all_to_all: null buffer");
  ncclComm_t c = static_cast<ncclComm_t>(comm);
  int W = 0;
  LANCET_NCCL(nccl().CommCount(c, &W));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const char* s = static_cast<const char*>(send);
  char* r = static_cast<char*>(recv);
  LANCET_NCCL(nccl().GroupStart());
  for (int i = 0; i < W; ++i) {
    ncclResult_t a = nccl().Send(s + (size_t)i * bytes_per_rank, bytes_per_rank, ncclInt8, i, c, st);
    ncclResult_t b = a == ncclSuccess ? nccl().Recv(r + (size_t)i * bytes_per_rank, bytes_per_rank, ncclInt8, i, c, st) : a;
    if (b != ncclSuccess) {
      nccl().GroupEnd();
      return fail(LANCET_ERR_COMM, "ncclSend/ncclRecv failed: %s", nccl().GetErrorString(b));
    }
  }
  LANCET_NCCL(nccl().GroupEnd());
  count_launch();
  return LANCET_OK;
}

int lancet_all_to_all_evenly(const void* send, void* recv, size_t total_bytes, lancet_comm_t comm, lancet_stream_t stream) {
  LANCET_REQUIRE(comm, LANCET_ERR_NULL, "lancet_all_to_all_evenly: null communicator");
  LANCET_REQUIRE(nccl().ok, LANCET_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  int W = 0;
  LANCET_NCCL(nccl().CommCount(static_cast<ncclComm_t>(comm), &W));
  LANCET_REQUIRE(W > 0 && total_bytes % (size_t)W == 0, LANCET_ERR_INVALID,
                 "Cannot evenly distribute input tensor to all ranks (%zu bytes over %d ranks).", total_bytes, W);
  return lancet_all_to_all(send, recv, total_bytes / W, comm, stream);
}

// Tuple form (nccl.cc:228-277 of the reference): the per-rank slices of all tensors are packed next to each
// other into `in_ws`, exchanged in one grouped all-to-all into `out_ws` and unpacked.  The reference issues
// 2*W*n_tensors cudaMemcpyAsync calls for the packing; here one kernel launch packs and one unpacks.
struct TupleTable {
  const void* src[16];
  void* dst[16];
  unsigned long long bytes_per_rank[16];
  unsigned long long offset[16];  // offset of tensor t inside a rank's packed block
  unsigned long long block;       // packed bytes per rank
};

__global__ void __launch_bounds__(256) a2a_pack_kernel(TupleTable t, unsigned char* __restrict__ ws, int pack) {
  const int tensor = blockIdx.y, rank = blockIdx.z;
  const unsigned long long n = t.bytes_per_rank[tensor];
  unsigned char* packed = ws + (unsigned long long)rank * t.block + t.offset[tensor];
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (pack) {
    const unsigned char* s = static_cast<const unsigned char*>(t.src[tensor]) + (unsigned long long)rank * n;
    if ((n & 15) == 0 && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(packed)) & 15) == 0) {
      for (unsigned long long i = tid; i < n / 16; i += stride) reinterpret_cast<uint4*>(packed)[i] = reinterpret_cast<const uint4*>(s)[i];
    } else {
      for (unsigned long long i = tid; i < n; i += stride) packed[i] = s[i];
    }
  } else {
    unsigned char* d = static_cast<unsigned char*>(t.dst[tensor]) + (unsigned long long)rank * n;
    if ((n & 15) == 0 && ((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(packed)) & 15) == 0) {
      for (unsigned long long i = tid; i < n / 16; i += stride) reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(packed)[i];
    } else {
      for (unsigned long long i = tid; i < n; i += stride) d[i] = packed[i];
    }
  }
}

int lancet_all_to_all_tuple(const void* const* sends, void* const* recvs, const size_t* nbytes, int n_tensors, void* in_ws,
                            void* out_ws, size_t ws_bytes, lancet_comm_t comm, lancet_stream_t stream) {
  LANCET_REQUIRE(n_tensors >= 1 && n_tensors <= 16, LANCET_ERR_INVALID, "lancet_all_to_all_tuple: 1 to 16 tensors, got %d", n_tensors);
  LANCET_REQUIRE(sends && recvs && nbytes && in_ws && out_ws && comm, LANCET_ERR_NULL, "lancet_all_to_all_tuple: null argument");
  LANCET_REQUIRE(nccl().ok, LANCET_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  int W = 0;
  LANCET_NCCL(nccl().CommCount(static_cast<ncclComm_t>(comm), &W));
  TupleTable t;
  size_t total = 0, block = 0;
  for (int i = 0; i < n_tensors; ++i) {
    LANCET_REQUIRE(sends[i] && recvs[i], LANCET_ERR_NULL, "lancet_all_to_all_tuple: tensor %d is null", i);
    LANCET_REQUIRE(nbytes[i] % (size_t)W == 0, LANCET_ERR_INVALID,
                   "Cannot evenly distribute input tensor to all ranks (tensor %d: %zu bytes over %d ranks).", i, nbytes[i], W);
    t.src[i] = sends[i];
    t.dst[i] = recvs[i];
    t.bytes_per_rank[i] = nbytes[i] / W;
    t.offset[i] = block;
    block += nbytes[i] / W;
    total += nbytes[i];
  }
  t.block = block;
  LANCET_REQUIRE(ws_bytes >= total, LANCET_ERR_INVALID, "lancet_all_to_all_tuple: workspaces of %zu bytes are smaller than the %zu needed",
                 ws_bytes, total);
  if (total == 0) return LANCET_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int bx = sm_count() * 4 / (n_tensors * W) + 1;
  a2a_pack_kernel<<<dim3(bx, n_tensors, W), 256, 0, st>>>(t, static_cast<unsigned char*>(in_ws), 1);
  if (int rc = launch_status("a2a_pack_kernel")) return rc;
  if (int rc = lancet_all_to_all(in_ws, out_ws, block, comm, stream)) return rc;
  a2a_pack_kernel<<<dim3(bx, n_tensors, W), 256, 0, st>>>(t, static_cast<unsigned char*>(out_ws), 0);
  return launch_status("a2a_pack_kernel");
}

int lancet_all_to_all_p2p(const void* send, void* const* peer_recv, size_t bytes_per_rank, int W, int rank,
                          lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeersA2A && rank >= 0 && rank < W, LANCET_ERR_INVALID,
                 "lancet_all_to_all_p2p: bad world %d / rank %d (at most %d ranks)", W, rank, kMaxPeersA2A);
  if (bytes_per_rank == 0) return LANCET_OK;
  LANCET_REQUIRE(send && peer_recv, LANCET_ERR_NULL, "lancet_all_to_all_p2p: null argument");
  LANCET_REQUIRE(bytes_per_rank % 16 == 0 && aligned(send, 16), LANCET_ERR_INVALID,
                 "lancet_all_to_all_p2p: the per-rank chunk (%zu bytes) must be a multiple of 16 bytes and aligned", bytes_per_rank);
  PeerTableA t;
  for (int i = 0; i < kMaxPeersA2A; ++i) t.ptr[i] = i < W ? peer_recv[i] : nullptr;
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(t.ptr[i] && aligned(t.ptr[i], 16), LANCET_ERR_NULL, "lancet_all_to_all_p2p: peer buffer %d is null or unaligned", i);
  const size_t vecs = bytes_per_rank / 16;
  long long bx = (long long)(((vecs + 255) / 256 * W + 7) / 8);
  long long cap = (long long)sm_count() * 8;
  if (exchange_cta_limit() > 0 && exchange_cta_limit() < cap) cap = exchange_cta_limit();
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ProfScope prof("a2a_store_kernel", st);
  a2a_store_kernel<<<(unsigned)bx, 256, 0, st>>>(static_cast<const uint4*>(send), t, vecs, W, rank);
  return launch_status("a2a_store_kernel");
}

int lancet_all_to_allv(const void* send, void* recv, const uint64_t* send_counts, uint64_t* recv_counts, int n_chunks,
                       size_t elem_size, size_t chunk_elems, lancet_comm_t comm, lancet_stream_t stream) {
  LANCET_REQUIRE(comm, LANCET_ERR_NULL, "lancet_all_to_allv: null communicator");
  LANCET_REQUIRE(nccl().ok, LANCET_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  LANCET_REQUIRE(n_chunks >= 1 && n_chunks <= 65535 && elem_size >= 1 && elem_size <= 16, LANCET_ERR_INVALID,
                 "lancet_all_to_allv: bad n_chunks %d or element size %zu", n_chunks, elem_size);
  LANCET_REQUIRE(send_counts && recv_counts, LANCET_ERR_NULL, "lancet_all_to_allv: null counts");
  const size_t chunk_bytes = chunk_elems * elem_size;
  int W = 0;
  LANCET_NCCL(nccl().CommCount(static_cast<ncclComm_t>(comm), &W));
  LANCET_REQUIRE(W >= 1 && W <= 65535, LANCET_ERR_INVALID, "lancet_all_to_allv: bad communicator size %d", W);
  if (int rc = lancet_all_to_all(send_counts, recv_counts, (size_t)n_chunks * sizeof(uint64_t), comm, stream)) return rc;
  if (chunk_bytes == 0) return LANCET_OK;
  LANCET_REQUIRE(send && recv, LANCET_ERR_NULL, "lancet_all_to_allv: null buffer");
  LANCET_REQUIRE(chunk_bytes % 16 == 0 && aligned(recv, 16), LANCET_ERR_INVALID,
                 "lancet_all_to_allv: the chunk (%zu bytes) must be a multiple of 16 bytes and recv 16-byte aligned", chunk_bytes);
  if (int rc = lancet_all_to_all(send, recv, (size_t)n_chunks * chunk_bytes, comm, stream)) return rc;
  long long bx = (long long)((chunk_bytes / 16 + 255) / 256);
  const long long cap = (long long)sm_count() * 8 / ((long long)W * n_chunks) + 1;
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  a2av_mask_kernel<<<dim3((unsigned)bx, n_chunks, W), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned char*>(recv), reinterpret_cast<const unsigned long long*>(recv_counts), n_chunks, chunk_bytes,
      (int)elem_size);
  return launch_status("a2av_mask_kernel");
}

int lancet_all_to_allv_p2p(const void* send, void* const* peer_recv, const uint64_t* send_counts,
                           void* const* peer_recv_counts, int n_chunks, size_t elem_size, size_t chunk_elems, int W,
                           int rank, lancet_stream_t stream) {
  LANCET_REQUIRE(W >= 1 && W <= kMaxPeersA2A && rank >= 0 && rank < W, LANCET_ERR_INVALID,
                 "lancet_all_to_allv_p2p: bad world %d / rank %d (at most %d ranks)", W, rank, kMaxPeersA2A);
  LANCET_REQUIRE(n_chunks >= 1 && n_chunks <= 65535 && elem_size >= 1 && elem_size <= 16, LANCET_ERR_INVALID,
                 "lancet_all_to_allv_p2p: bad n_chunks %d or element size %zu", n_chunks, elem_size);
  const size_t chunk_bytes = chunk_elems * elem_size;
  if (chunk_bytes == 0) return LANCET_OK;
  LANCET_REQUIRE(send && peer_recv && send_counts && peer_recv_counts, LANCET_ERR_NULL, "lancet_all_to_allv_p2p: null argument");
  LANCET_REQUIRE(chunk_bytes % 16 == 0 && aligned(send, 16), LANCET_ERR_INVALID,
                 "lancet_all_to_allv_p2p: the chunk (%zu bytes) must be a multiple of 16 bytes and aligned", chunk_bytes);
  PeerTableA t, tc;
  for (int i = 0; i < kMaxPeersA2A; ++i) {
    t.ptr[i] = i < W ? peer_recv[i] : nullptr;
    tc.ptr[i] = i < W ? peer_recv_counts[i] : nullptr;
  }
  for (int i = 0; i < W; ++i)
    LANCET_REQUIRE(t.ptr[i] && tc.ptr[i] && aligned(t.ptr[i], 16) && aligned(tc.ptr[i], 8), LANCET_ERR_NULL,
                   "lancet_all_to_allv_p2p: peer buffer %d is null or unaligned", i);
  long long bx = (long long)((chunk_bytes / 16 + 255) / 256);
  const long long cap = (long long)sm_count() * 8 / ((long long)W * n_chunks) + 1;
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  a2av_store_kernel<<<dim3((unsigned)bx, n_chunks, W), 256, 0, st>>>(
      static_cast<const unsigned char*>(send), t, tc, reinterpret_cast<const unsigned long long*>(send_counts), n_chunks,
      chunk_bytes, (int)elem_size, rank);
  return launch_status("a2av_store_kernel");
}
}
