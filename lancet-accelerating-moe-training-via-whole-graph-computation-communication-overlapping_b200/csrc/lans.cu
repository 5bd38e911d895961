// Multi-tensor LANS optimizer step: three launches for any number of tensors.
//
// Replaces multi_tensor_lans_cuda (src/op/dialect/cuda/kernels/multi_tensor_lans.cu:401-450)
// and LansImpl::Execute (src/op/dialect/cuda/lans.cc:92-148) of the reference, which run four
// separate L2-norm sweeps (each with a memset and a cleanup launch) around two update stages,
// split into many launches by a 4 KB kernel-argument table, store both update directions to
// memory, and read `step` back from the device every call.
//
// Here the data dependence of the algorithm sets the passes:
//   phase 1  reads g                   -> ||g||                                  ( 4 B/element)
//   phase 2  reads g, p, m, v          -> writes m, v; ||p||, ||u_m||, ||u_g||   (24 B/element)
//   phase 3  reads g, p, m, v          -> writes p                               (20 B/element)
// ||g|| has to be known before anything else (the gradient is scaled by it); ||p|| is only needed by phase 3, so it is
// summed in phase 2, which reads p anyway.
// The update directions u_m, u_g are recomputed in phase 3 instead of being stored.  The tensor
// table lives in device memory (no per-launch tensor limit).  Per-tensor norms are reduced in
// a fixed order (per-chunk partial sums, then the last block to finish a tensor adds them up),
// so results are reproducible run to run.  The gradient tensors are left untouched (the
// reference overwrites them with u_m as a side effect of its stage 1).
#include <vector>

#include "common.cuh"

namespace lancet {

constexpr int kLansChunk = 8192;  // elements per block
constexpr int kLansThreads = 256;

struct LansTensor {
  float* g;
  float* p;
  float* m;
  float* v;
  long long numel;
  int chunk_begin;
  int nchunks;
};

struct LansHyper {
  float lr, beta1, beta2, beta3, eps, bc1, bc2, wd;
  float inv_bc1, inv_bc2;  // reciprocals: one IEEE division per element instead of four
  int mode, normalize_grad;
};

struct LansLayout {
  size_t tensors_off, part1_off, part2_off, norms_off, counters_off, bc_off, map_off, total;
  long long nchunks;
};

static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

static LansLayout lans_layout(int n, const int64_t* numels) {
  LansLayout L;
  long long nch = 0;
  for (int i = 0; i < n; ++i) nch += (numels[i] + kLansChunk - 1) / kLansChunk;
  L.nchunks = nch;
  size_t off = 0;
  L.tensors_off = off; off += up256((size_t)n * sizeof(LansTensor));
  L.part1_off = off;   off += up256((size_t)(nch > 0 ? nch : 1) * sizeof(float2));
  L.part2_off = off;   off += up256((size_t)(nch > 0 ? nch : 1) * sizeof(float2));
  L.norms_off = off;   off += up256((size_t)n * sizeof(float4));
  L.counters_off = off; off += up256((size_t)n * 2 * sizeof(int));
  L.bc_off = off;       off += 256;  // 1/bias_correction1, 1/bias_correction2 when the step counter lives on the device
  L.map_off = off;      off += up256((size_t)(nch > 0 ? nch : 1) * sizeof(int));   // tensor of every chunk
  L.total = off;
  return L;
}

__device__ __forceinline__ int find_tensor(const LansTensor* __restrict__ t, int n, int chunk) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (t[mid].chunk_begin <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Built with the tensor table: the tensor a chunk belongs to.  A block lives for one chunk, and a binary search through
// the table in global memory (eight dependent loads for 200 tensors) was a quarter of the life of a phase-1 block.
__global__ void lans_chunk_map_kernel(const LansTensor* __restrict__ tensors, int n, int nchunks, int* __restrict__ map) {
  const int chunk = blockIdx.x * blockDim.x + threadIdx.x;
  if (chunk < nchunks) map[chunk] = find_tensor(tensors, n, chunk);
}

__device__ __forceinline__ float2 block_sum2(float a, float b) {
  __shared__ float2 red[kLansThreads / 32];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, d);
    b += __shfl_xor_sync(0xffffffffu, b, d);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = make_float2(a, b);
  __syncthreads();
  float2 r = make_float2(0.f, 0.f);
  if (threadIdx.x < 32) {
    float2 x = threadIdx.x < kLansThreads / 32 ? red[threadIdx.x] : make_float2(0.f, 0.f);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      x.x += __shfl_xor_sync(0xffffffffu, x.x, d);
      x.y += __shfl_xor_sync(0xffffffffu, x.y, d);
    }
    r = x;
  }
  return r;  // valid in thread 0
}

// Publishes this block's partial and, in the last block of the tensor, adds all partials in
// chunk order and writes sqrt of the sums to out[0] (and out[1] with n_out == 2).
__device__ __forceinline__ void finish_tensor(float2 mine, float2* __restrict__ partials, int* __restrict__ counter,
                                              const LansTensor& T, int chunk, float* __restrict__ out, int n_out = 2) {
  __shared__ int is_last;
  __syncthreads();   // a second call in the same kernel must not overwrite is_last under a thread still reading it
  if (threadIdx.x == 0) {
    partials[chunk] = mine;
    __threadfence();
    const int ticket = atomicAdd(counter, 1);
    is_last = (ticket == T.nchunks - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float a = 0.f, b = 0.f;
  for (int c = threadIdx.x; c < T.nchunks; c += kLansThreads) {
    const float2 q = __ldcg(&partials[T.chunk_begin + c]);
    a += q.x;
    b += q.y;
  }
  const float2 tot = block_sum2(a, b);
  if (threadIdx.x == 0) {
    out[0] = sqrtf(tot.x);
    if (n_out == 2) out[1] = sqrtf(tot.y);
    *counter = 0;  // ready for the next step
  }
}

// Hardware square root and reciprocal (one special-function instruction each, relative error about 2^-23)
// instead of the IEEE-rounded sequences: the difference is two orders below the 1e-5 tolerance of the op.
__device__ __forceinline__ float sqrt_fast(float x) {
  float y;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
  float y;
  asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// `inv_gn` is 1 / (||g|| + eps) when the gradient is normalised, else 1.  Multiplying by reciprocals
// instead of dividing changes results by at most a few ulp, far inside the 1e-5 tolerance.
__device__ __forceinline__ void lans_directions(float g, float p, float& m, float& v, float inv_gn, const LansHyper& h,
                                                float& um, float& ug) {
  float sg = g * inv_gn;
  if (h.mode == 0) sg = sg + h.wd * p;
  m = m * h.beta1 + h.beta3 * sg;
  v = v * h.beta2 + (1.0f - h.beta2) * sg * sg;
  const float r = rcp_fast(sqrt_fast(v * h.inv_bc2) + h.eps);
  const float sp = h.mode == 0 ? 0.0f : h.wd * p;
  um = (m * h.inv_bc1) * r + sp;
  ug = sg * r + sp;
}

// Same as above with m, v already updated (phase 3).
__device__ __forceinline__ void lans_directions_post(float g, float p, float m, float v, float inv_gn,
                                                     const LansHyper& h, float& um, float& ug) {
  float sg = g * inv_gn;
  if (h.mode == 0) sg = sg + h.wd * p;
  const float r = rcp_fast(sqrt_fast(v * h.inv_bc2) + h.eps);
  const float sp = h.mode == 0 ? 0.0f : h.wd * p;
  um = (m * h.inv_bc1) * r + sp;
  ug = sg * r + sp;
}

__device__ __forceinline__ float grad_scale(float gnorm, const LansHyper& h) {
  return (h.normalize_grad && gnorm != 0.0f) ? 1.0f / (gnorm + h.eps) : 1.0f;
}

struct ChunkView {
  long long off;
  int n;      // elements in this chunk
  int nvec;   // float4 groups handled with 16-byte accesses
};

__device__ __forceinline__ ChunkView chunk_view(const LansTensor& T, int chunk, bool need_mv) {
  ChunkView c;
  c.off = (long long)(chunk - T.chunk_begin) * kLansChunk;
  const long long left = T.numel - c.off;
  c.n = left < kLansChunk ? (int)left : kLansChunk;
  uintptr_t bits = reinterpret_cast<uintptr_t>(T.g) | reinterpret_cast<uintptr_t>(T.p);
  if (need_mv) bits |= reinterpret_cast<uintptr_t>(T.m) | reinterpret_cast<uintptr_t>(T.v);
  c.nvec = (bits & 15) == 0 ? c.n / 4 : 0;
  return c;
}

__global__ void __launch_bounds__(kLansThreads)
lans_phase1_kernel(const LansTensor* __restrict__ tensors, const int* __restrict__ chunk_map, float2* __restrict__ part1,
                   float4* __restrict__ norms, int* __restrict__ counters) {
  const int chunk = blockIdx.x;
  const int t = chunk_map[chunk];
  const LansTensor T = tensors[t];
  const ChunkView c = chunk_view(T, chunk, false);
  const float4* g4 = reinterpret_cast<const float4*>(T.g + c.off);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int i = threadIdx.x;
  // a full chunk is eight vectors per thread: all eight loads are issued before the first sum (a block lives for one
  // chunk only, so what it has in flight at once is what hides the memory latency)
  for (; i + 7 * kLansThreads < c.nvec; i += 8 * kLansThreads) {
    float4 a[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) a[u] = __ldcs(g4 + i + u * kLansThreads);
#pragma unroll
    for (int u = 0; u < 8; u += 4) {
      s0 += a[u].x * a[u].x + a[u].y * a[u].y + a[u].z * a[u].z + a[u].w * a[u].w;
      s1 += a[u + 1].x * a[u + 1].x + a[u + 1].y * a[u + 1].y + a[u + 1].z * a[u + 1].z + a[u + 1].w * a[u + 1].w;
      s2 += a[u + 2].x * a[u + 2].x + a[u + 2].y * a[u + 2].y + a[u + 2].z * a[u + 2].z + a[u + 2].w * a[u + 2].w;
      s3 += a[u + 3].x * a[u + 3].x + a[u + 3].y * a[u + 3].y + a[u + 3].z * a[u + 3].z + a[u + 3].w * a[u + 3].w;
    }
  }
  for (; i < c.nvec; i += kLansThreads) {
    const float4 a = g4[i];
    s0 += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  for (int e = c.nvec * 4 + threadIdx.x; e < c.n; e += kLansThreads) {
    const float a = T.g[c.off + e];
    s0 += a * a;
  }
  const float2 mine = block_sum2((s0 + s1) + (s2 + s3), 0.f);
  finish_tensor(mine, part1, counters + 2 * t, T, chunk, reinterpret_cast<float*>(norms + t), 1);
}

// 1/bias_correction from a step counter that lives on the device (a float scalar, as the reference's op takes it:
// src/op/dialect/cuda/lans.cc:102-113, which copies it to the host first).
__global__ void lans_bias_correction_kernel(const float* __restrict__ step, float beta1, float beta2, int bias_correction,
                                            float* __restrict__ inv_bc) {
  float bc1 = 1.0f, bc2 = 1.0f;
  if (bias_correction == 1) {
    const int n = (int)step[0];
    bc1 = (float)(1 - pow((double)beta1, n));
    bc2 = (float)(1 - pow((double)beta2, n));
  }
  inv_bc[0] = 1.0f / bc1;
  inv_bc[1] = 1.0f / bc2;
}

__device__ __forceinline__ void load_bc(LansHyper& h, const float* __restrict__ inv_bc_dev) {
  if (inv_bc_dev) {
    h.inv_bc1 = __ldg(inv_bc_dev);
    h.inv_bc2 = __ldg(inv_bc_dev + 1);
  }
}

__device__ __forceinline__ void phase2_vec(const float4& g, const float4& p, float4& m, float4& v, float inv_gn,
                                           const LansHyper& h, float& sm, float& sq) {
  float um, ug;
  lans_directions(g.x, p.x, m.x, v.x, inv_gn, h, um, ug); sm += um * um; sq += ug * ug;
  lans_directions(g.y, p.y, m.y, v.y, inv_gn, h, um, ug); sm += um * um; sq += ug * ug;
  lans_directions(g.z, p.z, m.z, v.z, inv_gn, h, um, ug); sm += um * um; sq += ug * ug;
  lans_directions(g.w, p.w, m.w, v.w, inv_gn, h, um, ug); sm += um * um; sq += ug * ug;
}

// Two vectors of each of the four arrays are loaded before any arithmetic or store: the stores of one iteration
// cannot be moved below the next iteration's loads by the compiler (the arrays may alias as far as it knows), so
// with one vector per array a thread had 64 bytes in flight and the kernel sat at 0.82 of the copy bandwidth.
__global__ void __launch_bounds__(kLansThreads)
lans_phase2_kernel(const LansTensor* __restrict__ tensors, const int* __restrict__ chunk_map, LansHyper h,
                   const float* __restrict__ inv_bc_dev, float2* __restrict__ part1, float2* __restrict__ part2,
                   float4* __restrict__ norms, int* __restrict__ counters) {
  const int chunk = blockIdx.x;
  const int t = chunk_map[chunk];
  const LansTensor T = tensors[t];
  const ChunkView c = chunk_view(T, chunk, true);
  load_bc(h, inv_bc_dev);
  const float gnorm = grad_scale(__ldcg(reinterpret_cast<const float*>(norms + t)), h);
  const float4* g4 = reinterpret_cast<const float4*>(T.g + c.off);
  const float4* p4 = reinterpret_cast<const float4*>(T.p + c.off);
  float4* m4 = reinterpret_cast<float4*>(T.m + c.off);
  float4* v4 = reinterpret_cast<float4*>(T.v + c.off);
  float sm = 0.f, sq = 0.f, sm2 = 0.f, sq2 = 0.f, sp = 0.f, sp2 = 0.f;
  int i = threadIdx.x;
  for (; i + kLansThreads < c.nvec; i += 2 * kLansThreads) {
    const int j = i + kLansThreads;
    const float4 ga = __ldcs(g4 + i), pa = __ldcs(p4 + i), gb = __ldcs(g4 + j), pb = __ldcs(p4 + j);
    float4 ma = __ldcs(m4 + i), va = __ldcs(v4 + i), mb = __ldcs(m4 + j), vb = __ldcs(v4 + j);
    sp += pa.x * pa.x + pa.y * pa.y + pa.z * pa.z + pa.w * pa.w;
    sp2 += pb.x * pb.x + pb.y * pb.y + pb.z * pb.z + pb.w * pb.w;
    phase2_vec(ga, pa, ma, va, gnorm, h, sm, sq);
    phase2_vec(gb, pb, mb, vb, gnorm, h, sm2, sq2);
    m4[i] = ma;
    v4[i] = va;
    m4[j] = mb;
    v4[j] = vb;
  }
  for (; i < c.nvec; i += kLansThreads) {
    const float4 g = g4[i], p = p4[i];
    float4 m = m4[i], v = v4[i];
    sp += p.x * p.x + p.y * p.y + p.z * p.z + p.w * p.w;
    phase2_vec(g, p, m, v, gnorm, h, sm, sq);
    m4[i] = m;
    v4[i] = v;
  }
  for (int e = c.nvec * 4 + threadIdx.x; e < c.n; e += kLansThreads) {
    float m = T.m[c.off + e], v = T.v[c.off + e], um, ug;
    const float p = T.p[c.off + e];
    sp += p * p;
    lans_directions(T.g[c.off + e], p, m, v, gnorm, h, um, ug);
    sm += um * um;
    sq += ug * ug;
    T.m[c.off + e] = m;
    T.v[c.off + e] = v;
  }
  const float2 mine = block_sum2(sm + sm2, sq + sq2);
  const float2 minep = block_sum2(sp + sp2, 0.f);
  finish_tensor(mine, part2, counters + 2 * t + 1, T, chunk, reinterpret_cast<float*>(norms + t) + 2);
  // ||p||: the partial array and the ticket counter of phase 1 are free again (its last block reset the counter)
  finish_tensor(minep, part1, counters + 2 * t, T, chunk, reinterpret_cast<float*>(norms + t) + 1, 1);
}

__device__ __forceinline__ void phase3_vec(const float4& g, float4& p, const float4& m, const float4& v, float inv_gn,
                                           const LansHyper& h, float rm, float rg) {
  float um, ug;
  lans_directions_post(g.x, p.x, m.x, v.x, inv_gn, h, um, ug); p.x = p.x - rm * um - rg * ug;
  lans_directions_post(g.y, p.y, m.y, v.y, inv_gn, h, um, ug); p.y = p.y - rm * um - rg * ug;
  lans_directions_post(g.z, p.z, m.z, v.z, inv_gn, h, um, ug); p.z = p.z - rm * um - rg * ug;
  lans_directions_post(g.w, p.w, m.w, v.w, inv_gn, h, um, ug); p.w = p.w - rm * um - rg * ug;
}

__global__ void __launch_bounds__(kLansThreads)
lans_phase3_kernel(const LansTensor* __restrict__ tensors, const int* __restrict__ chunk_map, LansHyper h,
                   const float* __restrict__ inv_bc_dev, const float4* __restrict__ norms) {
  const int chunk = blockIdx.x;
  const int t = chunk_map[chunk];
  const LansTensor T = tensors[t];
  const ChunkView c = chunk_view(T, chunk, true);
  load_bc(h, inv_bc_dev);
  const float4 nr = __ldcg(norms + t);  // ||g||, ||p||, ||u_m||, ||u_g||
  float rm = (nr.z != 0.0f && nr.y != 0.0f) ? h.lr * (nr.y / nr.z) : h.lr;
  float rg = (nr.w != 0.0f && nr.y != 0.0f) ? h.lr * (nr.y / nr.w) : h.lr;
  rm *= h.beta1;
  rg *= h.beta3;
  const float inv_gn = grad_scale(nr.x, h);
  const float4* g4 = reinterpret_cast<const float4*>(T.g + c.off);
  float4* p4 = reinterpret_cast<float4*>(T.p + c.off);
  const float4* m4 = reinterpret_cast<const float4*>(T.m + c.off);
  const float4* v4 = reinterpret_cast<const float4*>(T.v + c.off);
  int i = threadIdx.x;
  for (; i + kLansThreads < c.nvec; i += 2 * kLansThreads) {
    const int j = i + kLansThreads;
    const float4 ga = __ldcs(g4 + i), ma = __ldcs(m4 + i), va = __ldcs(v4 + i);
    const float4 gb = __ldcs(g4 + j), mb = __ldcs(m4 + j), vb = __ldcs(v4 + j);
    float4 pa = __ldcs(p4 + i), pb = __ldcs(p4 + j);
    phase3_vec(ga, pa, ma, va, inv_gn, h, rm, rg);
    phase3_vec(gb, pb, mb, vb, inv_gn, h, rm, rg);
    p4[i] = pa;
    p4[j] = pb;
  }
  for (; i < c.nvec; i += kLansThreads) {
    const float4 g = g4[i], m = m4[i], v = v4[i];
    float4 p = p4[i];
    phase3_vec(g, p, m, v, inv_gn, h, rm, rg);
    p4[i] = p;
  }
  for (int e = c.nvec * 4 + threadIdx.x; e < c.n; e += kLansThreads) {
    float um, ug;
    const float p = T.p[c.off + e];
    lans_directions_post(T.g[c.off + e], p, T.m[c.off + e], T.v[c.off + e], inv_gn, h, um, ug);
    T.p[c.off + e] = p - rm * um - rg * ug;
  }
}

}  // namespace lancet

extern "C" {
using namespace lancet;

size_t lancet_lans_workspace_bytes(int n_tensors, const int64_t* numels) {
  if (n_tensors <= 0 || !numels) return 0;
  for (int i = 0; i < n_tensors; ++i)
    if (numels[i] < 0) return 0;
  return lans_layout(n_tensors, numels).total;
}

static int lans_impl(void* ws, size_t ws_bytes, int n_tensors, const int64_t* numels, void* const* g, void* const* p,
                     void* const* m, void* const* v, int dtype, int step, const float* step_dev, float lr, float beta1,
                     float beta2, float eps, int bias_correction, float weight_decay, int grad_averaging, int mode,
                     int normalize_grad, int flags, lancet_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  LANCET_REQUIRE(n_tensors >= 0, LANCET_ERR_INVALID, "lancet_lans: negative tensor count %d", n_tensors);
  if (n_tensors == 0) return LANCET_OK;
  LANCET_REQUIRE(dtype == LANCET_F32, LANCET_ERR_UNSUPPORTED,
                 "lancet_lans: only float32 tensors are supported (dtype code %d)", dtype);
  LANCET_REQUIRE(ws && numels, LANCET_ERR_NULL, "lancet_lans: null workspace or numels");
  LANCET_REQUIRE((flags & ~LANCET_LANS_TABLES_READY) == 0, LANCET_ERR_INVALID, "lancet_lans: unknown flag bits 0x%x", flags);
  LANCET_REQUIRE(mode == 0 || mode == 1, LANCET_ERR_INVALID, "lancet_lans: mode must be 0 or 1, got %d", mode);
  LANCET_REQUIRE(step_dev || step >= 1, LANCET_ERR_INVALID, "lancet_lans: step must be >= 1, got %d", step);
  for (int i = 0; i < n_tensors; ++i)
    LANCET_REQUIRE(numels[i] >= 0, LANCET_ERR_INVALID, "lancet_lans: tensor %d has negative size", i);
  const LansLayout L = lans_layout(n_tensors, numels);
  LANCET_REQUIRE(ws_bytes >= L.total, LANCET_ERR_INVALID, "lancet_lans: workspace of %zu bytes is smaller than the %zu needed",
                 ws_bytes, L.total);
  LANCET_REQUIRE(aligned(ws, 16), LANCET_ERR_INVALID, "lancet_lans: workspace must be 16-byte aligned");
  LANCET_REQUIRE(L.nchunks < (1ll << 31), LANCET_ERR_INVALID, "lancet_lans: too many elements");
  char* base = static_cast<char*>(ws);
  LansTensor* d_tensors = reinterpret_cast<LansTensor*>(base + L.tensors_off);
  if (!(flags & LANCET_LANS_TABLES_READY)) {
    LANCET_REQUIRE(g && p && m && v, LANCET_ERR_NULL, "lancet_lans: null pointer table");
    std::vector<LansTensor> host((size_t)n_tensors);
    int begin = 0;
    for (int i = 0; i < n_tensors; ++i) {
      LANCET_REQUIRE(numels[i] == 0 || (g[i] && p[i] && m[i] && v[i]), LANCET_ERR_NULL, "lancet_lans: tensor %d has a null pointer", i);
      LANCET_REQUIRE(aligned(g[i], 4) && aligned(p[i], 4) && aligned(m[i], 4) && aligned(v[i], 4), LANCET_ERR_INVALID,
                     "lancet_lans: tensor %d is not 4-byte aligned", i);
      host[i].g = static_cast<float*>(g[i]);
      host[i].p = static_cast<float*>(p[i]);
      host[i].m = static_cast<float*>(m[i]);
      host[i].v = static_cast<float*>(v[i]);
      host[i].numel = numels[i];
      host[i].chunk_begin = begin;
      host[i].nchunks = (int)((numels[i] + kLansChunk - 1) / kLansChunk);
      begin += host[i].nchunks;
    }
    // pageable source: the runtime stages the bytes before returning, so `host` may go out of scope
    LANCET_CUDA(cudaMemcpyAsync(d_tensors, host.data(), host.size() * sizeof(LansTensor), cudaMemcpyHostToDevice, stream));
    LANCET_CUDA(cudaMemsetAsync(base + L.counters_off, 0, (size_t)n_tensors * 2 * sizeof(int), stream));
    // tensors without elements never finish a block: their norms stay defined as zero
    LANCET_CUDA(cudaMemsetAsync(base + L.norms_off, 0, (size_t)n_tensors * sizeof(float4), stream));
    if (L.nchunks > 0) {
      lans_chunk_map_kernel<<<(int)((L.nchunks + 255) / 256), 256, 0, stream>>>(d_tensors, n_tensors, (int)L.nchunks,
                                                                               reinterpret_cast<int*>(base + L.map_off));
      if (int st = launch_status("lans_chunk_map_kernel")) return st;
    }
  }
  if (L.nchunks == 0) return LANCET_OK;
  LansHyper h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.wd = weight_decay;
  h.mode = mode; h.normalize_grad = normalize_grad ? 1 : 0;
  // host-side bias correction, as src/op/dialect/cuda/lans.cc:108-117 of the reference
  h.bc1 = 1.0f; h.bc2 = 1.0f;
  float* inv_bc_dev = nullptr;
  if (step_dev) {
    inv_bc_dev = reinterpret_cast<float*>(base + L.bc_off);
    lans_bias_correction_kernel<<<1, 1, 0, stream>>>(step_dev, beta1, beta2, bias_correction, inv_bc_dev);
    if (int st = launch_status("lans_bias_correction_kernel")) return st;
  } else if (bias_correction == 1) {
    h.bc1 = (float)(1 - std::pow((double)beta1, step));
    h.bc2 = (float)(1 - std::pow((double)beta2, step));
  }
  h.beta3 = grad_averaging == 1 ? 1 - beta1 : 1.0f;
  h.inv_bc1 = 1.0f / h.bc1;
  h.inv_bc2 = 1.0f / h.bc2;
  float2* part1 = reinterpret_cast<float2*>(base + L.part1_off);
  float2* part2 = reinterpret_cast<float2*>(base + L.part2_off);
  float4* norms = reinterpret_cast<float4*>(base + L.norms_off);
  int* counters = reinterpret_cast<int*>(base + L.counters_off);
  const int* chunk_map = reinterpret_cast<const int*>(base + L.map_off);
  const int grid = (int)L.nchunks;
  {
    ProfScope prof("lans_phase1_kernel", stream);
    lans_phase1_kernel<<<grid, kLansThreads, 0, stream>>>(d_tensors, chunk_map, part1, norms, counters);
  }
  if (int st = launch_status("lans_phase1_kernel")) return st;
  {
    ProfScope prof("lans_phase2_kernel", stream);
    lans_phase2_kernel<<<grid, kLansThreads, 0, stream>>>(d_tensors, chunk_map, h, inv_bc_dev, part1, part2, norms, counters);
  }
  if (int st = launch_status("lans_phase2_kernel")) return st;
  {
    ProfScope prof("lans_phase3_kernel", stream);
    lans_phase3_kernel<<<grid, kLansThreads, 0, stream>>>(d_tensors, chunk_map, h, inv_bc_dev, norms);
  }
  return launch_status("lans_phase3_kernel");
}

int lancet_lans(void* ws, size_t ws_bytes, int n_tensors, const int64_t* numels, void* const* g, void* const* p,
                void* const* m, void* const* v, int dtype, int step, float lr, float beta1, float beta2, float eps,
                int bias_correction, float weight_decay, int grad_averaging, int mode, int normalize_grad, int flags,
                lancet_stream_t stream) {
  return lans_impl(ws, ws_bytes, n_tensors, numels, g, p, m, v, dtype, step, nullptr, lr, beta1, beta2, eps, bias_correction,
                   weight_decay, grad_averaging, mode, normalize_grad, flags, stream);
}

int lancet_lans_dev_step(void* ws, size_t ws_bytes, int n_tensors, const int64_t* numels, void* const* g, void* const* p,
                         void* const* m, void* const* v, int dtype, const float* step_dev, float lr, float beta1, float beta2,
                         float eps, int bias_correction, float weight_decay, int grad_averaging, int mode,
                         int normalize_grad, int flags, lancet_stream_t stream) {
  LANCET_REQUIRE(step_dev, LANCET_ERR_NULL, "lancet_lans_dev_step: null step pointer");
  return lans_impl(ws, ws_bytes, n_tensors, numels, g, p, m, v, dtype, 0, step_dev, lr, beta1, beta2, eps, bias_correction,
                   weight_decay, grad_averaging, mode, normalize_grad, flags, stream);
}
}
