// Expert FFN grouped GEMM on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces the cuBLAS calls behind the reference's expert layers: GemmImpl
// (src/op/dialect/cublas/matmul.cc:30-78, fp16/bf16 inputs with fp32 accumulation),
// SparseExpertMatmulNtImpl (:211-303, which as shipped multiplies the whole padded buffer) and the
// per-expert loop of Experts.forward (models/benchmark/pytorch/utils.py:546-562).
//
//   D[g] = act(A[g] * B[e(g)]^T + bias[e(g)])        g = group = (source rank, local expert)
//
// A is the post-exchange expert input [groups][C][K] (row blocks of C rows, K contiguous), B the
// expert weights [LE][N][K] in nn.Linear layout (K contiguous), D [groups][C][N].  Only the first
// counts[g] rows of a group are live: tiles past them are skipped, which is what the reference's
// count-aware path intended (cublas/matmul.cc:221-247, commented out there).
//
// Two forms of the kernel.  In the paired form (the default whenever the shape allows it) the two CTAs of a
// thread-block cluster share one 256 x 256 output tile through tcgen05.mma.cta_group::2: each CTA stages its own 128
// rows of A and its own 128 of the 256 columns' worth of B (32 KB per pipeline stage instead of 48, six stages instead
// of four), the even CTA issues the MMAs for both, and every CTA keeps its 128 x 256 half of the accumulator in its
// own TMEM.  Half the B bytes per FLOP pass through shared memory, which is what limits the single-CTA form.  All TMA
// loads are plain (no cluster multicast): each CTA fetches its own operands and signals the even CTA's barrier.
//
// Single-CTA form: one persistent CTA per SM walks a static list of 128 x 256 output tiles.  Warp 0 is the TMA
// producer (cp.async.bulk.tensor into 128-byte-swizzled shared memory, 4 stages of 64-wide K
// blocks), warp 1 issues tcgen05.mma (one thread) into one of two 256-column TMEM accumulators,
// warps 2-9 are the epilogue (tcgen05.ld, bias + activation, 16-byte stores; two warps per TMEM lane quadrant), so the epilogue of
// tile i overlaps the main loop of tile i+1.  Every mbarrier wait is bounded: when a limit runs
// out the CTA raises an abort flag, records the site in *status, lets copies in flight land, frees
// its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

namespace lancet {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int MAX_GROUPS = 1024;              // row-parallel forms keep a per-group tile table in shared memory
constexpr int SCHED_BYTES = (2 * MAX_GROUPS + 1) * 4;
// CTA2 = the paired form: a CTA holds B for 128 of the tile's 256 columns
template <bool CTA2>
struct Cfg {
  static constexpr int STAGES = CTA2 ? 6 : 4;
  static constexpr int B_COLS = CTA2 ? BN / 2 : BN;          // output columns whose B operand this CTA stages
  static constexpr int B_STAGE_BYTES = B_COLS * BK * 2;       // 16 or 32 KB
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int SMEM_DATA = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = SMEM_DATA + 1024 /*alignment slack*/ + 256 /*barriers*/ + SCHED_BYTES;
};
constexpr int EPI_WARPS = 8;                 // two warps per TMEM lane quadrant, each takes half of the columns
constexpr int THREADS = 64 + 32 * EPI_WARPS; // warps: 0 TMA, 1 MMA, 2.. epilogue
constexpr int TMEM_COLS = 512;               // two accumulators of BN fp32 columns
constexpr int MAX_BAND = 16;                 // upper bound of the m-units per band (L2 reuse of A against a sweep of B)
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// MODE_ROWS:   D[g] (C x N) = epilogue(A[g] (C x K) * op(B[e])), tiles over (group, m-tile, n-tile), reduction over K.
//              B is [LE][N][K] (K-major, "NT") or [LE][K][N] (N contiguous, "NN", B_MN).
// MODE_REDUCE: D[e] (Mout x N) = sum over groups g of expert e and their live rows r of A[g][r][:]^T * B[g][r][:]
//              ("TN": weight gradients), tiles over (expert, m-tile, n-tile), reduction over rows.
constexpr int MODE_ROWS = 0, MODE_REDUCE = 1;
constexpr int EPI_ACT = 0, EPI_DACT = 1, EPI_ACT_PRE = 2;  // ACT_PRE: as ACT, and the pre-activation is stored too

struct Params {
  int groups, LE, C, N, K;
  int Mout;               // MODE_REDUCE: output rows per expert
  int m_tiles, n_tiles, tiles_per_group, total_tiles;
  int band;               // MODE_ROWS: m-units per band of the tile order
  int expert_major;       // MODE_ROWS: walk all groups of an expert before the next expert's
  const int32_t* counts;  // [groups] live rows (end of the row window), or null
  const int32_t* row_lo;  // [groups] first row of the window (rounded down to a tile boundary), or null; MODE_ROWS only
  int interleaved;        // MODE_ROWS: A, D and preact are [C][groups][.] (row c of group g at c * groups + g) instead of [groups][C][.]
  const void* bias;       // [LE][N] or null
  void* D;
  void* preact;           // EPI_ACT: optional copy of the pre-activation; EPI_DACT: the saved pre-activation (input)
  int act;                // 0 none, 1 relu, 2 gelu (erf), 3 gelu (tanh)
  int epi;
  int paired;             // host side: launch the paired (two CTAs per 256 x 256 tile) form
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (now_ns() - t0 > WAIT_LIMIT_NS) {
      *abort_flag = 1;
      atomicCAS(status, 0, site);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// 3-D form for tensors viewed [groups][C][cols]: rows past C are out of bounds in their own dimension and
// arrive as zeros instead of running into the next group.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Paired form: the same loads, completing on the mbarrier of the even CTA of the pair (`bar` is a shared::cluster
// address made with leader_addr); no multicast, every CTA loads its own operands.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// arrives (once the MMAs issued so far have completed) on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 64 bf16 (128 bytes) with the
// 128-byte swizzle TMA applies: 8 rows form a 1024-byte atom, atoms follow each other along M/N.
// 32-byte store (one full sector per lane): half as many store transactions as two 16-byte stores.
__device__ __forceinline__ void st_global_32B(void* ptr, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
               "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}

__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);   // start address
  d |= (uint64_t)1 << 16;                  // leading byte offset (unused with swizzle, canonical value 1)
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset: next group of 8 rows
  d |= (uint64_t)1 << 46;                  // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                  // 128-byte swizzle
  return d;
}

// Descriptor of an MN-major tile stored as TMA boxes of 64 reduction rows x 64 elements (128 bytes, swizzled):
// inside a box 8 reduction rows form a 1024-byte atom (stride byte offset), the next 64 elements along M/N
// live in the next box, BOX_BYTES further (leading byte offset).
constexpr int BOX_BYTES = 64 * 128;
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)(BOX_BYTES >> 4) << 16;   // leading byte offset: next block of 64 along M/N
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset: next group of 8 reduction rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <typename T>
__device__ __forceinline__ uint32_t instr_desc(bool a_mn, bool b_mn, int m_rows) {
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;  // 0 = f16, 1 = bf16
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(m_rows >> 4) << 24);  // D = f32; 128 rows, or 256 over a CTA pair
}

// Upper tail of the normal distribution and its density factor: q = Q(|x|) = 0.5 erfc(|x| / sqrt 2) and e = exp(-x^2 / 2),
// from one reciprocal, one exp2 and a degree-5 polynomial (Abramowitz & Stegun 7.1.26, absolute error 3e-7 in q: three
// orders below the rounding of a 16-bit output; the tail keeps its relative accuracy because q is formed as a product,
// not as 1 - erf).  All constants are folded: 13 instructions for GELU, 14 for its derivative.  The library erff costs
// about twice that, and at the power cap every FP32 instruction per output element shows in the GEMM's time.
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void normal_tail(float x, float* q, float* e) {
  const float t = rcp_approx(fmaf(0.3275911f * 0.70710678118654752f, fabsf(x), 1.0f));
  float poly = fmaf(0.5f * 1.061405429f, t, 0.5f * -1.453152027f);
  poly = fmaf(poly, t, 0.5f * 1.421413741f);
  poly = fmaf(poly, t, 0.5f * -0.284496736f);
  poly = fmaf(poly, t, 0.5f * 0.254829592f);
  *e = ex2_approx(x * x * (-0.5f * 1.4426950408889634f));
  *q = poly * (t * *e);
}

// Two float32 values in one 64-bit register, for the packed FP32 instructions of this architecture (fma / mul .f32x2:
// one instruction works on both halves).  The polynomial part of the GELU epilogue runs on element pairs with them.
#define LANCET_GELU_PACKED 1
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 splat2(float a) { return pack2(a, a); }

// normal_tail for two values at once: the same operations in the same order per value (bit-identical to the scalar form).
__device__ __forceinline__ void normal_tail2(float x0, float x1, float& q0, float& q1, float& e0, float& e1) {
  const float t0 = rcp_approx(fmaf(0.3275911f * 0.70710678118654752f, fabsf(x0), 1.0f));
  const float t1 = rcp_approx(fmaf(0.3275911f * 0.70710678118654752f, fabsf(x1), 1.0f));
  const f32x2 t = pack2(t0, t1);
  f32x2 poly = fma2(splat2(0.5f * 1.061405429f), t, splat2(0.5f * -1.453152027f));
  poly = fma2(poly, t, splat2(0.5f * 1.421413741f));
  poly = fma2(poly, t, splat2(0.5f * -0.284496736f));
  poly = fma2(poly, t, splat2(0.5f * 0.254829592f));
  const f32x2 x = pack2(x0, x1);
  float a0, a1;
  unpack2(mul2(mul2(x, x), splat2(-0.5f * 1.4426950408889634f)), a0, a1);
  e0 = ex2_approx(a0);
  e1 = ex2_approx(a1);
  unpack2(mul2(poly, mul2(t, pack2(e0, e1))), q0, q1);
}

// Hardware tanh (one special-function instruction, relative error about 2^-11: below the rounding of a 16-bit output).
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int act>
__device__ __forceinline__ float dactivate(float x) {
  if (act == 1) return x > 0.f ? 1.f : 0.f;
  if (act == 2) {   // Phi(x) + x phi(x); Phi(x) = 1 - q for x >= 0, q for x < 0
    float q, e;
    normal_tail(x, &q, &e);
    return fmaf(x * e, 0.3989422804014327f, x >= 0.f ? 1.0f - q : q);
  }
  if (act == 3) {
    const float x2 = x * x;
    const float t = tanh_fast(x * fmaf(0.0356774081f, x2, 0.7978845608028654f));
    return fmaf(0.5f * x * fmaf(-t, t, 1.0f), fmaf(0.1070322243f, x2, 0.7978845608028654f), fmaf(0.5f, t, 0.5f));
  }
  return 1.f;
}

struct Tile {
  int group, mt, nt, rows;  // mt = this CTA's 128-row tile; rows = live rows of the group
};

// Number of 64-row reduction blocks of group g (MODE_REDUCE).
__device__ __forceinline__ int group_row_blocks(const Params& p, int g) {
  int rows = p.C;
  if (p.counts) {
    rows = p.counts[g];
    rows = rows < 0 ? 0 : (rows > p.C ? p.C : rows);
  }
  return (rows + BK - 1) / BK;
}

// Row-parallel forms walk a compacted list of the live tiles only: group g contributes the m-tiles
// [lo[g], lo[g] + nm[g]) of its row window, each times n_tiles column tiles, ordered
// (group, band of p.band m-units, n-tile, m-unit in band) so that a band of A stays in L2 against a sweep of B.
// An m-unit is one 128-row tile, or in the paired form two consecutive ones (the second may lie past the live rows).
struct Sched {
  const int* pref;  // [groups + 1] exclusive prefix of live m-units, by position in the walk
  const int* lo;    // [groups] first live m-tile, by position
  int g;            // position of the previous tile of this walker (tile indices only grow)
};

// The walk visits all groups of one expert before the next expert's (group index = source * LE + expert), so that
// an expert's weights are fetched from DRAM once and stay in L2 while every source's rows are multiplied with them.
__device__ __forceinline__ int group_at(const Params& p, int pos) {
  if (!p.expert_major) return pos;
  const int per = p.groups / p.LE;
  return (pos % per) * p.LE + pos / per;
}

template <int MODE>
__device__ __forceinline__ int live_tiles(const Params& p, const Sched& sc) {
  return MODE == MODE_REDUCE ? p.total_tiles : sc.pref[p.groups] * p.n_tiles;
}

template <int MODE, bool CTA2>
__device__ __forceinline__ Tile decode_tile(const Params& p, Sched& sc, int t, int rank) {
  Tile tl;
  if (MODE == MODE_REDUCE) {
    // tiles_per_group = m_units * n_tiles per expert; `group` holds the expert index
    // the index that runs fastest is the one with fewer tiles, so that the tiles in flight at any time form a
    // block as square as possible in (m, n) and share the most operand slabs through L2
    tl.group = t / p.tiles_per_group;
    const int r = t - tl.group * p.tiles_per_group;
    int mu;
    if (p.n_tiles < p.m_tiles) {
      mu = r / p.n_tiles;
      tl.nt = r - mu * p.n_tiles;
    } else {
      tl.nt = r / p.m_tiles;
      mu = r - tl.nt * p.m_tiles;
    }
    tl.mt = CTA2 ? 2 * mu + rank : mu;
    tl.rows = p.Mout;
    return tl;
  }
  int g = sc.g;
  while (t >= sc.pref[g + 1] * p.n_tiles) ++g;
  sc.g = g;
  tl.group = group_at(p, g);
  int r = t - sc.pref[g] * p.n_tiles;
  const int nm = sc.pref[g + 1] - sc.pref[g];
  const int band_tiles = p.band * p.n_tiles;
  const int band = r / band_tiles;
  r -= band * band_tiles;
  const int m_in_band = min(p.band, nm - band * p.band);
  tl.nt = r / m_in_band;
  const int mu = band * p.band + (r - tl.nt * m_in_band);
  tl.mt = sc.lo[g] + (CTA2 ? 2 * mu + rank : mu);
  int rows = p.C;
  if (p.counts) {
    rows = p.counts[tl.group];
    rows = rows < 0 ? 0 : (rows > p.C ? p.C : rows);
  }
  tl.rows = rows;
  return tl;
}

template <int act>
__device__ __forceinline__ float activate(float v) {
  if (act == 1) return fmaxf(v, 0.f);
  if (act == 2) {   // v Phi(v) = relu(v) - |v| Q(|v|)
    float q, e;
    normal_tail(v, &q, &e);
    return fmaf(-fabsf(v), q, fmaxf(v, 0.f));
  }
  if (act == 3) {   // tanh form: 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3)))
    const float h = 0.5f * v;
    return fmaf(h, tanh_fast(v * fmaf(0.0356774081f, v * v, 0.7978845608028654f)), h);
  }
  return v;
}

// Two outputs at a time: the erf GELU and its derivative share the packed polynomial, everything else is the scalar form.
template <int act>
__device__ __forceinline__ void activate_pair(float v0, float v1, float& o0, float& o1) {
  if (act == 2 && LANCET_GELU_PACKED) {
    float q0, q1, e0, e1;
    normal_tail2(v0, v1, q0, q1, e0, e1);
    o0 = fmaf(-fabsf(v0), q0, fmaxf(v0, 0.f));
    o1 = fmaf(-fabsf(v1), q1, fmaxf(v1, 0.f));
  } else {
    o0 = activate<act>(v0);
    o1 = activate<act>(v1);
  }
}
template <int act>
__device__ __forceinline__ void dactivate_pair(float x0, float x1, float& d0, float& d1) {
  if (act == 2 && LANCET_GELU_PACKED) {
    float q0, q1, e0, e1;
    normal_tail2(x0, x1, q0, q1, e0, e1);
    d0 = fmaf(x0 * e0, 0.3989422804014327f, x0 >= 0.f ? 1.0f - q0 : q0);
    d1 = fmaf(x1 * e1, 0.3989422804014327f, x1 >= 0.f ? 1.0f - q1 : q1);
  } else {
    d0 = dactivate<act>(x0);
    d1 = dactivate<act>(x1);
  }
}

template <int MODE>
__device__ __forceinline__ int tile_k_blocks(const Params& p, const Tile& tl) {
  if (MODE == MODE_ROWS) return (p.K + BK - 1) / BK;
  int n = 0;
  for (int g = tl.group; g < p.groups; g += p.LE) n += group_row_blocks(p, g);
  return n;
}

// ACT is a template parameter: with the activation chosen at run time inside the element loop every element
// became its own chain of basic blocks, the 32 independent chains of a lane could not be interleaved, and the
// GELU epilogue (latency-bound, 1.5 ms against 1.1 ms without it) held the tensor pipe back.
template <typename T, int MODE, bool B_MN, int EPI, int ACT, bool CTA2>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  using C = Cfg<CTA2>;
  constexpr int STAGES = C::STAGES;
  constexpr int B_STAGE_BYTES = C::B_STAGE_BYTES;
  constexpr bool A_MN = (MODE == MODE_REDUCE);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;
  unsigned char* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::SMEM_DATA);
  // barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const uint32_t bar_tfull = smem_u32(bars + 2 * STAGES), bar_tempty = smem_u32(bars + 2 * STAGES + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_pref = reinterpret_cast<int*>(smem + C::SMEM_DATA + 256);
  int* s_lo = s_pref + MAX_GROUPS + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // paired form: rank of this CTA in its pair; the even CTA (leader) issues the MMAs and owns the barriers that
  // gather both CTAs' loads and both CTAs' epilogues
  const int rank = CTA2 ? (int)cluster_ctarank() : 0;
  const int worker = CTA2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_workers = CTA2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  if (MODE == MODE_ROWS && warp == 2) {
    // live m-units of every group and their exclusive prefix (warp scan, 32 groups a round)
    int carry = 0;
    for (int base = 0; base < p.groups; base += 32) {
      const int g = base + lane;            // position in the walk
      int lo = 0, nm = 0;
      if (g < p.groups) {
        const int grp = group_at(p, g);
        int rows = p.C;
        if (p.counts) {
          rows = p.counts[grp];
          rows = rows < 0 ? 0 : (rows > p.C ? p.C : rows);
        }
        if (p.row_lo) {
          lo = p.row_lo[grp];
          lo = (lo < 0 ? 0 : lo) / BM;
        }
        nm = (rows + BM - 1) / BM - lo;
        nm = nm < 0 ? 0 : nm;
        if (CTA2) nm = (nm + 1) >> 1;
      }
      int incl = nm;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
      }
      if (g < p.groups) {
        s_pref[g] = carry + incl - nm;
        s_lo[g] = lo;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_pref[p.groups] = carry;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, CTA2 ? 2 * EPI_WARPS : EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (CTA2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTA2) cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA; in the paired form each CTA loads its own halves) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Sched sc{s_pref, s_lo, 0};
      const int n_live = live_tiles<MODE>(p, sc);
      const int b_col_off = CTA2 ? rank * (BN / 2) : 0;   // this CTA's share of the tile's columns (B operand)
      for (int t = worker; t < n_live && ok; t += n_workers) {
        const Tile tl = decode_tile<MODE, CTA2>(p, sc, t, rank);
        if (MODE == MODE_ROWS) {
          const int e = tl.group % p.LE;
          const int a_row = tl.group * p.C + tl.mt * BM;
          const int k_blocks = (p.K + BK - 1) / BK;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, 1))) break;
            const uint32_t a_dst = smem_u32(sA + stage * A_STAGE_BYTES);
            const uint32_t b_dst = smem_u32(sB + stage * B_STAGE_BYTES);
            if (!CTA2) {
              const uint32_t full = bar_full + 8 * stage;
              mbar_expect_tx(full, C::STAGE_BYTES);
              if (p.interleaved)
                tma_load_3d(a_dst, &tmA, full, kb * BK, tl.group, tl.mt * BM);
              else
                tma_load_2d(a_dst, &tmA, full, kb * BK, a_row);
              if (!B_MN) {
                tma_load_2d(b_dst, &tmB, full, kb * BK, e * p.N + tl.nt * BN);
              } else {
#pragma unroll
                for (int j = 0; j < BN / 64; ++j)
                  tma_load_2d(b_dst + j * BOX_BYTES, &tmB, full, tl.nt * BN + j * 64, e * p.K + kb * BK);
              }
            } else {
              if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * C::STAGE_BYTES);   // both CTAs' bytes
              const uint32_t full = cluster_addr(bar_full + 8 * stage, 0);
              if (p.interleaved)
                tma_load_3d_pair(a_dst, &tmA, full, kb * BK, tl.group, tl.mt * BM);
              else
                tma_load_2d_pair(a_dst, &tmA, full, kb * BK, a_row);
              if (!B_MN) {
                tma_load_2d_pair(b_dst, &tmB, full, kb * BK, e * p.N + tl.nt * BN + b_col_off);
              } else {
#pragma unroll
                for (int j = 0; j < BN / 128; ++j)
                  tma_load_2d_pair(b_dst + j * BOX_BYTES, &tmB, full, tl.nt * BN + b_col_off + j * 64, e * p.K + kb * BK);
              }
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        } else {
          for (int g = tl.group; g < p.groups && ok; g += p.LE) {
            const int nb = group_row_blocks(p, g);
            for (int rb = 0; rb < nb; ++rb) {
              if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, 1))) break;
              const uint32_t a_dst = smem_u32(sA + stage * A_STAGE_BYTES);
              const uint32_t b_dst = smem_u32(sB + stage * B_STAGE_BYTES);
              if (!CTA2) {
                const uint32_t full = bar_full + 8 * stage;
                mbar_expect_tx(full, C::STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < BM / 64; ++j) tma_load_3d(a_dst + j * BOX_BYTES, &tmA, full, tl.mt * BM + j * 64, rb * BK, g);
#pragma unroll
                for (int j = 0; j < BN / 64; ++j) tma_load_3d(b_dst + j * BOX_BYTES, &tmB, full, tl.nt * BN + j * 64, rb * BK, g);
              } else {
                if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * C::STAGE_BYTES);
                const uint32_t full = cluster_addr(bar_full + 8 * stage, 0);
#pragma unroll
                for (int j = 0; j < BM / 64; ++j)
                  tma_load_3d_pair(a_dst + j * BOX_BYTES, &tmA, full, tl.mt * BM + j * 64, rb * BK, g);
#pragma unroll
                for (int j = 0; j < BN / 128; ++j)
                  tma_load_3d_pair(b_dst + j * BOX_BYTES, &tmB, full, tl.nt * BN + b_col_off + j * 64, rb * BK, g);
              }
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (paired form: the even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = instr_desc<T>(A_MN, B_MN, CTA2 ? 2 * BM : BM);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t tphase[2] = {0, 0};
      bool ok = true;
      Sched sc{s_pref, s_lo, 0};
      const int n_live = live_tiles<MODE>(p, sc);
      for (int t = worker; t < n_live && ok; t += n_workers) {
        const Tile tl = decode_tile<MODE, CTA2>(p, sc, t, rank);
        // an empty reduction (weight-gradient form, all counts zero) still hands the accumulator over:
        // the epilogue masks its contents to zero
        const int k_blocks = tile_k_blocks<MODE>(p, tl);
        if (!(ok = mbar_wait(bar_tempty + 8 * buf, tphase[buf] ^ 1, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 elements further inside the 128-byte row; MN-major: 16 reduction rows = two 1024-byte atoms
            const uint64_t adesc = A_MN ? smem_desc_mn_sw128(a_addr + k * 2048) : smem_desc_k_sw128(a_addr + k * UMMA_K * 2);
            const uint64_t bdesc = B_MN ? smem_desc_mn_sw128(b_addr + k * 2048) : smem_desc_k_sw128(b_addr + k * UMMA_K * 2);
            if (CTA2)
              umma_f16_pair(tmem_d, adesc, bdesc, idesc, (kb | k) ? 1u : 0u);
            else
              umma_f16(tmem_d, adesc, bdesc, idesc, (kb | k) ? 1u : 0u);
          }
          // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if (CTA2) umma_commit_pair(bar_empty + 8 * stage); else umma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (CTA2) umma_commit_pair(bar_tfull + 8 * buf); else umma_commit(bar_tfull + 8 * buf);   // accumulator complete
        tphase[buf] ^= 1;
        buf ^= 1;
      }
    }
  } else {
    // ---------------- epilogue: warps 2.., TMEM lane quadrant = warp % 4, column half = (warp - 2) / 4 ----------------
    const int quad = warp & 3;
    const int c_begin = ((warp - 2) >> 2) * (BN / 32 / (EPI_WARPS / 4));
    const int c_end = c_begin + BN / 32 / (EPI_WARPS / 4);
    int buf = 0;
    uint32_t tphase[2] = {0, 0};
    bool ok = true;
    T* D = static_cast<T*>(p.D);
    T* PRE = static_cast<T*>(p.preact);
    const T* bias = static_cast<const T*>(p.bias);
    Sched sc{s_pref, s_lo, 0};
    const int n_live = live_tiles<MODE>(p, sc);
    for (int t = worker; t < n_live && ok; t += n_workers) {
      const Tile tl = decode_tile<MODE, CTA2>(p, sc, t, rank);
      // row-parallel forms always reduce over K >= 1; only the weight-gradient form can meet an empty
      // reduction, whose accumulator holds stale values: they are masked to zero bit-wise (no branch in
      // the hot loop: extra control flow here made the compiler serialise the epilogue)
      const uint32_t acc_mask = (MODE == MODE_ROWS || tile_k_blocks<MODE>(p, tl) > 0) ? 0xffffffffu : 0u;
      ok = mbar_wait(bar_tfull + 8 * buf, tphase[buf], abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row_in_tile = quad * 32 + lane;
      int e;
      size_t out_row;
      bool row_live;
      if (MODE == MODE_ROWS) {
        const int row_in_group = tl.mt * BM + row_in_tile;
        row_live = row_in_group < tl.rows;
        out_row = p.interleaved ? (size_t)row_in_group * p.groups + tl.group : (size_t)tl.group * p.C + row_in_group;
        e = tl.group % p.LE;
      } else {
        const int r = tl.mt * BM + row_in_tile;
        row_live = r < p.Mout;
        out_row = (size_t)tl.group * p.Mout + r;
        e = tl.group;
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
        if (MODE == MODE_REDUCE) {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] &= acc_mask;
        }
        const int col0 = tl.nt * BN + c * 32;
        if (row_live) {
          alignas(16) T o[32];
          if (EPI == EPI_DACT) {
            alignas(16) T pre[32];
            const uint4* pp = reinterpret_cast<const uint4*>(PRE + out_row * p.N + col0);
#pragma unroll
            for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(pre)[q] = pp[q];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float d0, d1;
              dactivate_pair<ACT>(Num<T>::to_f(pre[i]), Num<T>::to_f(pre[i + 1]), d0, d1);
              o[i] = Num<T>::from_f(__uint_as_float(r[i]) * d0);
              o[i + 1] = Num<T>::from_f(__uint_as_float(r[i + 1]) * d1);
            }
          } else {
            alignas(16) T pre[32];
            alignas(16) T bv[32];
#pragma unroll
            for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(bv)[q] = make_uint4(0, 0, 0, 0);
            if (bias) {
              // N is a multiple of 256 and col0 of 32: 16-byte loads as long as the bias base is 16-byte aligned
              const uint4* bp = reinterpret_cast<const uint4*>(bias + (size_t)e * p.N + col0);
#pragma unroll
              for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(bv)[q] = __ldg(bp + q);
            }
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float v0 = __uint_as_float(r[i]) + Num<T>::to_f(bv[i]);
              const float v1 = __uint_as_float(r[i + 1]) + Num<T>::to_f(bv[i + 1]);
              pre[i] = Num<T>::from_f(v0);
              pre[i + 1] = Num<T>::from_f(v1);
              float a0, a1;
              activate_pair<ACT>(v0, v1, a0, a1);
              o[i] = Num<T>::from_f(a0);
              o[i + 1] = Num<T>::from_f(a1);
            }
            if (EPI == EPI_ACT_PRE) {
              uint4* dp = reinterpret_cast<uint4*>(PRE + out_row * p.N + col0);
#pragma unroll
              for (int q = 0; q < 4; q += 2)
                st_global_32B(dp + q, reinterpret_cast<const uint4*>(pre)[q], reinterpret_cast<const uint4*>(pre)[q + 1]);
            }
          }
          uint4* dst = reinterpret_cast<uint4*>(D + out_row * p.N + col0);
#pragma unroll
          for (int q = 0; q < 4; q += 2)
            st_global_32B(dst + q, reinterpret_cast<const uint4*>(o)[q], reinterpret_cast<const uint4*>(o)[q + 1]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        // the MMA issuer (even CTA of a pair) may overwrite this accumulator once both CTAs' epilogues have read it
        if (CTA2) mbar_arrive_cluster(cluster_addr(bar_tempty + 8 * buf, 0)); else mbar_arrive(bar_tempty + 8 * buf);
      }
      tphase[buf] ^= 1;
      buf ^= 1;
    }
  }
  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: let TMA copies that may still be in flight land before the CTA goes away
    const unsigned long long t0 = now_ns();
    while (now_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (CTA2) cluster_sync_all();   // the peer no longer signals this CTA's barriers or reads its shared memory
  if (warp == 1) {
    tc_fence_after();
    if (CTA2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Rows [counts[g], end of the last 128-row tile holding a live row) of every group are set to zero, so that
// a consumer that reduces over rows in blocks of 64 (the weight-gradient form) meets zeros, not stale data.
// A kernel of its own: merged into the epilogue above it slowed the live path down 2.5x.
template <typename T>
__global__ void __launch_bounds__(256)
zero_dead_rows_kernel(T* __restrict__ D, const int32_t* __restrict__ counts, int C, int N, int groups, int interleaved,
                      int to_end) {
  const int g = blockIdx.y;
  int rows = counts[g];
  rows = rows < 0 ? 0 : (rows > C ? C : rows);
  int end = to_end ? C : (rows + BM - 1) / BM * BM;
  if (end > C) end = C;
  const size_t vec_per_row = (size_t)N * sizeof(T) / 16;
  const size_t total = (size_t)(end - rows) * vec_per_row;
  if (!interleaved) {
    uint4* base = reinterpret_cast<uint4*>(D + ((size_t)g * C + rows) * N);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
      base[i] = make_uint4(0, 0, 0, 0);
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const size_t r = rows + i / vec_per_row, v = i % vec_per_row;
      reinterpret_cast<uint4*>(D + (r * groups + g) * N)[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Live rows of every source block from the element counts the count-aware all-to-all returns
// (uint64, entry offset + g * stride, scaled, divided by the row length; src/op/dialect/cublas/matmul.cc:221-247).
__global__ void nelements_to_rows_kernel(const uint64_t* __restrict__ nelem, int offset, int stride, int scale, int M, int C,
                                         int G, int32_t* __restrict__ counts) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= G) return;
  const unsigned long long rows = nelem[(size_t)offset + (size_t)g * stride] * (unsigned long long)scale / (unsigned long long)M;
  counts[g] = rows > (unsigned long long)C ? C : (int)rows;
}

// Bias gradient of an expert layer: db[e][n] = sum over the groups g of expert e and their live rows r of dY[g][r][n].
// Two deterministic stages: partial sums over row slices, then a sum over the slices in fixed order.
// Stage 1: a block owns 256 columns (8 per lane, 16-byte loads) and one row slice; each of its 8 warps walks its rows
// four at a time (four independent 16-byte loads in flight per lane), the warps' sums are added in warp order.
constexpr int kColsumSplits = 32;
constexpr int kColsumCols = 256;
template <typename T>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* __restrict__ dY, const int32_t* __restrict__ counts, int groups, int LE, int C, int N,
                      float* __restrict__ partial) {
  __shared__ float red[8][kColsumCols];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * kColsumCols + lane * 8;
  const int split = blockIdx.y, e = blockIdx.z;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (col < N) {   // N is a multiple of 8 here: a lane's 8 columns are all inside or all outside
    const int stride = kColsumSplits * 8;
    for (int g = e; g < groups; g += LE) {
      int rows = counts ? counts[g] : C;
      rows = rows < 0 ? 0 : (rows > C ? C : rows);
      const T* base = dY + (size_t)g * C * N + col;
      int r = split * 8 + warp;
      for (; r + 3 * stride < rows; r += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcs(reinterpret_cast<const uint4*>(base + (size_t)(r + u * stride) * N));
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const T* h = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += Num<T>::to_f(h[i]);
        }
      }
      for (; r < rows; r += stride) {
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(base + (size_t)r * N));
        const T* h = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += Num<T>::to_f(h[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[warp][lane * 8 + i] = acc[i];
  __syncthreads();
  const int c = blockIdx.x * kColsumCols + threadIdx.x;
  if (c < N) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
    partial[((size_t)e * kColsumSplits + split) * N + c] = t;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, int LE, int N, T* __restrict__ db) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= LE * N) return;
  const int e = i / N, col = i - e * N;
  float acc = 0.f;
  for (int s = 0; s < kColsumSplits; ++s) acc += partial[((size_t)e * kColsumSplits + s) * N + col];
  db[i] = Num<T>::from_f(acc);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows][cols] of 16-bit elements, box = box_rows x 64 columns, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, int dtype) {
  EncodeTiledFn fn = encode_fn();
  LANCET_REQUIRE(fn, LANCET_ERR_CUDA, "grouped gemm: the driver does not provide cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == LANCET_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LANCET_REQUIRE(r == CUDA_SUCCESS, LANCET_ERR_CUDA, "grouped gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LANCET_OK;
}

// 3-D tensor [groups][rows][cols] of 16-bit elements, box = box_groups x box_rows x 64, 128-byte swizzle.
static int make_map3(CUtensorMap* map, const void* base, uint64_t groups, uint64_t rows, uint64_t cols, int dtype,
                     uint32_t box_rows = 64, uint32_t box_groups = 1) {
  EncodeTiledFn fn = encode_fn();
  LANCET_REQUIRE(fn, LANCET_ERR_CUDA, "grouped gemm: the driver does not provide cuTensorMapEncodeTiled");
  cuuint64_t dims[3] = {cols, rows, groups};
  cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
  cuuint32_t box[3] = {(cuuint32_t)BK, box_rows, box_groups};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype == LANCET_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LANCET_REQUIRE(r == CUDA_SUCCESS, LANCET_ERR_CUDA, "grouped gemm: cuTensorMapEncodeTiled (3-D) failed with code %d", (int)r);
  return LANCET_OK;
}

template <typename T, int MODE, bool B_MN, int EPI, int ACT, bool CTA2>
static int launch_f(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, const char* name, cudaStream_t st) {
  constexpr int SMEM_BYTES = Cfg<CTA2>::SMEM_BYTES;
  auto kernel = grouped_gemm_kernel<T, MODE, B_MN, EPI, ACT, CTA2>;
  static bool attr_set = false;
  if (!attr_set) {
    LANCET_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_set = true;
  }
  int grid = sm_count();
  if (gemm_cta_limit() > 0 && gemm_cta_limit() < grid) grid = gemm_cta_limit();
  // total_tiles counts the units one worker takes at a time: a tile, or in the paired form a 256-row pair of tiles
  const long long max_ctas = (long long)p.total_tiles * (CTA2 ? 2 : 1);
  if (grid > max_ctas) grid = (int)max_ctas;
  if (CTA2) grid &= ~1;
  if (grid < (CTA2 ? 2 : 1)) grid = CTA2 ? 2 : 1;
  {
    ProfScope prof(name, st);
    if (CTA2) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)grid);
      cfg.blockDim = dim3(THREADS);
      cfg.dynamicSmemBytes = SMEM_BYTES;
      cfg.stream = st;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, p);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(LANCET_ERR_CUDA, "launch of %s (paired form) failed: %s", name, cudaGetErrorString(e));
      }
    } else {
      kernel<<<grid, THREADS, SMEM_BYTES, st>>>(tmA, tmB, p);
    }
  }
  return launch_status(name);
}

template <typename T, int MODE, bool B_MN, int EPI, int ACT>
static int launch_a(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, const char* name, cudaStream_t st) {
  if (p.paired) return launch_f<T, MODE, B_MN, EPI, ACT, true>(tmA, tmB, p, name, st);
  return launch_f<T, MODE, B_MN, EPI, ACT, false>(tmA, tmB, p, name, st);
}

// Only the combinations that exist are instantiated: the forward form takes any activation, the data-gradient form
// either none (EPI_ACT) or the derivative of one (EPI_DACT), the weight-gradient form none.
template <typename T, int MODE, bool B_MN, int EPI>
static int launch_t(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, const char* name, cudaStream_t st) {
  if constexpr (MODE == MODE_ROWS && (EPI == EPI_DACT || !B_MN)) {
    if (p.act == 1) return launch_a<T, MODE, B_MN, EPI, 1>(tmA, tmB, p, name, st);
    if (p.act == 2) return launch_a<T, MODE, B_MN, EPI, 2>(tmA, tmB, p, name, st);
    if (p.act == 3) return launch_a<T, MODE, B_MN, EPI, 3>(tmA, tmB, p, name, st);
  }
  if constexpr (EPI == EPI_DACT)
    return fail(LANCET_ERR_INVALID, "%s: an activation derivative needs an activation", name);
  else
    return launch_a<T, MODE, B_MN, EPI, 0>(tmA, tmB, p, name, st);
}

template <int MODE, bool B_MN, int EPI>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, int dtype, const char* name, cudaStream_t st) {
  int rc = dtype == LANCET_BF16 ? launch_t<__nv_bfloat16, MODE, B_MN, EPI>(tmA, tmB, p, name, st)
                                : launch_t<__half, MODE, B_MN, EPI>(tmA, tmB, p, name, st);
  if (rc != LANCET_OK || MODE != MODE_ROWS || !p.counts) return rc;
  // both 16-bit types have the same size: one instantiation serves them
  zero_dead_rows_kernel<__half><<<dim3(8, p.groups), 256, 0, st>>>(static_cast<__half*>(p.D), p.counts, p.C, p.N, p.groups,
                                                                    p.interleaved, 0);
  return launch_status("zero_dead_rows_kernel");
}

// Shared argument checks and tile bookkeeping of the row-parallel forms (NT, NN).
static int rows_common(const char* fn, const void* A, const void* B, void* D, int groups, int LE, int C, int N, int K,
                       int act, int dtype, int32_t* status, Params* p) {
  LANCET_REQUIRE(dtype == LANCET_BF16 || dtype == LANCET_F16, LANCET_ERR_UNSUPPORTED,
                 "%s: inputs must be bfloat16 or float16 (dtype code %d)", fn, dtype);
  LANCET_REQUIRE(groups >= 1 && LE >= 1 && groups % LE == 0 && C >= 0 && N >= 1 && K >= 1, LANCET_ERR_INVALID,
                 "%s: bad sizes groups=%d LE=%d C=%d N=%d K=%d", fn, groups, LE, C, N, K);
  LANCET_REQUIRE(groups <= MAX_GROUPS, LANCET_ERR_INVALID, "%s: at most %d groups (got %d)", fn, MAX_GROUPS, groups);
  LANCET_REQUIRE(N % BN == 0 && K % 8 == 0, LANCET_ERR_INVALID, "%s: N=%d must be a multiple of %d and K=%d a multiple of 8",
                 fn, N, BN, K);
  LANCET_REQUIRE(act >= 0 && act <= 3, LANCET_ERR_INVALID, "%s: unknown activation %d", fn, act);
  if (C == 0) return LANCET_OK;
  LANCET_REQUIRE(A && B && D && status, LANCET_ERR_NULL, "%s: null pointer argument", fn);
  LANCET_REQUIRE(aligned(A, 16) && aligned(B, 16) && aligned(D, 32), LANCET_ERR_INVALID,
                 "%s: inputs must be 16-byte aligned, the output 32-byte aligned", fn);
  LANCET_REQUIRE((long long)groups * C < (1ll << 31) && (long long)LE * N < (1ll << 31) && (long long)LE * K < (1ll << 31),
                 LANCET_ERR_INVALID, "%s: row counts exceed 2^31", fn);
  p->groups = groups; p->LE = LE; p->C = C; p->N = N; p->K = K; p->Mout = 0;
  p->paired = gemm_paired_enabled() ? 1 : 0;
  p->expert_major = gemm_option(1) ? 0 : 1;
  p->m_tiles = (C + BM - 1) / BM;
  if (p->paired) p->m_tiles = (p->m_tiles + 1) / 2;
  p->n_tiles = N / BN;
  p->tiles_per_group = p->m_tiles * p->n_tiles;
  const long long total = (long long)p->tiles_per_group * groups;
  LANCET_REQUIRE(total < (1ll << 31), LANCET_ERR_INVALID, "%s: too many tiles", fn);
  p->total_tiles = (int)total;
  p->status = status;
  p->act = act;
  p->row_lo = nullptr;
  p->interleaved = 0;
  // A band of m-units is swept against all column tiles of an expert: the band's rows of A (band x rows x K) and the
  // expert's B (N x K) should stay in L2 together.  About 20 MB for the band keeps both resident beside the outputs.
  {
    const long long unit_bytes = (long long)(p->paired ? 2 * BM : BM) * K * 2;
    long long band = (20ll << 20) / (unit_bytes > 0 ? unit_bytes : 1);
    p->band = (int)(band < 2 ? 2 : (band > MAX_BAND ? MAX_BAND : band));
  }
  return LANCET_OK;
}

}  // namespace gemm
}  // namespace lancet

extern "C" {
using namespace lancet;

int lancet_grouped_gemm_nt_window(const void* A, const void* B, void* D, const void* bias, void* preact, int groups, int LE,
                                  int C, int N, int K, const int32_t* row_begin, const int32_t* row_end, int act, int dtype,
                                  int32_t* status, lancet_stream_t stream) {
  using namespace lancet::gemm;
  Params p;
  if (int rc = rows_common("lancet_grouped_gemm_nt", A, B, D, groups, LE, C, N, K, act, dtype, status, &p)) return rc;
  if (C == 0) return LANCET_OK;
  LANCET_REQUIRE(aligned(bias, 16) && aligned(preact, 32), LANCET_ERR_INVALID,
                 "lancet_grouped_gemm_nt: bias must be 16-byte aligned, preact 32-byte aligned");
  p.counts = row_end; p.row_lo = row_begin; p.bias = bias; p.D = D; p.preact = preact; p.epi = EPI_ACT;
  CUtensorMap tmA, tmB;
  if (int rc = make_map(&tmA, A, (uint64_t)groups * C, (uint64_t)K, BM, dtype)) return rc;
  if (int rc = make_map(&tmB, B, (uint64_t)LE * N, (uint64_t)K, p.paired ? BN / 2 : BN, dtype)) return rc;
  if (preact)
    return launch<MODE_ROWS, false, EPI_ACT_PRE>(tmA, tmB, p, dtype, "grouped_gemm_nt_kernel", static_cast<cudaStream_t>(stream));
  return launch<MODE_ROWS, false, EPI_ACT>(tmA, tmB, p, dtype, "grouped_gemm_nt_kernel", static_cast<cudaStream_t>(stream));
}

int lancet_grouped_gemm_nt(const void* A, const void* B, void* D, const void* bias, void* preact, int groups, int LE,
                           int C, int N, int K, const int32_t* counts, int act, int dtype, int32_t* status,
                           lancet_stream_t stream) {
  return lancet_grouped_gemm_nt_window(A, B, D, bias, preact, groups, LE, C, N, K, nullptr, counts, act, dtype, status, stream);
}

int lancet_grouped_gemm_nn(const void* A, const void* B, void* D, const void* preact, int groups, int LE, int C, int N,
                           int K, const int32_t* counts, int act, int dtype, int32_t* status, lancet_stream_t stream) {
  return lancet_grouped_gemm_nn_window(A, B, D, preact, groups, LE, C, N, K, nullptr, counts, act, dtype, status, stream);
}

int lancet_grouped_gemm_nn_window(const void* A, const void* B, void* D, const void* preact, int groups, int LE, int C, int N,
                                  int K, const int32_t* row_begin, const int32_t* counts, int act, int dtype, int32_t* status,
                                  lancet_stream_t stream) {
  using namespace lancet::gemm;
  Params p;
  if (int rc = rows_common("lancet_grouped_gemm_nn", A, B, D, groups, LE, C, N, K, act, dtype, status, &p)) return rc;
  if (C == 0) return LANCET_OK;
  LANCET_REQUIRE(K % BK == 0, LANCET_ERR_INVALID, "lancet_grouped_gemm_nn: K=%d must be a multiple of %d", K, BK);
  LANCET_REQUIRE(act == 0 || preact, LANCET_ERR_NULL, "lancet_grouped_gemm_nn: an activation derivative needs the saved pre-activation");
  LANCET_REQUIRE(aligned(preact, 16), LANCET_ERR_INVALID, "lancet_grouped_gemm_nn: preact must be 16-byte aligned");
  p.counts = counts; p.row_lo = row_begin; p.bias = nullptr; p.D = D; p.preact = const_cast<void*>(preact);
  p.epi = (act != 0) ? EPI_DACT : EPI_ACT;
  if (act == 0) p.preact = nullptr;
  CUtensorMap tmA, tmB;
  if (int rc = make_map(&tmA, A, (uint64_t)groups * C, (uint64_t)K, BM, dtype)) return rc;
  if (int rc = make_map(&tmB, B, (uint64_t)LE * K, (uint64_t)N, 64, dtype)) return rc;
  if (p.epi == EPI_DACT)
    return launch<MODE_ROWS, true, EPI_DACT>(tmA, tmB, p, dtype, "grouped_gemm_nn_kernel", static_cast<cudaStream_t>(stream));
  return launch<MODE_ROWS, true, EPI_ACT>(tmA, tmB, p, dtype, "grouped_gemm_nn_kernel", static_cast<cudaStream_t>(stream));
}

int lancet_grouped_gemm_tn(const void* A, const void* B, void* D, int groups, int LE, int C, int Mout, int N,
                           const int32_t* counts, int dtype, int32_t* status, lancet_stream_t stream) {
  using namespace lancet::gemm;
  LANCET_REQUIRE(dtype == LANCET_BF16 || dtype == LANCET_F16, LANCET_ERR_UNSUPPORTED,
                 "lancet_grouped_gemm_tn: inputs must be bfloat16 or float16 (dtype code %d)", dtype);
  LANCET_REQUIRE(groups >= 1 && LE >= 1 && groups % LE == 0 && C >= 0 && Mout >= 1 && N >= 1, LANCET_ERR_INVALID,
                 "lancet_grouped_gemm_tn: bad sizes groups=%d LE=%d C=%d Mout=%d N=%d", groups, LE, C, Mout, N);
  LANCET_REQUIRE(Mout % BM == 0 && N % BN == 0, LANCET_ERR_INVALID,
                 "lancet_grouped_gemm_tn: Mout=%d must be a multiple of %d and N=%d of %d", Mout, BM, N, BN);
  LANCET_REQUIRE(D && status && (C == 0 || (A && B)), LANCET_ERR_NULL, "lancet_grouped_gemm_tn: null pointer argument");
  LANCET_REQUIRE(aligned(A, 16) && aligned(B, 16) && aligned(D, 32), LANCET_ERR_INVALID,
                 "lancet_grouped_gemm_tn: inputs must be 16-byte aligned, the output 32-byte aligned");
  LANCET_REQUIRE((long long)groups * C < (1ll << 31) && (long long)LE * Mout < (1ll << 31), LANCET_ERR_INVALID,
                 "lancet_grouped_gemm_tn: row counts exceed 2^31");
  Params p;
  p.groups = groups; p.LE = LE; p.C = C; p.N = N; p.K = 0; p.Mout = Mout;
  p.paired = (gemm_paired_enabled() && Mout % (2 * BM) == 0) ? 1 : 0;
  p.m_tiles = Mout / (p.paired ? 2 * BM : BM); p.n_tiles = N / BN;
  p.tiles_per_group = p.m_tiles * p.n_tiles;
  p.total_tiles = p.tiles_per_group * LE;
  p.band = 1;
  p.expert_major = 0;
  p.counts = counts; p.row_lo = nullptr; p.interleaved = 0; p.bias = nullptr; p.D = D; p.preact = nullptr; p.act = 0;
  p.epi = EPI_ACT;
  p.status = status;
  CUtensorMap tmA, tmB;
  if (C == 0) {
    LANCET_CUDA(cudaMemsetAsync(D, 0, (size_t)LE * Mout * N * 2, static_cast<cudaStream_t>(stream)));
    return LANCET_OK;
  }
  if (int rc = make_map3(&tmA, A, (uint64_t)groups, (uint64_t)C, (uint64_t)Mout, dtype)) return rc;
  if (int rc = make_map3(&tmB, B, (uint64_t)groups, (uint64_t)C, (uint64_t)N, dtype)) return rc;
  return launch<MODE_REDUCE, true, EPI_ACT>(tmA, tmB, p, dtype, "grouped_gemm_tn_kernel", static_cast<cudaStream_t>(stream));
}

size_t lancet_sparse_expert_matmul_nt_workspace_bytes(int G) {
  if (G < 1) return 0;
  return ((size_t)G * sizeof(int32_t) + 255) / 256 * 256 + 256;
}

int lancet_sparse_expert_matmul_nt(const void* data, const void* weight, void* out, const uint64_t* nelements_per_gpu,
                                   int nelements_offset, int nelements_stride, int nelements_scale, int C, int G, int M, int N,
                                   int dtype, void* ws, size_t ws_bytes, lancet_stream_t stream) {
  using namespace lancet::gemm;
  LANCET_REQUIRE(nelements_offset >= 0 && nelements_stride >= 1 && nelements_scale >= 1, LANCET_ERR_INVALID,
                 "lancet_sparse_expert_matmul_nt: bad nelements offset %d / stride %d / scale %d", nelements_offset,
                 nelements_stride, nelements_scale);
  LANCET_REQUIRE(G >= 1 && ws && ws_bytes >= lancet_sparse_expert_matmul_nt_workspace_bytes(G) && aligned(ws, 16),
                 LANCET_ERR_INVALID, "lancet_sparse_expert_matmul_nt: workspace missing, too small or unaligned");
  int32_t* counts = static_cast<int32_t*>(ws);
  int32_t* status = reinterpret_cast<int32_t*>(static_cast<char*>(ws) + lancet_sparse_expert_matmul_nt_workspace_bytes(G) - 256);
  Params p;
  if (int rc = rows_common("lancet_sparse_expert_matmul_nt", data, weight, out, G, 1, C, N, M, 0, dtype, status, &p)) return rc;
  if (C == 0) return LANCET_OK;
  LANCET_REQUIRE(nelements_per_gpu, LANCET_ERR_NULL, "lancet_sparse_expert_matmul_nt: null nelements_per_gpu");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LANCET_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
  nelements_to_rows_kernel<<<(G + 127) / 128, 128, 0, st>>>(nelements_per_gpu, nelements_offset, nelements_stride,
                                                          nelements_scale, M, C, G, counts);
  if (int rc = launch_status("nelements_to_rows_kernel")) return rc;
  p.counts = counts; p.interleaved = 1; p.bias = nullptr; p.D = out; p.preact = nullptr; p.epi = EPI_ACT;
  CUtensorMap tmA, tmB;
  // data [C][G][M]: dimension order (M, G, C), one group and 128 rows of it per box
  if (int rc = make_map3(&tmA, data, (uint64_t)C, (uint64_t)G, (uint64_t)M, dtype, 1, BM)) return rc;
  if (int rc = make_map(&tmB, weight, (uint64_t)N, (uint64_t)M, p.paired ? BN / 2 : BN, dtype)) return rc;
  const int rc = dtype == LANCET_BF16
                     ? launch_t<__nv_bfloat16, MODE_ROWS, false, EPI_ACT>(tmA, tmB, p, "sparse_expert_matmul_nt_kernel", st)
                     : launch_t<__half, MODE_ROWS, false, EPI_ACT>(tmA, tmB, p, "sparse_expert_matmul_nt_kernel", st);
  if (rc != LANCET_OK) return rc;
  // every row past the count is zero in the output (the reference's intended path memsets it, matmul.cc:289)
  zero_dead_rows_kernel<__half><<<dim3(8, G), 256, 0, st>>>(static_cast<__half*>(out), counts, C, N, G, 1, 1);
  return launch_status("zero_dead_rows_kernel");
}

size_t lancet_grouped_bias_grad_workspace_bytes(int LE, int N) {
  if (LE < 1 || N < 1) return 0;
  return (size_t)LE * lancet::gemm::kColsumSplits * N * sizeof(float);
}

int lancet_grouped_bias_grad(const void* dY, void* db, int groups, int LE, int C, int N, const int32_t* counts, int dtype,
                             void* ws, size_t ws_bytes, lancet_stream_t stream) {
  using namespace lancet::gemm;
  LANCET_REQUIRE(dtype == LANCET_BF16 || dtype == LANCET_F16, LANCET_ERR_UNSUPPORTED,
                 "lancet_grouped_bias_grad: inputs must be bfloat16 or float16 (dtype code %d)", dtype);
  LANCET_REQUIRE(groups >= 1 && LE >= 1 && groups % LE == 0 && C >= 0 && N >= 1, LANCET_ERR_INVALID,
                 "lancet_grouped_bias_grad: bad sizes groups=%d LE=%d C=%d N=%d", groups, LE, C, N);
  LANCET_REQUIRE(dY && db && ws, LANCET_ERR_NULL, "lancet_grouped_bias_grad: null pointer argument");
  LANCET_REQUIRE(ws_bytes >= lancet_grouped_bias_grad_workspace_bytes(LE, N), LANCET_ERR_INVALID,
                 "lancet_grouped_bias_grad: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(ws);
  LANCET_REQUIRE(N % 8 == 0 && aligned(dY, 16), LANCET_ERR_INVALID,
                 "lancet_grouped_bias_grad: N=%d must be a multiple of 8 and dY 16-byte aligned", N);
  const dim3 grid1((N + kColsumCols - 1) / kColsumCols, kColsumSplits, LE);
  const int grid2 = (LE * N + 255) / 256;
  if (dtype == LANCET_BF16) {
    colsum_partial_kernel<__nv_bfloat16><<<grid1, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dY), counts, groups, LE, C, N, partial);
    if (int rc = launch_status("colsum_partial_kernel")) return rc;
    colsum_final_kernel<__nv_bfloat16><<<grid2, 256, 0, st>>>(partial, LE, N, static_cast<__nv_bfloat16*>(db));
  } else {
    colsum_partial_kernel<__half><<<grid1, 256, 0, st>>>(static_cast<const __half*>(dY), counts, groups, LE, C, N, partial);
    if (int rc = launch_status("colsum_partial_kernel")) return rc;
    colsum_final_kernel<__half><<<grid2, 256, 0, st>>>(partial, LE, N, static_cast<__half*>(db));
  }
  return launch_status("colsum_final_kernel");
}
}
