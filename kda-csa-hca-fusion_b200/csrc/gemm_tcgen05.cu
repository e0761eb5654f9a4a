// bf16 linear layer on the 5th-generation tensor cores (sm_100a):
//   C[M,N] = A[M,K] . W[N,K]^T, fp32 accumulation in tensor memory, one rounding to bf16,
//   optional residual add.  Every dense projection of the hybrid layer goes through here
//   (q/k/v/g/beta, the fused CSA 6-way KV/indexer projection, W_DQ/W_UQ/W_IUQ, o_proj).
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0      : TMA producer — cp.async.bulk.tensor tiles of A (128x64) and W (BNx64), 128-byte
//                 swizzle, into a 4..10-stage shared-memory ring (no multicast: every CTA fetches its own).
//   warp 1      : allocates tensor memory, then one elected lane issues tcgen05.mma (M=128, N=BN,
//                 K=16 per instruction, four per stage) and tcgen05.commit to release stages.
//   warps 2..9  : epilogue — tcgen05.ld of the fp32 accumulator (each warp its 32-lane quarter and one
//                 half of the tile's columns), bf16 rounding, optional activations / residual, a 32x32 transpose
//                 through shared memory and stores of whole 64-byte row segments.
// Two accumulator buffers in tensor memory let the epilogue of tile i overlap the main loop of
// tile i+1.  Every wait on an mbarrier is bounded; on expiry the kernel records a status word,
// leaves its loops, frees tensor memory and returns.
//
// Large products (M >= 512, N > 128) run on CTA pairs: clusters of two CTAs share a 256 x 256 tile through
// tcgen05.mma.cta_group::2 (M = 256).  Each CTA loads its own 128 rows of A and half of the W tile
// (cp.async.bulk.tensor.cta_group::2, bytes counted on the even CTA's barrier), the even CTA's MMA lane issues
// one instruction for both and commits to the barriers of both CTAs (two unicast commits), each CTA's epilogue
// warps drain their own 128 x 256 accumulator.  A CTA then moves 32 KB per k-block instead of 48 KB and the
// ring holds six stages; measured 1.26-1.31 PFLOP/s against 1.20-1.22 with one CTA per tile at M = 131072.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>

#include "kch_common.cuh"

#define TG_BM 128
#define TG_BK 64
#define TG_THREADS 320
#define TG_EPI_LD 80
#define TG_SPIN_LIMIT (1u << 24)

__device__ unsigned int g_kch_status = 0;  // nonzero: a bounded wait expired (see kch_device_status)

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// bounded wait; returns false (and records `code`) if the phase never completes within `limit` polls
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned code, uint32_t limit = TG_SPIN_LIMIT) {
  uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    // someone else already gave up?  Looked at rarely: a global load after every failed try would sit on the
    // critical path of each wake-up
    if ((it & 1023) == 1023 && *((volatile unsigned int*)&g_kch_status) != 0) return false;
  }
  atomicCAS(&g_kch_status, 0u, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- CTA-pair (cta_group::2) forms: two CTAs of a cluster work on one 256-row tile, the even CTA issues the MMAs
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  // relaxed: the arrival orders nothing but itself (tensor-memory reads are ordered by tcgen05.fence); a release at
  // cluster scope would wait for every global store of the tile
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile into this CTA's shared memory, bytes counted on a barrier that may live in the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// K-major operand tile, rows of 64 bf16 (128 bytes) under the 128-byte swizzle: 8-row groups are
// 1024 bytes apart (stride byte offset); the leading byte offset is not used for this layout.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // descriptor version for sm_100
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

// Column-segment activations applied in the epilogue (the rounding points of the unfused chain are kept:
// the product is rounded to bf16 first, every further step reads bf16, computes in fp32, rounds to bf16).
struct TgEpilogue {
  int nseg;            // 0: plain store
  int seg_end[8];      // exclusive end column of segment s (ascending)
  int seg_act[8];      // 0 none, KCH_ACT_*
  float seg_param[8];
};

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// Fast intrinsics (ex2.approx, approximate reciprocal): a few fp32 ulp, far below the bf16 rounding
// that follows every step, so a fused result differs from the unfused chain by at most one bf16 rounding.
__device__ __forceinline__ float ep_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
// Ring depth: as many (A tile + W tile) stages as fit in about 200 KB, so that narrow tiles (small BN) keep
// the same number of bytes in flight per SM as the 256-wide tile does with 4 stages.
// row pitch (in floats) of the fp32 partial tile a split-K CTA leaves in shared memory: 16 bytes of padding keep the
// row-per-lane float4 stores free of bank conflicts
#define TG_RED_LD(BN) ((BN) + 4)
template <int BN>
struct TgStages { static constexpr int value = BN >= 256 ? 4 : BN >= 128 ? 6 : BN >= 64 ? 8 : 10; };

// SK ("skinny", a decode batch of at most 64 rows): the A box is 64 rows and the ring is sized to about 96 KB, so two
// CTAs share an SM -- the launch is a stream of weights and wants many CTAs with bytes in flight, not a deep ring in
// few.  The MMA still spans 128 rows: rows 64..127 of its A operand are whatever follows in shared memory (the next A
// stage, or the first W stage behind the last one), which only reaches accumulator rows that are never stored.
// With `ksplit` > 1 the K loop of a tile is divided over the CTAs of a cluster (see the kernel).
template <int BN, bool TWO = false, bool SK = false>
struct TgSmem {
  // a CTA of a pair holds half of the W tile, which buys two more stages
  static constexpr int A_ROWS = SK ? 64 : TG_BM;
  static constexpr int STAGES = TWO ? 6 : SK ? (BN >= 128 ? 4 : BN >= 64 ? 6 : 8) : TgStages<BN>::value;
  static constexpr int B_ROWS = TWO ? BN / 2 : BN;
  static constexpr int EPI_WARPS = BN == 256 ? 8 : 4;   // narrower tiles are stored by warps 2..5 alone
  alignas(1024) bf16 a[STAGES][A_ROWS * TG_BK];
  alignas(1024) bf16 b[STAGES][B_ROWS * TG_BK];
  alignas(16) uint8_t epi[EPI_WARPS][32 * TG_EPI_LD];   // per epilogue warp: a 32 x 32 bf16 chunk, rows padded to 80 bytes
  alignas(8) uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
};

template <int BN, bool TWO, bool SK = false>
__global__ void __launch_bounds__(TG_THREADS, SK ? 2 : 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    bf16* __restrict__ C, const bf16* __restrict__ R, int64_t M, int N, int K,
                    int64_t ldc, int64_t ldr, int vec_ok, const TgEpilogue ep, int slab_k, int64_t slab_rows,
                    int ksplit) {
  // ksplit > 1 (SK only; launched as clusters of `ksplit` CTAs, one tile per cluster): CTA r of the cluster runs
  // k-blocks [r * kper, (r + 1) * kper) into its own tensor memory, leaves the fp32 partial tile in its shared
  // memory, and after a cluster barrier finishes rows [r * 64 / ksplit, ...) of the tile: partials are summed in
  // rank order through distributed shared memory (so the result does not depend on which CTA adds them), then the
  // same activation / residual / rounding steps as the single-CTA epilogue.
  // slab_k > 0: the K columns of A lie in K / slab_k slabs of [slab_rows][slab_k] one after the other (the
  // rank-major buffer an all-gather of per-GPU column slices leaves behind); map_a then describes all slabs as one
  // [slabs * slab_rows][slab_k] matrix and k-block kb is read from slab kb * 64 / slab_k
  extern __shared__ uint8_t smem_raw[];
  TgSmem<BN, TWO, SK>& sm = *reinterpret_cast<TgSmem<BN, TWO, SK>*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int TG_STAGES = TgSmem<BN, TWO, SK>::STAGES;
  constexpr int A_ROWS = TgSmem<BN, TWO, SK>::A_ROWS;
  constexpr int BM_T = TWO ? 2 * TG_BM : TG_BM;       // rows of a tile: a CTA pair takes 256, each CTA its 128
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = TWO ? cluster_ctarank() : 0u;
  const bool split = SK && ksplit > 1;
  const uint32_t ks = split ? cluster_ctarank() : 0u;
  const int64_t unit = TWO ? (blockIdx.x >> 1) : split ? (blockIdx.x / ksplit) : blockIdx.x;
  const int64_t nunits = TWO ? (gridDim.x >> 1) : split ? (gridDim.x / ksplit) : gridDim.x;
  const int n_tiles = (N + BN - 1) / BN;
  const int64_t m_tiles = (M + BM_T - 1) / BM_T;
  const int64_t total_tiles = m_tiles * n_tiles;
  const int kblocks_all = (K + TG_BK - 1) / TG_BK;
  const int kper = split ? (kblocks_all + ksplit - 1) / ksplit : kblocks_all;
  const int kb_first = (int)ks * kper;
  const int kblocks = min(kblocks_all - kb_first, kper);     // this CTA's share (the host keeps every share non-empty)
  constexpr uint32_t ACC_COLS = BN;                 // fp32 accumulator columns per buffer
  constexpr uint32_t TMEM_COLS = (2 * ACC_COLS) < 32 ? 32 : 2 * ACC_COLS;  // power of two >= 32

  if (threadIdx.x == 0) {
    // pair: the even CTA's `full` counts the bytes of both producers, its `acc_empty` the epilogue warps of both CTAs
    for (int s = 0; s < TG_STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], TWO ? 16 : 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (TWO) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (TWO) cluster_sync_all();     // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = unit; tile < total_tiles && ok; tile += nunits) {
        const int64_t mb = tile / n_tiles;
        const int nb = (int)(tile % n_tiles);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % TG_STAGES, ph = (it / TG_STAGES) & 1;
          if (!mbar_wait(&sm.empty[s], ph ^ 1, 1)) { ok = false; break; }
          const int kcw = (kb_first + kb) * TG_BK;     // column of W; of A unless A lies in slabs
          int kc = kcw;
          int64_t roff = 0;
          if (slab_k > 0) { const int sidx = kc / slab_k; kc -= sidx * slab_k; roff = (int64_t)sidx * slab_rows; }
          if constexpr (TWO) {
            // this CTA's 128 rows of A and its half of the W tile; the bytes count on the even CTA's barrier, which
            // that CTA's producer arms for both (the odd CTA's bytes may land first: the count is signed)
            const uint32_t full_addr = mapa_u32(smem_u32(&sm.full[s]), 0);
            if (rank == 0) mbar_expect_tx(&sm.full[s], 2 * (TG_BM + BN / 2) * TG_BK * 2);
            tma_load_2d_pair(sm.a[s], &map_a, kc, (int)(mb * BM_T + rank * TG_BM + roff), full_addr);
            tma_load_2d_pair(sm.b[s], &map_w, kcw, nb * BN + (int)rank * (BN / 2), full_addr);
          } else {
            mbar_expect_tx(&sm.full[s], (A_ROWS + BN) * TG_BK * 2);
            tma_load_2d(sm.a[s], &map_a, kc, (int)(mb * TG_BM + roff), &sm.full[s]);
            tma_load_2d(sm.b[s], &map_w, kcw, nb * BN, &sm.full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM_T >> 4) << 24);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int64_t tile = unit; tile < total_tiles && ok; tile += nunits, ++tcount) {
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        if (!mbar_wait(&sm.acc_empty[acc], aph ^ 1, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % TG_STAGES, ph = (it / TG_STAGES) & 1;
          if (!mbar_wait(&sm.full[s], ph, 3)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_u32(sm.a[s]));
          const uint64_t bdesc = make_smem_desc(smem_u32(sm.b[s]));
          if constexpr (TWO) {
            // one instruction covers both CTAs: A rows and W-tile halves are read from both shared memories
            // at these offsets, each CTA's 128 x BN result lands in its own tensor memory
#pragma unroll
            for (int k = 0; k < TG_BK / 16; ++k)
              tc_mma_bf16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
            tc_commit_pair(smem_u32(&sm.empty[s]));
            tc_commit_pair(mapa_u32(smem_u32(&sm.empty[s]), 1));
          } else {
#pragma unroll
            for (int k = 0; k < TG_BK / 16; ++k)
              tc_mma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
            tc_commit(&sm.empty[s]);  // stage reusable once these MMAs have read it
          }
        }
        if (ok) {
          if constexpr (TWO) {
            tc_commit_pair(smem_u32(&sm.acc_full[acc]));
            tc_commit_pair(mapa_u32(smem_u32(&sm.acc_full[acc]), 1));
          } else {
            tc_commit(&sm.acc_full[acc]);
          }
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    // 8 warps: warps 2..5 take the first half of a 256-column tile, warps 6..9 the second half (narrower
    // tiles are handled by warps 2..5 alone); each warp reads its own 32-lane quarter of tensor memory
    const int quarter = warp & 3;  // tensor-memory lanes 32*quarter .. 32*quarter+31
    const int half = (warp - 2) >> 2;
    const int c_begin = (BN == 256) ? half * 128 : 0;
    const int c_end = (BN == 256) ? c_begin + 128 : (half == 0 ? BN : 0);
    uint32_t tcount = 0;
    bool ok = true;
    if (split) {
      // this CTA's partial sums of rows 0..63, as fp32, to shared memory (the ring is drained: every MMA has retired)
      if (quarter < 2 && unit < total_tiles && mbar_wait(&sm.acc_full[0], 0, 4)) {
        tc_fence_after();
        float* red = reinterpret_cast<float*>(&sm.a[0][0]) + (size_t)(quarter * 32 + lane) * TG_RED_LD(BN);
        const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tc_ld32(tbase + c0, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(red + c0 + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
      }
      ok = false;      // the tile is finished after the cluster barrier below
    }
    for (int64_t tile = unit; tile < total_tiles && ok; tile += nunits, ++tcount) {
      const int64_t mb = tile / n_tiles;
      const int nb = (int)(tile % n_tiles);
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      if (!mbar_wait(&sm.acc_full[acc], aph, 4)) { ok = false; break; }
      tc_fence_after();
      const int64_t row = mb * BM_T + rank * TG_BM + quarter * 32 + lane;
      const uint32_t tbase = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      float nrm = 1.f;
      // the accumulator chunk after the current one is already on its way from tensor memory
      uint32_t rn[32];
      if (c_begin < c_end) tc_ld32(tbase + c_begin, rn);
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        uint32_t r[32];
        const int col = nb * BN + c0;
        int act = 0;
        float prm = 0.f;
        if (ep.nseg) {
          int sidx = 0;
          while (sidx < ep.nseg - 1 && col >= ep.seg_end[sidx]) ++sidx;
          act = ep.seg_act[sidx];
          prm = ep.seg_param[sidx];
          if (act == KCH_ACT_SILU_L2NORM && (c0 & 127) == 0) {
            // norm of this row's 128-column head: a thread owns a whole accumulator row, no exchange needed
            float ss = 0.f;
            for (int qd = 0; qd < 4; ++qd) {
              tc_ld32(tbase + c0 + 32 * qd, r);
              tc_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float sv = bf16r(ep_silu(bf16r(__uint_as_float(r[j]))));
                ss = fmaf(sv, sv, ss);
              }
            }
            nrm = __fdividef(1.0f, fmaxf(bf16r(sqrtf(ss)), 1e-12f));
          }
        }
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = rn[j];
        if (c0 + 32 < c_end) tc_ld32(tbase + c0 + 32, rn);
        // the activation is uniform over the chunk: branch once, then 32 independent element pipelines
        if (act == KCH_ACT_SILU_L2NORM) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(bf16r(ep_silu(bf16r(__uint_as_float(r[j])))) * nrm);
        } else if (act == KCH_ACT_SILU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(ep_silu(bf16r(__uint_as_float(r[j]))));
        } else if (act == KCH_ACT_SIGMOID) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            r[j] = __float_as_uint(__fdividef(1.0f, 1.0f + __expf(-bf16r(__uint_as_float(r[j])))));
        } else if (act == KCH_ACT_NEG_SOFTPLUS) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = bf16r(__uint_as_float(r[j]));
            r[j] = __float_as_uint(-bf16r(v > 20.f ? v : __logf(1.0f + __expf(v))) * prm);
          }
        }
        if (vec_ok && col + 32 <= N) {
          // Transpose the 32 x 32 chunk through shared memory so that a store instruction writes 8 row segments
          // of 64 contiguous bytes (full 32-byte sectors) instead of 16 bytes in each of 32 rows.
          uint8_t* stg = sm.epi[warp - 2];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2 * j]), __uint_as_float(r[8 * v + 2 * j + 1]));
              o[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(stg + lane * TG_EPI_LD + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
          }
          __syncwarp();
          const int64_t row0 = mb * BM_T + rank * TG_BM + quarter * 32;
          const int piece = lane & 3;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int rr = (lane >> 2) + 8 * j;
            const int64_t grow = row0 + rr;
            uint4 cv = *reinterpret_cast<const uint4*>(stg + rr * TG_EPI_LD + piece * 16);
            if (grow < M) {
              if (R) {
                const uint4 resv = *reinterpret_cast<const uint4*>(R + grow * ldr + col + piece * 8);
                uint32_t* cw = &cv.x;
                const uint32_t* rw = &resv.x;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const __nv_bfloat162 hc = *reinterpret_cast<const __nv_bfloat162*>(&cw[e]);
                  const __nv_bfloat162 hr = *reinterpret_cast<const __nv_bfloat162*>(&rw[e]);
                  __nv_bfloat162 hs = __floats2bfloat162_rn(__bfloat162float(hc.x) + __bfloat162float(hr.x),
                                                            __bfloat162float(hc.y) + __bfloat162float(hr.y));
                  cw[e] = *reinterpret_cast<uint32_t*>(&hs);
                }
              }
              *reinterpret_cast<uint4*>(C + grow * ldc + col + piece * 8) = cv;
            }
          }
          __syncwarp();
        } else if (row < M && col < N) {
          bf16* cp = C + row * ldc + col;
          const bf16* rp = R ? R + row * ldr + col : nullptr;
          for (int j = 0; j < 32 && col + j < N; ++j) {
            float f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[j])));
            if (rp) f += __bfloat162float(rp[j]);
            cp[j] = __float2bfloat16_rn(f);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (TWO) mbar_arrive_cluster(mapa_u32(smem_u32(&sm.acc_empty[acc]), 0));
        else mbar_arrive(&sm.acc_empty[acc]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (TWO) cluster_sync_all();     // neither CTA leaves while the other may still touch its memory
  if constexpr (SK) {
    if (split) {
      cluster_sync_all();                    // every CTA's partial tile is in its shared memory
      constexpr int CPL = BN / 32;           // columns per lane: a warp covers one row of the tile
      const int rows_per = 64 / ksplit;
      const int nb = (int)(unit % n_tiles);
      const uint32_t red0 = smem_u32(&sm.a[0][0]);
      if (unit < total_tiles) {
        for (int rr = warp; rr < rows_per; rr += TG_THREADS / 32) {
          const int row = (int)ks * rows_per + rr;
          if (row >= M) continue;
          float v[CPL];
#pragma unroll
          for (int j = 0; j < CPL; ++j) v[j] = 0.f;
          const uint32_t off = red0 + (uint32_t)(row * TG_RED_LD(BN) + lane * CPL) * 4u;
          for (int p = 0; p < ksplit; ++p) {
            const uint32_t src = mapa_u32(off, (uint32_t)p);
            if constexpr (CPL == 4) {
              float x0, x1, x2, x3;
              asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x0), "=f"(x1), "=f"(x2), "=f"(x3) : "r"(src) : "memory");
              v[0] += x0; v[1] += x1; v[2] += x2; v[3] += x3;
            } else if constexpr (CPL == 2) {
              float x0, x1;
              asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(x0), "=f"(x1) : "r"(src) : "memory");
              v[0] += x0; v[1] += x1;
            } else {
              float x0;
              asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(x0) : "r"(src) : "memory");
              v[0] += x0;
            }
          }
          const int col = nb * BN + lane * CPL;
          int act = 0;
          float prm = 0.f;
          if (ep.nseg) {
            int sidx = 0;
            while (sidx < ep.nseg - 1 && col >= ep.seg_end[sidx]) ++sidx;
            act = ep.seg_act[sidx];
            prm = ep.seg_param[sidx];
          }
          // the head norm spans the 128 columns of the tile (the host pairs that activation with BN = 128)
          float ss = 0.f;
          if (act == KCH_ACT_SILU_L2NORM) {
#pragma unroll
            for (int j = 0; j < CPL; ++j) { v[j] = bf16r(ep_silu(bf16r(v[j]))); ss = fmaf(v[j], v[j], ss); }
          }
#pragma unroll
          for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (act == KCH_ACT_SILU_L2NORM) {
            const float nrm = __fdividef(1.0f, fmaxf(bf16r(sqrtf(ss)), 1e-12f));
#pragma unroll
            for (int j = 0; j < CPL; ++j) v[j] *= nrm;
          } else if (act == KCH_ACT_SILU) {
#pragma unroll
            for (int j = 0; j < CPL; ++j) v[j] = ep_silu(bf16r(v[j]));
          } else if (act == KCH_ACT_SIGMOID) {
#pragma unroll
            for (int j = 0; j < CPL; ++j) v[j] = __fdividef(1.0f, 1.0f + __expf(-bf16r(v[j])));
          } else if (act == KCH_ACT_NEG_SOFTPLUS) {
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
              const float t = bf16r(v[j]);
              v[j] = -bf16r(t > 20.f ? t : __logf(1.0f + __expf(t))) * prm;
            }
          }
          bf16* cp = C + (int64_t)row * ldc + col;
          const bf16* rp = R ? R + (int64_t)row * ldr + col : nullptr;
#pragma unroll
          for (int j = 0; j < CPL; ++j) {
            if (col + j < N) {
              float f = bf16r(v[j]);
              if (rp) f += __bfloat162float(rp[j]);
              cp[j] = __float2bfloat16_rn(f);
            }
          }
        }
      }
      cluster_sync_all();                    // no CTA leaves while another may still read its partial tile
    }
  }
  if (warp == 1) {
    tc_fence_after();
    if constexpr (TWO)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host side -----------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  });
  return fn;
}

static int make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                       uint32_t box_rows, uint32_t box_cols) {
  PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode_fn();
  if (!enc) { kch_set_error("cuTensorMapEncodeTiled is not available from the driver"); return KCH_ERR_CUDA; }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { kch_set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return KCH_ERR_CUDA; }
  return KCH_OK;
}

// bf16 [rows][cols] tensor map with the 128-byte swizzle for other translation units (box = box_rows x box_cols)
int kch_make_tensor_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                                uint32_t box_rows, uint32_t box_cols) {
  return make_map_2d(map, base, rows, cols, ld_elems, box_rows, box_cols);
}

// bf16 [rows][64 * katoms] matrix seen as {64 elements, rows, katoms}: a box of `box_katoms` k-blocks lands as that
// many consecutive [box_rows x 128 bytes] stages under the 128-byte swizzle (one copy instead of one per k-block)
int kch_make_tensor_map_katoms_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t katoms, uint64_t ld_elems,
                                    uint32_t box_rows, uint32_t box_katoms) {
  PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode_fn();
  if (!enc) { kch_set_error("cuTensorMapEncodeTiled is not available from the driver"); return KCH_ERR_CUDA; }
  cuuint64_t gdim[3] = {64, rows, katoms};
  cuuint64_t gstr[2] = {ld_elems * 2, 128};
  cuuint32_t box[3] = {64, box_rows, box_katoms};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { kch_set_error("cuTensorMapEncodeTiled (k-block view) failed with code %d", (int)r); return KCH_ERR_CUDA; }
  return KCH_OK;
}

// bf16 [rows][nh * 128] activations seen as {128 channels, nh heads, rows}: a box {64, box_heads, box_rows} lands as
// one 64-channel panel of a [box_rows x box_heads rows][64] operand tile (row = token-major, head-minor) under the
// 128-byte swizzle; heads beyond nh read as zeros
int kch_make_tensor_map_qtile_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint32_t nh, uint64_t ld_elems,
                                   uint32_t box_heads, uint32_t box_rows) {
  PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode_fn();
  if (!enc) { kch_set_error("cuTensorMapEncodeTiled is not available from the driver"); return KCH_ERR_CUDA; }
  cuuint64_t gdim[3] = {128, nh, rows};
  cuuint64_t gstr[2] = {256, ld_elems * 2};
  cuuint32_t box[3] = {64, box_heads, box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { kch_set_error("cuTensorMapEncodeTiled (query tile view) failed with code %d", (int)r); return KCH_ERR_CUDA; }
  return KCH_OK;
}

bool kch_linear_tcgen05_supported(const void* A, const void* W, const void* C, const void* R, int64_t M, int N,
                                  int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype) {
  if (dtype != KCH_BF16) return false;
  if (M < 1 || N < 1 || K < 8) return false;
  if ((K % 8) || (lda % 8) || (ldw % 8)) return false;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return false;
  if (M > 0x7FFFFFFFLL) return false;
  (void)C; (void)R; (void)ldc; (void)ldr;
  return true;
}

template <int BN>
static int launch_tg(const void* A, const void* W, void* C, const void* R, int64_t M, int N, int K, int64_t lda,
                     int64_t ldw, int64_t ldc, int64_t ldr, const TgEpilogue& ep, cudaStream_t s, int slab_k = 0,
                     bool skinny = false) {
  CUtensorMap ma, mw;
  skinny = skinny && BN <= 128 && M <= 64;
  const uint32_t a_rows = skinny ? 64 : TG_BM;
  int rc = slab_k > 0 ? make_map_2d(&ma, A, (uint64_t)M * (uint64_t)(K / slab_k), (uint64_t)slab_k, (uint64_t)slab_k, a_rows, TG_BK)
                      : make_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, a_rows, TG_BK);
  if (rc) return rc;
  rc = make_map_2d(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN, TG_BK);
  if (rc) return rc;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    KCH_CUDA_OK(cudaGetDevice(&dev));
    KCH_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  int64_t tiles = ((M + TG_BM - 1) / TG_BM) * ((N + BN - 1) / BN);
  int grid = (int)(tiles < sms ? tiles : sms);
  int vec_ok = (ldc % 8 == 0) && (((uintptr_t)C & 15) == 0) && (!R || ((ldr % 8 == 0) && (((uintptr_t)R & 15) == 0)));
  if constexpr (BN <= 128) {
    if (skinny) {
      size_t smem = sizeof(TgSmem<BN, false, true>) + 1024;
      KCH_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      // Split the K loop over a cluster when the tiles alone would leave most SMs idle: two CTAs fit on an SM, so up
      // to 2 * sms CTAs run at once.  Every share of k-blocks must be non-empty.  (KCH_GEMM_KSPLIT=1 turns it off.)
      static const int ks_max = [] { const char* e = getenv("KCH_GEMM_KSPLIT"); return e && e[0] >= '1' && e[0] <= '4' ? e[0] - '0' : 4; }();
      const int kblocks = (K + TG_BK - 1) / TG_BK;
      int ksplit = 1;
      for (int c = 4; c >= 2; c >>= 1)
        if (c <= ks_max && kblocks >= 4 * c && tiles * c <= 2 * (int64_t)sms) { ksplit = c; break; }
      while (ksplit > 1 && (ksplit - 1) * ((kblocks + ksplit - 1) / ksplit) >= kblocks) ksplit >>= 1;
      if (ksplit > 1) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)ksplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.gridDim = dim3((unsigned)(tiles * ksplit)); cfg.blockDim = dim3(TG_THREADS); cfg.dynamicSmemBytes = smem;
        cfg.stream = s; cfg.attrs = attr; cfg.numAttrs = 1;
        KCH_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN, false, true>, ma, mw, (bf16*)C, (const bf16*)R, M, N, K,
                                       ldc, ldr, vec_ok, ep, slab_k, M, ksplit));
        kch_note_launch(1);
        return KCH_OK;
      }
      gemm_tcgen05_kernel<BN, false, true><<<grid, TG_THREADS, smem, s>>>(ma, mw, (bf16*)C, (const bf16*)R, M, N, K, ldc, ldr,
                                                                         vec_ok, ep, slab_k, M, 1);
      KCH_LAUNCH_OK();
      return KCH_OK;
    }
  }
  size_t smem = sizeof(TgSmem<BN>) + 1024;
  KCH_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  gemm_tcgen05_kernel<BN, false><<<grid, TG_THREADS, smem, s>>>(ma, mw, (bf16*)C, (const bf16*)R, M, N, K, ldc, ldr, vec_ok, ep,
                                                               slab_k, M, 1);
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// 256 x 256 tiles on CTA pairs (clusters of two, tcgen05 cta_group::2): each CTA loads its 128 rows of A and half
// of the W tile, so a CTA moves 32 KB per k-block instead of 48 KB and the ring holds six stages.
static int launch_tg_pair(const void* A, const void* W, void* C, const void* R, int64_t M, int N, int K, int64_t lda,
                          int64_t ldw, int64_t ldc, int64_t ldr, const TgEpilogue& ep, cudaStream_t s, int slab_k = 0) {
  constexpr int BN = 256;
  CUtensorMap ma, mw;
  int rc = slab_k > 0 ? make_map_2d(&ma, A, (uint64_t)M * (uint64_t)(K / slab_k), (uint64_t)slab_k, (uint64_t)slab_k, TG_BM, TG_BK)
                      : make_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TG_BM, TG_BK);
  if (rc) return rc;
  rc = make_map_2d(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN / 2, TG_BK);
  if (rc) return rc;
  size_t smem = sizeof(TgSmem<BN, true>) + 1024;
  KCH_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(TG_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s; cfg.attrs = attr; cfg.numAttrs = 1;
  static int max_pairs = 0;
  if (!max_pairs) {
    cfg.gridDim = dim3(2);
    int nc = 0;
    KCH_CUDA_OK(cudaOccupancyMaxActiveClusters(&nc, gemm_tcgen05_kernel<BN, true>, &cfg));
    KCH_REQUIRE(nc > 0, "kch_linear: no CTA pair of the tcgen05 GEMM fits on this device");
    max_pairs = nc;
  }
  int64_t tiles = ((M + 2 * TG_BM - 1) / (2 * TG_BM)) * ((N + BN - 1) / BN);
  int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
  cfg.gridDim = dim3(2 * pairs);
  int vec_ok = (ldc % 8 == 0) && (((uintptr_t)C & 15) == 0) && (!R || ((ldr % 8 == 0) && (((uintptr_t)R & 15) == 0)));
  KCH_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN, true>, ma, mw, (bf16*)C, (const bf16*)R, M, N, K, ldc, ldr,
                                 vec_ok, ep, slab_k, M, 1));
  kch_note_launch(1);
  return KCH_OK;
}

// Can the epilogue described by `e` run fused?  Segment boundaries must fall on 32-column chunks and
// L2-norm heads (128 columns) on 128-column boundaries of a tile that is at least 128 wide.
bool kch_linear_tcgen05_epilogue_ok(const kch_epilogue* e, int N) {
  if (!e || e->n_segments == 0) return true;
  if (e->n_segments > 8) return false;
  int start = 0;
  for (int i = 0; i < e->n_segments; ++i) {
    const int end = e->seg_end[i];
    if (end <= start || end > N) return false;
    if (i + 1 < e->n_segments && (end % 32) != 0) return false;
    if (e->seg_act[i] == KCH_ACT_SILU_L2NORM && (e->group != 128 || (start % 128) != 0 || ((end - start) % 128) != 0 || N <= 64))
      return false;
    start = end;
  }
  return start == N;
}

int kch_linear_decode_tc5(const void* A, const void* W, void* C, const void* R, int64_t M, int N, int K, int64_t lda,
                          int64_t ldw, int64_t ldc, int64_t ldr, const kch_epilogue* e, void* stream);

int kch_linear_tcgen05(const void* A, const void* W, void* C, const void* R, int64_t M, int N, int K, int64_t lda,
                       int64_t ldw, int64_t ldc, int64_t ldr, const kch_epilogue* e, void* stream, int slab_k) {
  cudaStream_t s = kch_stream(stream);
  TgEpilogue ep = {};
  if (e && e->n_segments) {
    ep.nseg = e->n_segments;
    for (int i = 0; i < e->n_segments; ++i) { ep.seg_end[i] = e->seg_end[i]; ep.seg_act[i] = e->seg_act[i]; ep.seg_param[i] = e->seg_param[i]; }
  }
  if (M <= 64 && slab_k == 0) {
    // a decode batch: the kernel built for it (one copy per operand, K split over a cluster); -100 = not its shape
    const int rc = kch_linear_decode_tc5(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, e, stream);
    if (rc != -100) return rc;
  }
  if (M <= TG_BM && N > 128) {
    // One row of tiles (a decode batch): the launch is a weight stream, so spread it over many SMs with
    // narrow tiles.  A fused L2-norm needs a whole 128-column head inside the tile.
    bool l2 = false;
    for (int i = 0; i < ep.nseg; ++i) l2 = l2 || ep.seg_act[i] == KCH_ACT_SILU_L2NORM;
    // (KCH_GEMM_SKINNY=0 keeps the 128-row A box for a batch of at most 64 rows, for comparison)
    static const bool sk_on = [] { const char* e = getenv("KCH_GEMM_SKINNY"); return !(e && e[0] == '0'); }();
    if (l2) return launch_tg<128>(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, ep, s, slab_k, sk_on);
    return launch_tg<32>(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, ep, s, slab_k, sk_on);
  }
  // large products: 256 x 256 tiles on CTA pairs (KCH_GEMM=1 keeps one CTA per tile, for comparison)
  static const bool pair_on = [] { const char* e = getenv("KCH_GEMM"); return !(e && e[0] == '1'); }();
  if (pair_on && N > 128 && M >= 4 * TG_BM) return launch_tg_pair(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, ep, s, slab_k);
  if (N > 128) return launch_tg<256>(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, ep, s, slab_k);
  if (N > 64) return launch_tg<128>(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, ep, s, slab_k);
  if (N > 32) return launch_tg<64>(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, ep, s, slab_k);
  return launch_tg<32>(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, ep, s, slab_k);
}

// =====================================================================================================
// Lightning-indexer logits on the same machinery (csa_lightning_indexer, ops_csa.py:503-554):
//   logits[t, n] = sum_h w[t,h] relu(scale q_h[t] . k[n] / ||q_h[t]||)  =  sum_h c[t,h] relu(q_h[t] . k[n]),
//   c[t,h] = w[t,h] scale / max(||q_h[t]||, 1e-12)  (the positive factor commutes with the ReLU).
// Queries are the bf16 rows the projection wrote (exact operands, read in place through a tensor map);
// the normalised fp32 keys arrive as three bf16 terms (hi + mid + lo, 24 bits of mantissa), so per head a
// 128-query x 256-block tile is 12 tcgen05.mma (3 terms x K = 64) into one tensor-memory accumulator.
// Epilogue warps apply c relu(.) and sum the heads in registers; the two accumulator buffers let the
// epilogue of head h overlap the MMAs of head h+1.  Tiles are the causally visible ones only, taken in
// strips of one key tile (the key operand stays in shared memory for a whole strip) and dealt out to the
// persistent CTAs in equal contiguous runs.
// =====================================================================================================
#define IX_BM 128
#define IX_BN 256
#define IX_D 64
#define IX_ASTAGES 4
#define IX_MAX_STRIPS 256

struct IxSched {
  int n_strips;                        // B * ceil(n / IX_BN)
  int total_tiles;
  int prefix[IX_MAX_STRIPS + 1];       // visible tiles before strip s
  short qt_first[IX_MAX_STRIPS];       // first query tile that sees strip s
};

struct IxSmem {
  alignas(1024) bf16 kb[3][IX_BN * IX_D];          // key tile, three terms
  alignas(1024) bf16 qa[IX_ASTAGES][IX_BM * IX_D]; // query tiles (one head each)
  alignas(8) uint64_t a_full[IX_ASTAGES];
  uint64_t a_empty[IX_ASTAGES];
  uint64_t b_full, b_empty;
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

__global__ void indexer_coef_kernel(const bf16* __restrict__ q, int64_t q_ld, const float* __restrict__ w,
                                    float* __restrict__ coef, int64_t rows, int HI, float scale, int normalize) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  for (int h = 0; h < HI; ++h) {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(q + row * q_ld + h * IX_D + 2 * lane);
    const float x = __uint_as_float(raw << 16), y = __uint_as_float(raw & 0xFFFF0000u);
    float ss = x * x + y * y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) {
      const float nrm = normalize ? fmaxf(sqrtf(ss), 1e-12f) : 1.f;
      coef[row * HI + h] = (w ? w[row * HI + h] : 1.f) * scale / nrm;
    }
  }
}

__global__ void __launch_bounds__(TG_THREADS, 1)
indexer_logits_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kh,
                              const __grid_constant__ CUtensorMap map_km, const __grid_constant__ CUtensorMap map_kl,
                              const __grid_constant__ IxSched sched, const float* __restrict__ coef,
                              float* __restrict__ logits, int T, int n, int HI, int64_t n_ld, int strips_per_batch) {
  extern __shared__ uint8_t smem_raw[];
  IxSmem& sm = *reinterpret_cast<IxSmem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * IX_BN;
  if (threadIdx.x == 0) {
    for (int s = 0; s < IX_ASTAGES; ++s) { mbar_init(&sm.a_full[s], 1); mbar_init(&sm.a_empty[s], 1); }
    mbar_init(&sm.b_full, 1); mbar_init(&sm.b_empty, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  // this CTA's run of visible tiles
  const int per = (sched.total_tiles + (int)gridDim.x - 1) / (int)gridDim.x;
  const int tile_lo = min(sched.total_tiles, (int)blockIdx.x * per), tile_hi = min(sched.total_tiles, tile_lo + per);
  auto strip_of = [&](int tile, int hint) {          // strips are visited in order: a short forward scan finds it
    int s = hint;
    while (s + 1 < sched.n_strips && sched.prefix[s + 1] <= tile) ++s;
    return s;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t ait = 0, bit = 0;
      int strip = 0, cur = -1;
      bool ok = true;
      for (int tile = tile_lo; tile < tile_hi && ok; ++tile) {
        strip = strip_of(tile, strip);
        const int b = strip / strips_per_batch, nt = strip % strips_per_batch;
        const int qt = sched.qt_first[strip] + (tile - sched.prefix[strip]);
        if (strip != cur) {
          if (!mbar_wait(&sm.b_empty, (bit & 1) ^ 1, 31)) { ok = false; break; }
          mbar_expect_tx(&sm.b_full, 3 * IX_BN * IX_D * 2);
          const int row = b * n + nt * IX_BN;
          tma_load_2d(sm.kb[0], &map_kh, 0, row, &sm.b_full);
          tma_load_2d(sm.kb[1], &map_km, 0, row, &sm.b_full);
          tma_load_2d(sm.kb[2], &map_kl, 0, row, &sm.b_full);
          ++bit;
          cur = strip;
        }
        for (int h = 0; h < HI; ++h, ++ait) {
          const uint32_t s = ait % IX_ASTAGES, ph = (ait / IX_ASTAGES) & 1;
          if (!mbar_wait(&sm.a_empty[s], ph ^ 1, 32)) { ok = false; break; }
          mbar_expect_tx(&sm.a_full[s], IX_BM * IX_D * 2);
          tma_load_2d(sm.qa[s], &map_q, h * IX_D, b * T + qt * IX_BM, &sm.a_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(IX_BN >> 3) << 17) | ((uint32_t)(IX_BM >> 4) << 24);
      uint32_t ait = 0, bit = 0, hcount = 0;
      int strip = 0, cur = -1;
      bool ok = true;
      for (int tile = tile_lo; tile < tile_hi && ok; ++tile) {
        strip = strip_of(tile, strip);
        if (strip != cur) {
          if (cur >= 0) tc_commit(&sm.b_empty);         // every MMA that read the previous key tile has completed
          if (!mbar_wait(&sm.b_full, bit & 1, 33)) { ok = false; break; }
          tc_fence_after();
          ++bit;
          cur = strip;
        }
        for (int h = 0; h < HI; ++h, ++ait, ++hcount) {
          const uint32_t acc = hcount & 1, aph = (hcount >> 1) & 1;
          const uint32_t s = ait % IX_ASTAGES, ph = (ait / IX_ASTAGES) & 1;
          if (!mbar_wait(&sm.acc_empty[acc], aph ^ 1, 34)) { ok = false; break; }
          if (!mbar_wait(&sm.a_full[s], ph, 35)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * IX_BN;
          const uint64_t adesc = make_smem_desc(smem_u32(sm.qa[s]));
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const uint64_t bdesc = make_smem_desc(smem_u32(sm.kb[term]));
#pragma unroll
            for (int k = 0; k < IX_D / 16; ++k)
              tc_mma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (term | k) ? 1u : 0u);
          }
          tc_commit(&sm.a_empty[s]);
          tc_commit(&sm.acc_full[acc]);
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int quarter = warp & 3;            // tensor-memory lanes 32*quarter .. +31 = query rows of the tile
    const int half = (warp - 2) >> 2;        // columns half*128 .. +127
    uint32_t hcount = 0;
    int strip = 0;
    bool ok = true;
    for (int tile = tile_lo; tile < tile_hi && ok; ++tile) {
      strip = strip_of(tile, strip);
      const int b = strip / strips_per_batch, nt = strip % strips_per_batch;
      const int qt = sched.qt_first[strip] + (tile - sched.prefix[strip]);
      const int64_t row = (int64_t)b * T + qt * IX_BM + quarter * 32 + lane;
      float out[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) out[j] = 0.f;
      for (int h = 0; h < HI; ++h, ++hcount) {
        const uint32_t acc = hcount & 1, aph = (hcount >> 1) & 1;
        if (!mbar_wait(&sm.acc_full[acc], aph, 36)) { ok = false; break; }
        tc_fence_after();
        const float c = coef[row * HI + h];
        const uint32_t tbase = tmem_base + acc * IX_BN + half * 128 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t r[32];
          tc_ld32(tbase + c0, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) out[c0 + j] = fmaf(c, fmaxf(__uint_as_float(r[j]), 0.f), out[c0 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.acc_empty[acc]);
      }
      if (!ok) break;
      const int col0 = nt * IX_BN + half * 128;
      float* dst = logits + row * n_ld + col0;
#pragma unroll
      for (int j = 0; j < 128; j += 4)
        if (col0 + j + 4 <= n_ld) *reinterpret_cast<float4*>(dst + j) = make_float4(out[j], out[j + 1], out[j + 2], out[j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Host side.  `coef` is caller workspace of B*T*HI floats; kh/km/kl are the three key terms, [B*n][64] bf16 each.
bool kch_indexer_logits_tcgen05_ok(int B, int T, int n, int HI, int64_t q_ld, const void* q) {
  static const bool off = [] { const char* e = getenv("KCH_INDEXER"); return e && e[0] == 'm'; }();   // "mma": legacy path
  const int strips = (n + IX_BN - 1) / IX_BN;
  return !off && T % IX_BM == 0 && HI >= 1 && HI <= 16 && (int64_t)B * strips <= IX_MAX_STRIPS && (q_ld % 8) == 0 &&
         (((uintptr_t)q) & 15) == 0 && T / IX_BM < 32768;
}

int kch_indexer_logits_tcgen05(const void* q, int64_t q_ld, int q_normalize, const void* kh, const void* km,
                               const void* kl, const float* w, float* coef, float* logits, int B, int T, int n, int HI,
                               int64_t n_ld, float scale, int m, int64_t t0, int n_visible, cudaStream_t s) {
  const int64_t rows = (int64_t)B * T;
  indexer_coef_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const bf16*)q, q_ld, w, coef, rows, HI, scale, q_normalize);
  KCH_LAUNCH_OK();
  CUtensorMap mq, mkh, mkm, mkl;
  int rc = make_map_2d(&mq, q, (uint64_t)rows, (uint64_t)HI * IX_D, (uint64_t)q_ld, IX_BM, IX_D);
  if (rc) return rc;
  const uint64_t krows = (uint64_t)B * n;
  if ((rc = make_map_2d(&mkh, kh, krows, IX_D, IX_D, IX_BN, IX_D))) return rc;
  if ((rc = make_map_2d(&mkm, km, krows, IX_D, IX_D, IX_BN, IX_D))) return rc;
  if ((rc = make_map_2d(&mkl, kl, krows, IX_D, IX_D, IX_BN, IX_D))) return rc;
  // visible tiles per strip: query tile qt sees key tile nt iff nt*256 < min(n, visible blocks of its last query)
  IxSched sch;
  const int strips = (n + IX_BN - 1) / IX_BN, QT = T / IX_BM;
  sch.n_strips = B * strips;
  int total = 0;
  for (int b = 0; b < B; ++b)
    for (int nt = 0; nt < strips; ++nt) {
      int first = QT;
      // visibility is monotone in qt: binary search the first visible query tile
      int lo = 0, hi = QT;
      while (lo < hi) {
        const int mid = (lo + hi) / 2;
        const int64_t tlast = (int64_t)mid * IX_BM + IX_BM - 1;
        int64_t vis = n_visible >= 0 ? n_visible : (m > 0 ? (t0 + tlast + 1) / m : n);
        if (vis > n) vis = n;
        if ((int64_t)nt * IX_BN < vis) hi = mid; else lo = mid + 1;
      }
      first = lo;
      const int sidx = b * strips + nt;
      sch.prefix[sidx] = total;
      sch.qt_first[sidx] = (short)first;
      total += QT - first;
    }
  sch.prefix[sch.n_strips] = total;
  sch.total_tiles = total;
  if (total == 0) return KCH_OK;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    KCH_CUDA_OK(cudaGetDevice(&dev));
    KCH_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const size_t smem = sizeof(IxSmem) + 1024;
  KCH_CUDA_OK(cudaFuncSetAttribute(indexer_logits_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = total < sms ? total : sms;
  indexer_logits_tcgen05_kernel<<<grid, TG_THREADS, smem, s>>>(mq, mkh, mkm, mkl, sch, coef, logits, T, n, HI, n_ld, strips);
  KCH_LAUNCH_OK();
  return KCH_OK;
}

unsigned int* kch_status_device_ptr() {
  static unsigned int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    unsigned int* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_kch_status) != cudaSuccess) return nullptr;
    cached[dev] = p;
  }
  return cached[dev];
}

// One CTA waits, with the kernels' own bounded wait, on an mbarrier that nothing ever arrives at.  The wait must
// give up after `limit` polls, record its code in the status word and return: the path every tcgen05 kernel of this
// library takes when a copy or an MMA it waits for never completes.  Nothing traps and the context stays usable.
__global__ void selftest_bounded_wait_kernel(uint32_t limit, unsigned int* polls_out) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool ok = mbar_wait(&bar, 0, KCH_STATUS_SELFTEST_WAIT, limit);
    if (polls_out) *polls_out = ok ? 0u : limit;
  }
}

extern "C" int kch_selftest_bounded_wait(unsigned int limit_polls, unsigned int* polls_out, void* stream) {
  KCH_REQUIRE(limit_polls >= 1 && limit_polls <= (1u << 20),
              "kch_selftest_bounded_wait: limit_polls=%u must be in [1, 2^20]", limit_polls);
  selftest_bounded_wait_kernel<<<1, 32, 0, kch_stream(stream)>>>(limit_polls, polls_out);
  KCH_LAUNCH_OK();
  return KCH_OK;
}

extern "C" unsigned int kch_device_status(int reset) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_kch_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
  if (reset && v) {
    unsigned int z = 0;
    cudaMemcpyToSymbol(g_kch_status, &z, sizeof(z));
  }
  return v;
}
