// F.linear for a decode batch (at most 64 rows): C[M,N] = A[M,K] . W[N,K]^T (+ activations, + residual) on tcgen05.
//
// One token per sequence makes every projection of the step (ops_fused.py:571-581,609,713,739; ops_csa.py:841-878;
// ops_hca.py:132-141) a stream of weights against 64 rows of activations: 8 to 26 MB of W per launch, a few microseconds
// of HBM time, so what is left to lose is latency -- issue slots of the copy engine, dependent round trips, barriers.
// This kernel is built around that:
//   * the operands are described as 3-D tensors {64 elements of K, rows, K / 64}: ONE cp.async.bulk.tensor per operand
//     brings all k-blocks of a CTA (up to 8 x [rows x 128 bytes], each landing as one 128-byte-swizzled stage), instead of
//     two copies per k-block at roughly a hundred issue cycles each;
//   * a tile of BN output columns is one cluster of `ksplit` CTAs along K, so that every SM holds two CTAs with their
//     whole share of the weights in flight at once;
//   * partial tiles are reduced through distributed shared memory.  BN = 32: every CTA PUSHES its fp32 partial rows
//     into the shared memory of the CTA that owns those rows (stores, no round trip), one cluster barrier, then each
//     CTA finishes its own rows from local memory and may leave.  BN = 128 (the tile a fused per-head L2 norm needs)
//     has no room for a separate landing buffer beside the ring, so partials stay where they are (over the drained
//     ring) and owners PULL them, all loads issued before the first add, with a second barrier before anyone leaves;
//   * partial sums are added in rank order, so the result does not depend on timing; activation, residual and
//     rounding steps are those of the large-batch kernel (product rounded to bf16, every further step reads bf16,
//     computes in fp32, rounds to bf16);
//   * the residual rows a thread will need are loaded right after the set-up, long before the accumulators exist.
// The MMA spans 128 rows although the A box holds 64: rows 64..127 of the operand are whatever follows in shared
// memory (the next stage), which only reaches accumulator rows that are never read.
// Every mbarrier wait is bounded (status word, see kch_device_status).  No multicast.
#include <cuda.h>
#include <stdlib.h>

#include "kch_common.cuh"
#include "tc5_utils.cuh"

#define GD_THREADS 128
#define GD_ROWS 64
#define GD_BK 64
#define GD_A_BYTES (GD_ROWS * GD_BK * 2)
#define GD_RED_LD(BN) ((BN) + 4)      // fp32 row pitch of a partial tile: 16 bytes of padding against bank conflicts
#define GD_SPIN (1u << 24)
#define GD_UNSUPPORTED (-100)

struct GdEpilogue {
  int nseg;
  int seg_end[8];
  int seg_act[8];
  float seg_param[8];
};

template <int BN>
struct GdCfg {
  static constexpr int G = BN >= 64 ? 4 : 8;             // k-blocks of one CTA (= stages, all in flight at once)
  static constexpr bool PUSH = BN < 128;
  static constexpr int W_BYTES = BN * GD_BK * 2;
  static constexpr int RING = G * (GD_A_BYTES + W_BYTES);
  static constexpr int RED_BYTES = 64 * GD_RED_LD(BN) * 4;
  static constexpr int BAR_OFF = RING + (PUSH ? RED_BYTES : 0);
  static constexpr int SMEM = BAR_OFF + 64 + 1024;        // + barriers / tensor-memory base, + alignment slack
  static_assert(PUSH || RED_BYTES <= RING, "the pulled partial tile lives over the drained ring");
};

__device__ __forceinline__ uint32_t gd_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t gd_mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void gd_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void gd_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void gd_tma_load_3d(uint32_t dst, const void* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(smem_addr_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ float gd_bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float gd_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int BN>
__global__ void __launch_bounds__(GD_THREADS)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                   bf16* __restrict__ C, const bf16* __restrict__ R, int M, int N, int kblocks_all, int kper,
                   int64_t ldc, int64_t ldr, int vec_ok, const GdEpilogue ep, int ksplit, int gr, int ng,
                   unsigned int* status) {
  // `gr` k-blocks per copy (the depth of a tensor-map box), `ng` groups of `gr` stages: ng = 1 when the CTA's whole
  // share fits the ring (one copy per operand), else 2 groups refilled in turn as their MMAs retire
  using Cfg = GdCfg<BN>;
  constexpr int RED_LD = GD_RED_LD(BN);
  constexpr int QPR = BN / 4;                               // float4 items per row of the tile
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ uint8_t gd_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)gd_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_addr_u32(base);
  const uint32_t a0 = sbase, w0 = sbase + Cfg::G * GD_A_BYTES;
  const uint32_t red0 = Cfg::PUSH ? sbase + Cfg::RING : sbase;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + Cfg::BAR_OFF);      // [0,1] group landed, [2,3] group drained, [4] accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool split = ksplit > 1;
  const int ks = split ? (int)gd_cluster_rank() : 0;
  const int nb = (int)(blockIdx.x / ksplit);                               // one tile per cluster
  const int kb_first = ks * kper;
  const int kblocks = min(kper, kblocks_all - kb_first);                   // >= 1 (the host keeps every share non-empty)

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) mbarrier_init(&bars[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (split && Cfg::PUSH) gd_cluster_arrive();       // "my shared memory exists": waited for before the first push
  const int nrounds = (kblocks + gr - 1) / gr;
  auto issue_round = [&](int r) {                    // k-blocks [r * gr, (r + 1) * gr) of this CTA into group r % ng
    const int gi = r % ng;
    mbarrier_expect_tx(&bars[gi], (uint32_t)gr * (GD_A_BYTES + Cfg::W_BYTES));       // a box is `gr` k-blocks deep
    gd_tma_load_3d(a0 + gi * gr * GD_A_BYTES, &map_a, 0, 0, kb_first + r * gr, &bars[gi]);
    gd_tma_load_3d(w0 + gi * gr * Cfg::W_BYTES, &map_w, 0, nb * BN, kb_first + r * gr, &bars[gi]);
  };
  if (tid == 0) {                                    // the operand copies, first thing
    for (int r = 0; r < min(ng, nrounds); ++r) issue_round(r);
  }

  // ---- the rows this thread finishes, and their residual values (an earlier kernel's output: ready now) ----------
  const int rows_per = 64 / ksplit;
  const int items = rows_per * QPR;
  uint2 rpre[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    rpre[i] = make_uint2(0u, 0u);
    const int it = tid + i * GD_THREADS;
    if (R && vec_ok && it < items) {
      const int row = ks * rows_per + it / QPR, col = nb * BN + (it % QPR) * 4;
      if (row < M && col + 4 <= N) rpre[i] = *reinterpret_cast<const uint2*>(R + (int64_t)row * ldr + col);
    }
  }

  // ---- one thread: every MMA of this CTA's share, once the operands have landed ------------------------------------
  bool ok = true;
  if (tid == 0) {
    const uint32_t idesc = t5_idesc(BN);
    for (int r = 0; r < nrounds && ok; ++r) {
      const int gi = r % ng, par = (r / ng) & 1;
      ok = mbarrier_wait_bounded(&bars[gi], par, KCH_STATUS_GEMM_DECODE, GD_SPIN, status);
      if (!ok) break;
      t5_fence_after();
      const int nk = min(gr, kblocks - r * gr);
      for (int j = 0; j < nk; ++j) {
        const int st = gi * gr + j;
        const uint64_t adesc = t5_desc(a0 + st * GD_A_BYTES), bdesc = t5_desc(w0 + st * Cfg::W_BYTES);
#pragma unroll
        for (int k = 0; k < GD_BK / 16; ++k) t5_mma(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (r | j | k) ? 1u : 0u);
      }
      if (r + ng < nrounds) {                          // refill this group once its MMAs have read it
        t5_commit(&bars[2 + gi]);
        ok = mbarrier_wait_bounded(&bars[2 + gi], par, KCH_STATUS_GEMM_DECODE, GD_SPIN, status);
        if (ok) issue_round(r + ng);
      }
    }
    if (ok) t5_commit(&bars[4]);
  }
  __syncwarp();
  if (split && Cfg::PUSH) gd_cluster_wait();          // every CTA of the cluster is running: its shared memory may be written

  // ---- accumulator rows 0..63 -> fp32 partial rows (warps 0 and 1 own tensor-memory lanes 0..63) ----------------------
  if (warp < 2) {
    ok = mbarrier_wait_bounded(&bars[4], 0, KCH_STATUS_GEMM_DECODE, GD_SPIN, status);
    t5_fence_after();
    const int row = warp * 32 + lane;
    uint32_t dst;
    if (Cfg::PUSH) {
      const int owner = row / rows_per, rl = row - owner * rows_per;
      dst = red0 + (uint32_t)((ks * rows_per + rl) * RED_LD) * 4u;          // slot `ks` of the owner's landing buffer
      if (split) dst = gd_mapa(dst, (uint32_t)owner);
    } else {
      dst = red0 + (uint32_t)(row * RED_LD) * 4u;                           // stays here; owners come and read
    }
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        t5_ld32(tmem + ((uint32_t)(warp * 32) << 16) + c0, r);
        t5_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t d = dst + (uint32_t)(c0 + 4 * j) * 4u;
          if (Cfg::PUSH && split)
            asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d), "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
          else
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d), "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
        }
      }
    }
    t5_fence_before();
  }
  if (split) { gd_cluster_arrive(); gd_cluster_wait(); } else { __syncthreads(); }

  // ---- finish this CTA's rows: sum the partials in rank order, activation, residual, store ----------------------------
  auto finish = [&](const int it, const uint2 rpre_v, const bool have_pre) {
    const bool live = it < items;                       // uniform over a warp (items is a multiple of 32 where it matters)
    const int rl = live ? it / QPR : 0, q = live ? it % QPR : 0;
    const int row = ks * rows_per + rl;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (Cfg::PUSH) {
#pragma unroll 1
      for (int p = 0; p < ksplit; ++p) {
        float x0, x1, x2, x3;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x0), "=f"(x1), "=f"(x2), "=f"(x3)
                     : "r"(red0 + (uint32_t)((p * rows_per + rl) * RED_LD + q * 4) * 4u) : "memory");
        v[0] += x0; v[1] += x1; v[2] += x2; v[3] += x3;
      }
    } else {
      float x[8][4];
      const uint32_t off = red0 + (uint32_t)(row * RED_LD + q * 4) * 4u;
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        x[p][0] = x[p][1] = x[p][2] = x[p][3] = 0.f;
        if (p < ksplit) {
          const uint32_t src = split ? gd_mapa(off, (uint32_t)p) : off;
          asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x[p][0]), "=f"(x[p][1]), "=f"(x[p][2]), "=f"(x[p][3])
                       : "r"(src) : "memory");
        }
      }
#pragma unroll
      for (int p = 0; p < 8; ++p) { v[0] += x[p][0]; v[1] += x[p][1]; v[2] += x[p][2]; v[3] += x[p][3]; }
    }
    const int col = nb * BN + q * 4;
    int act = 0;
    float prm = 0.f;
    if (ep.nseg) {
      int sidx = 0;
      while (sidx < ep.nseg - 1 && col >= ep.seg_end[sidx]) ++sidx;
      act = ep.seg_act[sidx];
      prm = ep.seg_param[sidx];
    }
    if (BN == 128) {
      // per-head L2 norm: the head is the 128 columns of this tile, one warp holds the row
      float ss = 0.f;
      if (act == KCH_ACT_SILU_L2NORM) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { v[j] = gd_bf16r(gd_silu(gd_bf16r(v[j]))); ss = fmaf(v[j], v[j], ss); }
      }
      ss = warp_sum(ss);
      if (act == KCH_ACT_SILU_L2NORM) {
        const float nrm = __fdividef(1.0f, fmaxf(gd_bf16r(sqrtf(ss)), 1e-12f));
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] *= nrm;
      }
    }
    if (act == KCH_ACT_SILU) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = gd_silu(gd_bf16r(v[j]));
    } else if (act == KCH_ACT_SIGMOID) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __fdividef(1.0f, 1.0f + __expf(-gd_bf16r(v[j])));
    } else if (act == KCH_ACT_NEG_SOFTPLUS) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float t = gd_bf16r(v[j]);
        v[j] = -gd_bf16r(t > 20.f ? t : __logf(1.0f + __expf(t))) * prm;
      }
    }
    if (!live || row >= M || col >= N) return;
    if (vec_ok && col + 4 <= N) {
      uint2 rv = make_uint2(0u, 0u);
      if (R) rv = have_pre ? rpre_v : *reinterpret_cast<const uint2*>(R + (int64_t)row * ldr + col);
      float f[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) f[j] = gd_bf16r(v[j]);
      if (R) {
        f[0] += __uint_as_float(rv.x << 16); f[1] += __uint_as_float(rv.x & 0xFFFF0000u);
        f[2] += __uint_as_float(rv.y << 16); f[3] += __uint_as_float(rv.y & 0xFFFF0000u);
      }
      const __nv_bfloat162 h0 = __floats2bfloat162_rn(f[0], f[1]), h1 = __floats2bfloat162_rn(f[2], f[3]);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&h0);
      o.y = *reinterpret_cast<const uint32_t*>(&h1);
      *reinterpret_cast<uint2*>(C + (int64_t)row * ldc + col) = o;
    } else {
      for (int j = 0; j < 4 && col + j < N; ++j) {
        float f = gd_bf16r(v[j]);
        if (R) f += __bfloat162float(R[(int64_t)row * ldr + col + j]);
        C[(int64_t)row * ldc + col + j] = __float2bfloat16_rn(f);
      }
    }
  };
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (i * GD_THREADS < items) finish(tid + i * GD_THREADS, rpre[i], true);
#pragma unroll 1
  for (int i = 4; i * GD_THREADS < items; ++i) finish(tid + i * GD_THREADS, make_uint2(0u, 0u), false);
  if (split && !Cfg::PUSH) { gd_cluster_arrive(); gd_cluster_wait(); }     // nobody leaves while a peer may still read its partials
  __syncthreads();
  if (warp == 1) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host ---------------------------------------------------------------------------------------------------------
int kch_make_tensor_map_katoms_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t katoms, uint64_t ld_elems,
                                    uint32_t box_rows, uint32_t box_katoms);

template <int BN>
static int launch_gd(const void* A, const void* W, void* C, const void* R, int M, int N, int K, int64_t lda, int64_t ldw,
                     int64_t ldc, int64_t ldr, const GdEpilogue& ep, cudaStream_t s) {
  using Cfg = GdCfg<BN>;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    KCH_CUDA_OK(cudaGetDevice(&dev));
    KCH_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const int kblocks = K / GD_BK;
  const int tiles = (N + BN - 1) / BN;
  // the fewest CTAs along K whose share fits the ring; more while two CTAs per SM can still hold the whole launch
  // and a share keeps at least two k-blocks
  // CTAs along K: as many as two per SM can hold at once, while a share keeps at least two k-blocks
  // (KCH_GD_KSPLIT=n overrides it for the 128-column tiles, for comparison)
  static const int forced = [] { const char* e = getenv("KCH_GD_KSPLIT"); return e ? atoi(e) : 0; }();
  int ksplit = 1;
  while (ksplit < 8 && (int64_t)tiles * ksplit * 2 <= 2 * (int64_t)sms && kblocks / (ksplit * 2) >= 2) ksplit <<= 1;
  if (BN == 128 && (forced == 1 || forced == 2 || forced == 4 || forced == 8)) ksplit = forced;
  int kper = (kblocks + ksplit - 1) / ksplit;
  while (ksplit > 1 && (ksplit - 1) * kper >= kblocks) { ksplit >>= 1; kper = (kblocks + ksplit - 1) / ksplit; }
  // the whole share in one copy per operand when it fits the ring, else two groups of half the ring refilled in turn
  const int gr = kper <= Cfg::G ? kper : Cfg::G / 2, ng = kper <= Cfg::G ? 1 : 2;
  CUtensorMap ma, mw;
  if (kch_make_tensor_map_katoms_bf16(&ma, A, (uint64_t)M, (uint64_t)kblocks, (uint64_t)lda, GD_ROWS, (uint32_t)gr) != KCH_OK ||
      kch_make_tensor_map_katoms_bf16(&mw, W, (uint64_t)N, (uint64_t)kblocks, (uint64_t)ldw, BN, (uint32_t)gr) != KCH_OK)
    return GD_UNSUPPORTED;                                // the driver refused the view: the caller falls back
  unsigned int* status = kch_status_device_ptr();
  KCH_REQUIRE(status != nullptr, "kch_linear: cannot resolve the device status word");
  const int vec_ok = (ldc % 4 == 0) && (((uintptr_t)C & 7) == 0) && (!R || ((ldr % 4 == 0) && (((uintptr_t)R & 7) == 0)));
  KCH_CUDA_OK(cudaFuncSetAttribute(gemm_decode_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ksplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3((unsigned)(tiles * ksplit)); cfg.blockDim = dim3(GD_THREADS); cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = s; cfg.attrs = attr; cfg.numAttrs = ksplit > 1 ? 1 : 0;
  KCH_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_decode_kernel<BN>, ma, mw, (bf16*)C, (const bf16*)R, M, N, kblocks, kper, ldc, ldr,
                                 vec_ok, ep, ksplit, gr, ng, status));
  kch_note_launch(1);
  return KCH_OK;
}

// KCH_OK when launched; GD_UNSUPPORTED (-100) when this shape belongs to the general kernel (the caller goes on).
int kch_linear_decode_tc5(const void* A, const void* W, void* C, const void* R, int64_t M, int N, int K, int64_t lda,
                          int64_t ldw, int64_t ldc, int64_t ldr, const kch_epilogue* e, void* stream) {
  static const bool off = [] { const char* v = getenv("KCH_GEMM_DECODE"); return v && v[0] == '0'; }();
  if (off || M < 1 || M > GD_ROWS || N < 8 || K < GD_BK || (K % GD_BK) != 0) return GD_UNSUPPORTED;
  if ((lda % 8) || (ldw % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return GD_UNSUPPORTED;
  GdEpilogue ep = {};
  bool l2 = false;
  if (e && e->n_segments) {
    if (e->n_segments > 8) return GD_UNSUPPORTED;
    ep.nseg = e->n_segments;
    for (int i = 0; i < e->n_segments; ++i) {
      ep.seg_end[i] = e->seg_end[i]; ep.seg_act[i] = e->seg_act[i]; ep.seg_param[i] = e->seg_param[i];
      l2 = l2 || e->seg_act[i] == KCH_ACT_SILU_L2NORM;
    }
  }
  cudaStream_t s = kch_stream(stream);
  if (l2) return launch_gd<128>(A, W, C, R, (int)M, N, K, lda, ldw, ldc, ldr, ep, s);
  static const int bn = [] { const char* v = getenv("KCH_GD_BN"); return v ? atoi(v) : 32; }();
  if (bn == 128) return launch_gd<128>(A, W, C, R, (int)M, N, K, lda, ldw, ldc, ldr, ep, s);
  if (bn == 64) return launch_gd<64>(A, W, C, R, (int)M, N, K, lda, ldw, ldc, ldr, ep, s);
  return launch_gd<32>(A, W, C, R, (int)M, N, K, lda, ldw, ldc, ldr, ep, s);
}
