// Joint-softmax MQA core of CSA / HCA prefill on the fifth-generation tensor cores (tcgen05) for the production
// geometry (c = 128, up to 16 heads, bf16, cosine scoring): same mathematics and entry list as attn_mma_kernel
// (naive_csa / naive_hca attention core, ops_csa.py / ops_hca.py).
//
// Every query has its own entry list (selected compressed rows or the visible prefix, then window rows), so queries
// cannot share the key operand; the gathered KEYS are the 128 rows of the MMA instead and the 16 heads its N:
//   S^T [128 keys x 16 heads] = X [128 x 128] . Q^T            8 instructions (K = 16 each) per 128-key tile
//   O^T [128 dims x 16 heads] += X^T [128 dims x keys] . P^T   8 instructions per tile; X is read in place as an
//                                                              MN-major operand (values are the keys)
// One persistent CTA per SM, 480 threads:
//   warps 0..7   : softmax + epilogue — tcgen05.ld of an S^T tile (a thread owns a key and 8 of the 16 heads),
//                  p = exp(s scale - shift_h) with the fixed shift max(|scale|, sink_h), p = 0 for invalid entries,
//                  bf16 P^T operand tile to shared memory; the row sums and O^T / l -> global one tile later
//   warp 8       : tensor-memory allocation; one lane issues the S^T products
//   warp 9       : one lane issues the P.X products
//   warp 10      : loads and normalises the next query's 16 x 128 rows into a K-major operand tile
//   warps 11..14 : gather — 16-byte cp.async of the entry rows into a ring of six 128-row tiles in the operand layout
//                  (two 64-channel panels, 128-byte swizzle), zero fill and a validity mask for invalid entries
// A ring stage owns its S^T columns and its P^T tile, so one barrier (the P.X commit) frees all three.
//
// Status: opt-in.  KCH_ATTEND=l uses the cp.async gather described above, KCH_ATTEND=t replaces warps 11..14 by one
// warp that issues copy-engine row gathers (cp.async.bulk.tensor ... tile::gather4: four 128-byte row pieces per
// instruction, swizzled by the engine, zero fill for invalid rows).  Results match attn_mma_kernel to one bf16
// rounding.  At the benchmark size (B=4, T=32768) the mma.sync kernel measures 7.0 ms (CSA, 1024 + 128 entries per
// query) and 2.3 ms (HCA); this kernel 9.5 / 5.4 ms with the cp.async gather and 24.9 / 6.9 ms with the row gather.
// The tensor products take about 430 cycles per 128-key tile; the cp.async gather of the tile takes 1300-2500 cycles
// on four warps (the LSU path moves about 25 bytes per clock and SM in both kernels), the copy engine about 90
// cycles per four-row instruction (5800 per tile), and the per-query epilogue about 2000.  The core is bound by the
// gather, not by the tensor pipe.
// Every mbarrier wait is bounded, records a status code and leaves the loops.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "mma_utils.cuh"

#define AT_KT 128
#define AT_NSTG 6
#define AT_THREADS 480
#define AT_SPIN (1u << 24)
#define AT_TILE_BYTES (AT_KT * 256)

struct AttnTcArgs {
  const bf16* q; int64_t q_ld;
  int B, T, nh;
  const bf16* comp; int64_t comp_batch_rows; int n_comp;
  const int32_t* sel; int topk;
  int m; int64_t t0; int nvis_fixed;
  const bf16* win; int64_t win_ld; int64_t win_batch_rows; int win_size; int win_t0;
  const void* sink; int sink_dtype;
  float scale;
  bf16* out;
  unsigned int* status;
};

// shared-memory map
#define AT_OFF_RING 0
#define AT_OFF_Q (AT_NSTG * AT_TILE_BYTES)                 // 2 x [2 panels][16][64] bf16
#define AT_OFF_P (AT_OFF_Q + 2 * 4096)                     // AT_NSTG x [2 panels][16][64] bf16
#define AT_OFF_MASK (AT_OFF_P + AT_NSTG * 4096)              // AT_NSTG x 4 words
#define AT_OFF_RED (AT_OFF_MASK + AT_NSTG * 16)            // 2 x 8 warps x 8 floats
#define AT_OFF_BARS (AT_OFF_RED + 2 * 8 * 8 * 4)
#define AT_NBARS (4 * AT_NSTG + 9)
#define AT_TOTAL (AT_OFF_BARS + AT_NBARS * 8 + 16)

__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void at_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr_u32(bar)) : "memory");
}
__device__ __forceinline__ void at_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void at_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void at_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 128-byte rows under the 128-byte swizzle, 8-row groups 1024 bytes apart.  K-major: rows are M / N, the 64 elements
// of a row the contraction index.  MN-major: rows are the contraction index, 64-element panels `lbo` bytes apart.
__device__ __forceinline__ uint64_t at_desc(uint32_t saddr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void at_cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// entry-list geometry of query bt (as in attn_mma_kernel)
struct AtQuery {
  int nvis, ns, nw, E, ntiles;
  int b, wrow0, nsp;          // batch, first window row, ns rounded up to the gather granularity
  const int32_t* selrow;
  const bf16* comp_b;
  const bf16* win_b;
};
// PAD = 4: the TMA row gather moves four entries per instruction, so the selected region is padded with invalid
// entries to a multiple of four and the window region starts on a four-entry boundary
template <int PAD>
__device__ __forceinline__ AtQuery at_query(const AttnTcArgs& a, int64_t bt) {
  AtQuery qy;
  const int t = (int)(bt % a.T), b = (int)(bt / a.T);
  int64_t nv64 = a.nvis_fixed >= 0 ? a.nvis_fixed : (a.m > 0 ? (a.t0 + t + 1) / a.m : a.n_comp);
  qy.nvis = (int)(nv64 < a.n_comp ? nv64 : a.n_comp);
  qy.ns = a.sel ? a.topk : qy.nvis;
  qy.nw = 0;
  int wrow0 = 0;
  if (a.win_size > 0 && a.win) { const int tw = t + a.win_t0; int lo = tw - a.win_size + 1; if (lo < 0) lo = 0; qy.nw = tw - lo + 1; wrow0 = lo; }
  qy.b = b; qy.wrow0 = wrow0;
  qy.nsp = (qy.ns + PAD - 1) / PAD * PAD;
  qy.E = qy.nsp + qy.nw;
  qy.ntiles = qy.E > 0 ? (qy.E + AT_KT - 1) / AT_KT : 1;     // a query without entries still runs one (empty) tile
  qy.selrow = a.sel ? a.sel + bt * a.topk : nullptr;
  qy.comp_b = a.comp ? a.comp + (int64_t)b * a.comp_batch_rows * 128 : nullptr;
  qy.win_b = a.win ? a.win + ((int64_t)b * a.win_batch_rows + wrow0) * a.win_ld : nullptr;
  return qy;
}
template <int PAD>
__device__ __forceinline__ int at_ntiles(const AttnTcArgs& a, int64_t bt) {
  const int t = (int)(bt % a.T);
  int64_t nv64 = a.nvis_fixed >= 0 ? a.nvis_fixed : (a.m > 0 ? (a.t0 + t + 1) / a.m : a.n_comp);
  const int nvis = (int)(nv64 < a.n_comp ? nv64 : a.n_comp);
  const int ns = a.sel ? a.topk : nvis;
  int nw = 0;
  if (a.win_size > 0 && a.win) { const int tw = t + a.win_t0; int lo = tw - a.win_size + 1; if (lo < 0) lo = 0; nw = tw - lo + 1; }
  const int E = (ns + PAD - 1) / PAD * PAD + nw;
  return E > 0 ? (E + AT_KT - 1) / AT_KT : 1;
}

// row gather by the copy engine: rows r0..r3 of a [rows][128] bf16 tensor, 64 columns from `col`, land as four
// consecutive 128-byte rows at `dst` (swizzled by the engine); rows outside the tensor read as zeros
__device__ __forceinline__ void at_gather4(uint32_t dst, const CUtensorMap* map, int col, int r0, int r1, int r2, int r3,
                                           uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(smem_addr_u32(bar)), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}

template <bool TMAG>
__global__ void __launch_bounds__(AT_THREADS, 1) attn_tc5_kernel(AttnTcArgs a, const __grid_constant__ CUtensorMap map_comp,
                                                                  const __grid_constant__ CUtensorMap map_win) {
  constexpr int PAD = TMAG ? 4 : 1;
  extern __shared__ uint8_t at_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>(((uintptr_t)at_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + AT_OFF_BARS);
  uint64_t* kfull = bars;                        // [AT_NSTG] gathered tile landed (4 producer warps)
  uint64_t* sfull = kfull + AT_NSTG;             // [AT_NSTG] S^T tile in tensor memory
  uint64_t* pready = sfull + AT_NSTG;            // [AT_NSTG] P^T operand tile written (8 softmax warps)
  uint64_t* done = pready + AT_NSTG;             // [AT_NSTG] P.X has read the stage: key tile, S^T columns, P^T tile free
  uint64_t* qfull = done + AT_NSTG;              // [2]
  uint64_t* qempty = qfull + 2;                  // [2]
  uint64_t* ofull = qempty + 2;                  // [2]
  uint64_t* oempty = ofull + 2;                  // [2]
  uint64_t* redbar = oempty + 2;                 // row sums of a query are in shared memory (8 softmax warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + AT_NBARS);
  uint32_t* maskbuf = reinterpret_cast<uint32_t*>(sm + AT_OFF_MASK);
  float* red = reinterpret_cast<float*>(sm + AT_OFF_RED);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nq = (int64_t)a.B * a.T;
  constexpr uint32_t TMEM_COLS = 128;            // S^T stages 6 x 16 | O^T 2 x 16

  if (threadIdx.x == 0) {
    for (int s = 0; s < AT_NSTG; ++s) { mbarrier_init(&kfull[s], TMAG ? 1 : 4); mbarrier_init(&sfull[s], 1); mbarrier_init(&pready[s], 8); mbarrier_init(&done[s], 1); }
    for (int i = 0; i < 2; ++i) { mbarrier_init(&qfull[i], 1); mbarrier_init(&qempty[i], 1); mbarrier_init(&ofull[i], 1); mbarrier_init(&oempty[i], 8); }
    mbarrier_init(redbar, 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  at_fence_before();
  __syncthreads();
  at_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + AT_NSTG * 16;

  if (warp >= 11) {
   if constexpr (TMAG) {
    // ------------------------------ gather by the copy engine (one warp) ------------------------------
    // A lane owns four consecutive entries of every tile: it turns them into row numbers of the compressed-row
    // tensor or of the window tensor and issues one four-row gather per 64-channel panel.  Invalid entries name
    // a row outside the tensor, which the engine fills with zeros.
    if (warp == 11) {
      constexpr int OOB = 0x3FFFFFF0;
      int64_t bt = blockIdx.x;
      int tile = 0;
      bool have = bt < nq;
      AtQuery qy = {};
      auto load_raw4 = [&](const AtQuery& q_, int tile_) -> int4 {
        const int e0 = tile_ * AT_KT + 4 * lane;
        if (q_.selrow && e0 < q_.ns) return *reinterpret_cast<const int4*>(q_.selrow + e0);
        return make_int4(e0, e0 + 1, e0 + 2, e0 + 3);
      };
      int4 raw = make_int4(0, 0, 0, 0);
      if (have) { qy = at_query<PAD>(a, bt); raw = load_raw4(qy, 0); }
      uint32_t g = 0;
      while (have) {
        // successor position and its index load first: the load's latency hides behind the wait below
        int64_t bt2 = bt;
        int tile2 = tile + 1;
        AtQuery qy2 = qy;
        bool have2 = true;
        if (tile2 == qy.ntiles) {
          tile2 = 0; bt2 = bt + gridDim.x; have2 = bt2 < nq;
          if (have2) qy2 = at_query<PAD>(a, bt2);
        }
        const int4 raw2 = have2 ? load_raw4(qy2, tile2) : make_int4(0, 0, 0, 0);
        const uint32_t s = g % AT_NSTG, kph = (g / AT_NSTG) & 1;
        const int e0 = tile * AT_KT + 4 * lane;
        const bool in_sel = e0 < qy.nsp;
        int rows[4];
        uint32_t vbits = 0;
        const int rr[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int e = e0 + j;
          int row = OOB;
          if (in_sel) {
            if (e < qy.ns && rr[j] >= 0 && rr[j] < qy.nvis) row = (int)((int64_t)qy.b * a.comp_batch_rows + rr[j]);
          } else {
            const int w = e - qy.nsp;
            if (w < qy.nw) row = (int)((int64_t)qy.b * a.win_batch_rows + qy.wrow0 + w);
          }
          rows[j] = row;
          vbits |= (row != OOB ? 1u : 0u) << j;
        }
        // validity mask of the tile's 128 rows: word w covers rows 32 w .. 32 w + 31 = lanes 8 w .. 8 w + 7
        uint32_t mw[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) mw[w] = __reduce_or_sync(0xffffffffu, (lane >> 3) == w ? vbits << (4 * (lane & 7)) : 0u);
        if (!mbarrier_wait_bounded(&done[s], kph ^ 1, 61, AT_SPIN, a.status)) break;
        if (lane == 0) {
#pragma unroll
          for (int w = 0; w < 4; ++w) maskbuf[s * 4 + w] = mw[w];
          mbarrier_expect_tx(&kfull[s], AT_TILE_BYTES);
        }
        __syncwarp();
        const uint32_t dst = smem_addr_u32(sm + AT_OFF_RING + (size_t)s * AT_TILE_BYTES) + (uint32_t)lane * 512u;
        const CUtensorMap* mp = in_sel ? &map_comp : &map_win;
        at_gather4(dst, mp, 0, rows[0], rows[1], rows[2], rows[3], &kfull[s]);
        at_gather4(dst + 16384u, mp, 64, rows[0], rows[1], rows[2], rows[3], &kfull[s]);
        ++g;
        bt = bt2; tile = tile2; qy = qy2; have = have2; raw = raw2;
      }
    }
   } else {
    // ------------------------------ gather producers ------------------------------
    // A tile is announced (kfull) when its copies have landed, which this warp learns from cp.async.wait_group.
    // The warp never blocks on a free ring stage while it has unannounced tiles in flight: it issues while stages
    // are free (up to MAXF tiles in flight), otherwise it waits for its oldest tile to land and announces it.
    const int pw = warp - 11;                                  // rows 32 pw .. 32 pw + 31 of every tile
    constexpr uint32_t MAXF = 4;
    int64_t bt = blockIdx.x;
    int tile = 0;
    bool have = bt < nq;
    AtQuery qy = {};
    // index of this lane's entry in the selection list (loaded one tile ahead of its use)
    auto load_raw = [&](const AtQuery& q_, int tile_) -> int {
      const int e = tile_ * AT_KT + 32 * pw + lane;
      return (q_.selrow && e < q_.ns) ? q_.selrow[e] : e;
    };
    auto entry_ptr = [&](const AtQuery& q_, int tile_, int raw_) -> const bf16* {
      const int e = tile_ * AT_KT + 32 * pw + lane;
      if (e >= q_.E) return nullptr;
      if (e < q_.ns) return (raw_ >= 0 && raw_ < q_.nvis) ? q_.comp_b + (int64_t)raw_ * 128 : nullptr;
      return q_.win_b + (int64_t)(e - q_.nsp) * a.win_ld;
    };
    int raw = 0;
    if (have) { qy = at_query<PAD>(a, bt); raw = load_raw(qy, 0); }
    uint32_t issued = 0, announced = 0;
    while (have || announced < issued) {
      const uint32_t s = issued % AT_NSTG, kph = (issued / AT_NSTG) & 1;
      bool can = false;
      if (have && issued - announced < MAXF) {
        uint32_t tst = 0;
        if (lane == 0) {
          asm volatile(
              "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
              : "=r"(tst) : "r"(smem_addr_u32(&done[s])), "r"(kph ^ 1) : "memory");
        }
        can = __shfl_sync(0xffffffffu, tst, 0) != 0;
      }
      if (can) {
        // successor position and its index load first: the load's latency hides behind this tile's copies
        int64_t bt2 = bt;
        int tile2 = tile + 1;
        AtQuery qy2 = qy;
        bool have2 = true;
        if (tile2 == qy.ntiles) {
          tile2 = 0; bt2 = bt + gridDim.x; have2 = bt2 < nq;
          if (have2) qy2 = at_query<PAD>(a, bt2);
        }
        const int raw2 = have2 ? load_raw(qy2, tile2) : 0;
        const bf16* p = entry_ptr(qy, tile, raw);
        const uint32_t vm = __ballot_sync(0xffffffffu, p != nullptr);
        if (lane == 0) maskbuf[s * 4 + pw] = vm;
        const uint32_t dst0 = smem_addr_u32(sm + AT_OFF_RING + (size_t)s * AT_TILE_BYTES);
        const int ch = lane & 15;
        const uint32_t dcol = (uint32_t)(ch >> 3) * 16384u;
#pragma unroll
        for (int it = 0; it < 16; ++it) {
          const int rl = 2 * it + (lane >> 4);                 // row of this warp's 32
          const bf16* rp = (const bf16*)__shfl_sync(0xffffffffu, (unsigned long long)p, rl);
          const int r = 32 * pw + rl;
          at_cp_async16(dst0 + dcol + swz<128>(r, ch & 7), rp ? (const void*)(rp + ch * 8) : (const void*)a.q, rp ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        ++issued;
        bt = bt2; tile = tile2; qy = qy2; have = have2; raw = raw2;
      } else if (announced < issued) {
        switch (issued - announced - 1) {                      // groups that may stay in flight
          case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
          case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
          case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
          default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        }
        at_fence_async_smem();
        __syncwarp();
        if (lane == 0) mbarrier_arrive(&kfull[announced % AT_NSTG]);
        ++announced;
      } else {
        // nothing in flight and the ring is full: wait for a stage
        if (!mbarrier_wait_bounded(&done[s], kph ^ 1, 61, AT_SPIN, a.status)) break;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
   }
  } else if (warp == 10) {
    // ------------------------------ query loader ------------------------------
    // the rows of the next query are in flight while the current one is normalised
    uint32_t qi = 0;
    uint2 nxt[16];
    auto load_rows = [&](int64_t bt_, uint2 (&dst)[16]) {
      const bf16* qrow = a.q + bt_ * a.q_ld;
#pragma unroll
      for (int h = 0; h < 16; ++h) dst[h] = h < a.nh ? *reinterpret_cast<const uint2*>(qrow + h * 128 + lane * 4) : make_uint2(0u, 0u);
    };
    if ((int64_t)blockIdx.x < nq) load_rows(blockIdx.x, nxt);
    for (int64_t bt = blockIdx.x; bt < nq; bt += gridDim.x, ++qi) {
      const uint32_t qb = qi & 1, qph = (qi >> 1) & 1;
      uint8_t* qt = sm + AT_OFF_Q + qb * 4096;
      uint2 raw[16];
#pragma unroll
      for (int h = 0; h < 16; ++h) raw[h] = nxt[h];
      if (bt + gridDim.x < nq) load_rows(bt + gridDim.x, nxt);
      float ss[16];
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        const float v0 = __uint_as_float(raw[h].x << 16), v1 = __uint_as_float(raw[h].x & 0xFFFF0000u);
        const float v2 = __uint_as_float(raw[h].y << 16), v3 = __uint_as_float(raw[h].y & 0xFFFF0000u);
        ss[h] = v0 * v0 + v1 * v1 + v2 * v2 + v3 * v3;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int h = 0; h < 16; ++h) ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], o);
      }
      if (!mbarrier_wait_bounded(&qempty[qb], qph ^ 1, 62, AT_SPIN, a.status)) break;
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        const float nrm = fmaxf(sqrtf(ss[h]), 1e-12f);
        const float v0 = __uint_as_float(raw[h].x << 16), v1 = __uint_as_float(raw[h].x & 0xFFFF0000u);
        const float v2 = __uint_as_float(raw[h].y << 16), v3 = __uint_as_float(raw[h].y & 0xFFFF0000u);
        uint2 o;
        o.x = pack2_bf16(v0 / nrm, v1 / nrm);
        o.y = pack2_bf16(v2 / nrm, v3 / nrm);
        const int d = 4 * lane;                                // channels d .. d + 3
        *reinterpret_cast<uint2*>(qt + (d >> 6) * 2048 + swz<128>(h, (d & 63) >> 3) + (d & 7) * 2) = o;
      }
      at_fence_async_smem();
      __syncwarp();
      if (lane == 0) mbarrier_arrive(&qfull[qb]);
    }
  } else if (warp == 8) {
    // ------------------------------ S^T products: X . Q^T ------------------------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint64_t kd0 = at_desc(smem_addr_u32(sm + AT_OFF_RING), 16), qd0 = at_desc(smem_addr_u32(sm + AT_OFF_Q), 16);
      uint32_t g = 0, qi = 0;
      bool ok = true;
      for (int64_t bt = blockIdx.x; bt < nq && ok; bt += gridDim.x, ++qi) {
        const int ntiles = at_ntiles<PAD>(a, bt);
        const uint32_t qb = qi & 1;
        if (!mbarrier_wait_bounded(&qfull[qb], (qi >> 1) & 1, 63, AT_SPIN, a.status)) break;
        const uint64_t qd = qd0 + (uint64_t)(qb * (4096 >> 4));
        for (int tile = 0; tile < ntiles; ++tile, ++g) {
          const uint32_t s = g % AT_NSTG, kph = (g / AT_NSTG) & 1;
          // the tile has landed; its stage (key tile, S^T columns, P^T tile) was released by the P.X of its
          // previous occupant before the gather started
          if (!mbarrier_wait_bounded(&kfull[s], kph, 65, AT_SPIN, a.status)) { ok = false; break; }
          at_fence_after();
          const uint64_t kd = kd0 + (uint64_t)(s * (AT_TILE_BYTES >> 4));
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            at_mma(tS + s * 16, kd + (uint64_t)((ks >> 2) * (16384 >> 4) + 2 * (ks & 3)),
                   qd + (uint64_t)((ks >> 2) * (2048 >> 4) + 2 * (ks & 3)), idesc, ks ? 1u : 0u);
          at_commit(&sfull[s]);
        }
        if (ok) at_commit(&qempty[qb]);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ O^T products: X^T . P^T ------------------------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint64_t kd0 = at_desc(smem_addr_u32(sm + AT_OFF_RING), 16384), pd0 = at_desc(smem_addr_u32(sm + AT_OFF_P), 16);
      uint32_t g = 0, qi = 0;
      bool ok = true;
      for (int64_t bt = blockIdx.x; bt < nq && ok; bt += gridDim.x, ++qi) {
        const int ntiles = at_ntiles<PAD>(a, bt);
        const uint32_t ob = qi & 1;
        if (!mbarrier_wait_bounded(&oempty[ob], ((qi >> 1) & 1) ^ 1, 66, AT_SPIN, a.status)) break;
        for (int tile = 0; tile < ntiles; ++tile, ++g) {
          const uint32_t s = g % AT_NSTG, kph = (g / AT_NSTG) & 1;
          if (!mbarrier_wait_bounded(&pready[s], kph, 67, AT_SPIN, a.status)) { ok = false; break; }
          at_fence_after();
          const uint64_t kd = kd0 + (uint64_t)(s * (AT_TILE_BYTES >> 4)), pd = pd0 + (uint64_t)(s * (4096 >> 4));
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            at_mma(tO + ob * 16, kd + (uint64_t)(ks * (2048 >> 4)),
                   pd + (uint64_t)((ks >> 2) * (2048 >> 4) + 2 * (ks & 3)), idesc, (tile | ks) ? 1u : 0u);
          at_commit(&done[s]);
        }
        if (ok) at_commit(&ofull[ob]);
      }
    }
  } else {
    // ------------------------------ softmax + epilogue (warps 0..7) ------------------------------
    const int quarter = warp & 3, hh = warp >> 2;              // tensor-memory lane quarter; heads 8 hh .. 8 hh + 7
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int row = quarter * 32 + lane;                       // key row of an S^T tile, channel of O^T
    const float ascale = fabsf(a.scale);
    float shift[8], sinkv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int h = 8 * hh + j;
      const float sk = (a.sink && h < a.nh) ? ld_any(a.sink, h, a.sink_dtype) : -INFINITY;
      shift[j] = fmaxf(ascale, sk);
      sinkv[j] = (a.sink && h < a.nh) ? __expf(sk - shift[j]) : 0.f;     // the sink's term of the denominator
    }
    uint32_t g = 0, qi = 0;
    bool ok = true;
    // O^T / l of a finished query goes out while the first tile of the next one is in the tensor pipe
    int64_t pend_bt = 0;
    uint32_t pend_qi = 0;
    bool pend = false;
    auto flush = [&]() -> bool {
      const float* rq = red + (pend_qi & 1) * 64 + hh * 32;    // [quarter][8] partial sums of this head half
      if (!mbarrier_wait_bounded(redbar, pend_qi & 1, 70, AT_SPIN, a.status)) return false;
      const uint32_t ob = pend_qi & 1, oph = (pend_qi >> 1) & 1;
      if (!mbarrier_wait_bounded(&ofull[ob], oph, 69, AT_SPIN, a.status)) return false;
      at_fence_after();
      uint32_t r[8];
      at_ld8(tO + lane_base + ob * 16 + 8 * hh, r);
      at_wait_ld();
      at_fence_before();
      __syncwarp();
      if (lane == 0) mbarrier_arrive(&oempty[ob]);
      bf16* orow = a.out + pend_bt * ((int64_t)a.nh * 128);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int h = 8 * hh + j;
        if (h < a.nh) {
          const float lt = rq[j] + rq[8 + j] + rq[16 + j] + rq[24 + j] + sinkv[j];
          const float inv = lt > 0.f ? __fdividef(1.f, lt) : 0.f;
          orow[h * 128 + row] = __float2bfloat16_rn(__uint_as_float(r[j]) * inv);
        }
      }
      return true;
    };
    for (int64_t bt = blockIdx.x; bt < nq && ok; bt += gridDim.x, ++qi) {
      const int ntiles = at_ntiles<PAD>(a, bt);
      float l[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) l[j] = 0.f;
      for (int tile = 0; tile < ntiles; ++tile, ++g) {
        const uint32_t s = g % AT_NSTG, kph = (g / AT_NSTG) & 1;
        if (!mbarrier_wait_bounded(&sfull[s], kph, 68, AT_SPIN, a.status)) { ok = false; break; }
        at_fence_after();
        uint32_t r[8];
        at_ld8(tS + lane_base + s * 16 + 8 * hh, r);
        at_wait_ld();
        const bool valid = (maskbuf[s * 4 + quarter] >> lane) & 1u;
        uint8_t* pt = sm + AT_OFF_P + s * 4096 + (row >> 6) * 2048 + (row & 7) * 2;
        const int chunk = (row & 63) >> 3;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float p = valid ? __expf(__uint_as_float(r[j]) * a.scale - shift[j]) : 0.f;
          l[j] += p;
          *reinterpret_cast<bf16*>(pt + swz<128>(8 * hh + j, chunk)) = __float2bfloat16_rn(p);
        }
        at_fence_async_smem();
        at_fence_before();
        __syncwarp();
        if (lane == 0) mbarrier_arrive(&pready[s]);
        if (tile == 0 && pend) {
          if (!flush()) { ok = false; break; }
          pend = false;
        }
      }
      if (!ok) break;
      // ---- row sums of this query: per warp here, over the four quarters in flush() --------------------------------
      float* rq = red + (qi & 1) * 64 + hh * 32 + quarter * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = warp_sum(l[j]);
        if (lane == 0) rq[j] = v;
      }
      __syncwarp();
      if (lane == 0) mbarrier_arrive(redbar);
      pend = true; pend_bt = bt; pend_qi = qi;
    }
    if (ok && pend) flush();
  }
  at_fence_before();
  __syncthreads();
  if (warp == 8) {
    at_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host ----------------------------------------------------------------------------------------------------
int kch_make_tensor_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                                uint32_t box_rows, uint32_t box_cols);   // gemm_tcgen05.cu

// KCH_ATTEND=t: tcgen05 core with the copy-engine row gather; KCH_ATTEND=l: the same core with the cp.async gather
static int attend_tc5_mode() {
  static const int mode = [] { const char* e = getenv("KCH_ATTEND"); return (e && e[0] == 't') ? 2 : (e && e[0] == 'l') ? 1 : 0; }();
  return mode;
}
bool kch_attend_tc5_enabled() { return attend_tc5_mode() != 0; }

int kch_attend_tc5(const kch_attend_args* p, void* stream) {
  AttnTcArgs a;
  a.q = (const bf16*)p->q; a.q_ld = p->q_ld;
  a.B = p->B; a.T = p->T; a.nh = p->nh;
  a.comp = (const bf16*)p->comp; a.comp_batch_rows = p->comp_batch_rows; a.n_comp = p->comp ? p->n_comp : 0;
  a.sel = p->sel_indices; a.topk = p->sel_indices ? p->topk : 0;
  a.m = p->m; a.t0 = p->t0; a.nvis_fixed = p->n_visible;
  const bool has_win = p->win && p->sliding_window > 0;
  a.win = has_win ? (const bf16*)p->win : nullptr; a.win_ld = p->win_ld; a.win_batch_rows = p->win_batch_rows;
  a.win_size = has_win ? p->sliding_window : 0; a.win_t0 = p->win_t0;
  a.sink = p->sink; a.sink_dtype = p->sink_dtype; a.scale = p->scale; a.out = (bf16*)p->out;
  a.status = kch_status_device_ptr();
  KCH_REQUIRE(a.status != nullptr, "kch_attend: cannot resolve the device status word");
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    KCH_CUDA_OK(cudaGetDevice(&dev));
    KCH_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const int64_t nq = (int64_t)p->B * p->T;
  if (nq == 0) return KCH_OK;
  const int grid = (int)(nq < sms ? nq : sms);
  const int smem = AT_TOTAL + 1024;
  // the row gather needs four-entry groups of the selection list to be 16-byte aligned and row numbers within int32
  const bool sel_ok = !a.sel || ((a.topk % 4) == 0 && (((uintptr_t)a.sel & 15) == 0));
  const bool rows_ok = (int64_t)a.B * a.comp_batch_rows < 0x3FFFFFF0LL && (int64_t)a.B * a.win_batch_rows < 0x3FFFFFF0LL;
  CUtensorMap mc, mw;
  if (attend_tc5_mode() == 2 && sel_ok && rows_ok && (a.comp || a.win)) {
    // one [rows][128] tensor per source, box 1 x 64: a gather moves four such boxes
    const bf16* cb = a.comp ? a.comp : a.win;
    const uint64_t crows = a.comp ? (uint64_t)a.B * a.comp_batch_rows : 1, cld = a.comp ? 128 : (uint64_t)a.win_ld;
    const bf16* wb = a.win ? a.win : a.comp;
    const uint64_t wrows = a.win ? (uint64_t)a.B * a.win_batch_rows : 1, wld = a.win ? (uint64_t)a.win_ld : 128;
    int rc = kch_make_tensor_map_2d_bf16(&mc, cb, crows, 128, cld, 1, 64);
    if (rc) return rc;
    rc = kch_make_tensor_map_2d_bf16(&mw, wb, wrows, 128, wld, 1, 64);
    if (rc) return rc;
    KCH_CUDA_OK(cudaFuncSetAttribute(attn_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attn_tc5_kernel<true><<<grid, AT_THREADS, smem, kch_stream(stream)>>>(a, mc, mw);
  } else {
    memset(&mc, 0, sizeof(mc));
    memset(&mw, 0, sizeof(mw));
    KCH_CUDA_OK(cudaFuncSetAttribute(attn_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attn_tc5_kernel<false><<<grid, AT_THREADS, smem, kch_stream(stream)>>>(a, mc, mw);
  }
  KCH_LAUNCH_OK();
  return KCH_OK;
}
