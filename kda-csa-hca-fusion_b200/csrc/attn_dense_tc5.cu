// Dense attention core on tcgen05: every visible compressed block plus the sliding window, no selection list
// (naive_hca, ops_hca.py:139-192: joint softmax over [all visible compressed entries | window] with the sink logit in the
// denominator; single KV head, the attended row is key and value at once).
//
// Nothing is gathered here, so the products can be real tiles: a CTA takes 8 consecutive queries of a sequence,
// 8 x 16 heads = the 128 rows of the MMA, and walks the entries they can see in tiles of 64 keys:
//   * Q tile [128 rows x 128 channels] by two TMA copies through a 3-D view {channel, head, token} of the projection
//     output (un-normalised bf16 as stored; 1 / ||q|| is applied to the score row in fp32 -- closer to the reference's
//     fp32 normalisation than a rounded normalised copy);
//   * key tiles [64 x 128] by TMA (128-byte swizzle, no multicast) through a 2-stage ring: ceil(ns / 64) tiles of
//     compressed rows, then the window rows of the 8 queries (at most 135) in tiles of their own;
//   * S = Q K^T (M = 128, N = 64, K = 128) into one of two tensor-memory buffers; four softmax warps (one row per
//     thread) read it, apply the per-query causal / window rule and exp(s * scale / ||q|| - shift) with the fixed shift
//     max(|scale|, sink_h) (|s| <= |scale| for unit rows, so partial sums simply add), write P as a bf16 K-major operand
//     tile and keep the row sum;
//   * O += P V (M = 128, N = 128, K = 64) with the SAME shared-memory key tile read as an MN-major B operand;
//   * the epilogue divides by the row sum (+ the sink term) and stores 256 contiguous bytes per (query, head).
// Every wait is bounded (status word, see kch_device_status).
#include <cuda.h>
#include <math.h>
#include <stdlib.h>

#include "kch_common.cuh"
#include "tc5_utils.cuh"

#define DT_C 128
#define DT_Q 8                         // queries per CTA
#define DT_KT 64                       // keys per tile
#define DT_KSTAGES 2
#define DT_THREADS 192
#define DT_SPIN (1u << 24)
#define DT_STATUS 0x6D04

struct DtArgs {
  int B, T, nh;
  int n_comp, m, nvis_fixed;
  int64_t t0;
  int64_t comp_batch_rows, win_batch_rows;
  int win_size, win_t0;
  int has_comp, has_win;
  const void* sink; int sink_dtype;
  float scale;
  bf16* out;
  unsigned int* status;
};

struct DtSmem {
  alignas(1024) bf16 q[2][128 * 64];                 // two 64-channel panels of [128 rows][64]
  alignas(1024) bf16 k[DT_KSTAGES][2][DT_KT * 64];   // per stage: two 64-channel panels of [64 keys][64]
  alignas(1024) bf16 p[2][128 * DT_KT];              // P tiles [128 rows][64 keys]
  alignas(8) uint64_t q_full;
  uint64_t k_full[DT_KSTAGES], k_empty[DT_KSTAGES];
  uint64_t s_full[2], p_full[2], pv_done[2];
  uint64_t o_full;
  uint32_t tmem;
};

__device__ __forceinline__ void dt_tma_load_3d(void* dst, const void* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_addr_u32(dst)), "l"(map), "r"(smem_addr_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__global__ void __launch_bounds__(DT_THREADS)
attn_dense_tc5_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap cmap,
                      const __grid_constant__ CUtensorMap wmap, DtArgs a) {
  extern __shared__ uint8_t dt_raw[];
  DtSmem& sm = *reinterpret_cast<DtSmem*>(((uintptr_t)dt_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_per_seq = (a.T + DT_Q - 1) / DT_Q;
  const int b = blockIdx.x / tiles_per_seq;
  const int tq0 = (blockIdx.x % tiles_per_seq) * DT_Q;
  const int t_last = min(tq0 + DT_Q, a.T) - 1;
  auto nvis_of = [&](int tt) -> int {
    int64_t nv64 = a.nvis_fixed >= 0 ? a.nvis_fixed : (a.m > 0 ? (a.t0 + tt + 1) / a.m : a.n_comp);
    return (int)(nv64 < a.n_comp ? nv64 : a.n_comp);
  };
  const int ns = a.has_comp ? nvis_of(t_last) : 0;                 // compressed rows the CTA walks: [0, ns)
  int nw = 0, wrow0 = 0;                                           // window rows the CTA walks: [wrow0, wrow0 + nw)
  if (a.has_win) { int lo = tq0 + a.win_t0 - a.win_size + 1; if (lo < 0) lo = 0; wrow0 = lo; nw = t_last + a.win_t0 - lo + 1; }
  const int nct = (ns + DT_KT - 1) / DT_KT, nwt = (nw + DT_KT - 1) / DT_KT;
  const int ntiles = nct + nwt;

  if (tid == 0) {
    mbarrier_init(&sm.q_full, 1);
    for (int s = 0; s < DT_KSTAGES; ++s) { mbarrier_init(&sm.k_full[s], 1); mbarrier_init(&sm.k_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbarrier_init(&sm.s_full[i], 1); mbarrier_init(&sm.p_full[i], 4); mbarrier_init(&sm.pv_done[i], 1); }
    mbarrier_init(&sm.o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr_u32(&sm.tmem)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem = sm.tmem;
  const uint32_t tS = tmem, tO = tmem + 128;                       // S buffers at columns 0 and 64, O at 128..255

  if (warp == 4) {
    // ------------------------------ producer: the query tile, then the key tiles -----------------------------------
    if (lane == 0) {
      mbarrier_expect_tx(&sm.q_full, 2 * 128 * 64 * 2);
      dt_tma_load_3d(sm.q[0], &qmap, 0, 0, b * a.T + tq0, &sm.q_full);
      dt_tma_load_3d(sm.q[1], &qmap, 64, 0, b * a.T + tq0, &sm.q_full);
      for (int i = 0; i < ntiles; ++i) {
        const int st = i % DT_KSTAGES;
        if (i >= DT_KSTAGES && !mbarrier_wait_bounded(&sm.k_empty[st], ((i / DT_KSTAGES) & 1) ^ 1, DT_STATUS, DT_SPIN, a.status)) break;
        mbarrier_expect_tx(&sm.k_full[st], 2 * DT_KT * 64 * 2);
        if (i < nct) {
          const int row = (int)((int64_t)b * a.comp_batch_rows) + i * DT_KT;
          t5_tma_load_2d(sm.k[st][0], &cmap, 0, row, &sm.k_full[st]);
          t5_tma_load_2d(sm.k[st][1], &cmap, 64, row, &sm.k_full[st]);
        } else {
          const int row = (int)((int64_t)b * a.win_batch_rows) + wrow0 + (i - nct) * DT_KT;
          t5_tma_load_2d(sm.k[st][0], &wmap, 0, row, &sm.k_full[st]);
          t5_tma_load_2d(sm.k[st][1], &wmap, 64, row, &sm.k_full[st]);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ----------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t id_s = t5_idesc(DT_KT), id_o = t5_idesc(128) | (1u << 16);
      bool ok = mbarrier_wait_bounded(&sm.q_full, 0, DT_STATUS, DT_SPIN, a.status);
      auto issue_pv = [&](int i) {             // O += P_i V_i; frees key stage and P buffer of tile i
        const int st = i % DT_KSTAGES, pb = i & 1;
        t5_fence_after();
        const uint32_t pa = smem_addr_u32(sm.p[pb]), kb = smem_addr_u32(sm.k[st][0]);
#pragma unroll
        for (int ks = 0; ks < DT_KT / 16; ++ks)
          t5_mma(tO, t5_desc(pa) + 2 * ks, t5_desc_mn(kb + (uint32_t)ks * 2048u, 8192u), id_o, (i | ks) ? 1u : 0u);
        t5_commit(&sm.k_empty[st]);
        t5_commit(&sm.pv_done[pb]);
      };
      for (int i = 0; i < ntiles && ok; ++i) {
        const int st = i % DT_KSTAGES;
        ok = mbarrier_wait_bounded(&sm.k_full[st], (i / DT_KSTAGES) & 1, DT_STATUS, DT_SPIN, a.status);
        if (!ok) break;
        t5_fence_after();
#pragma unroll
        for (int pan = 0; pan < 2; ++pan)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            t5_mma(tS + 64u * (i & 1), t5_desc(smem_addr_u32(sm.q[pan])) + 2 * ks, t5_desc(smem_addr_u32(sm.k[st][pan])) + 2 * ks,
                   id_s, (pan | ks) ? 1u : 0u);
        t5_commit(&sm.s_full[i & 1]);
        if (i >= 1) {
          ok = mbarrier_wait_bounded(&sm.p_full[(i - 1) & 1], ((i - 1) >> 1) & 1, DT_STATUS, DT_SPIN, a.status);
          if (ok) issue_pv(i - 1);
        }
      }
      if (ok && ntiles > 0) {
        ok = mbarrier_wait_bounded(&sm.p_full[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, DT_STATUS, DT_SPIN, a.status);
        if (ok) issue_pv(ntiles - 1);
      }
      if (ok) t5_commit(&sm.o_full);
    }
  } else {
    // ------------------------------ softmax + epilogue: one (query, head) row per thread -------------------------------
    const int r = warp * 32 + lane, qi = r >> 4, h = r & 15;
    const int t = tq0 + qi;
    const bool active = t < a.T && h < a.nh;
    const int nvis = (active && a.has_comp) ? nvis_of(t) : 0;
    const int tw = t + a.win_t0;
    const float ascale = fabsf(a.scale);
    float sink = -INFINITY;
    if (a.sink && h < a.nh) sink = ld_any(a.sink, h, a.sink_dtype);
    const float shift = fmaxf(ascale, sink);
    bool ok = mbarrier_wait_bounded(&sm.q_full, 0, DT_STATUS, DT_SPIN, a.status);
    // 1 / ||q|| of this row from the staged tile (chunk c of row r sits at r * 128 + ((c ^ (r & 7)) << 4) of its panel)
    float ss = 0.f;
    if (ok) {
#pragma unroll
      for (int pan = 0; pan < 2; ++pan)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(sm.q[pan]) + r * 128 + ((c ^ (r & 7)) << 4));
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x0 = __uint_as_float(w4[e] << 16), x1 = __uint_as_float(w4[e] & 0xFFFF0000u);
            ss = fmaf(x0, x0, ss);
            ss = fmaf(x1, x1, ss);
          }
        }
    }
    // exp(s * scale / ||q|| - shift) = 2^(s * qs2 - sh2): one FMA and one ex2 per entry
    const float qs2 = a.scale / fmaxf(sqrtf(ss), 1e-12f) * 1.4426950408889634f, sh2 = shift * 1.4426950408889634f;
    float l = 0.f;
    bool any_valid = false;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int i = 0; i < ntiles && ok; ++i) {
      const int pb = i & 1;
      ok = mbarrier_wait_bounded(&sm.s_full[pb], (i >> 1) & 1, DT_STATUS, DT_SPIN, a.status);
      if (ok && i >= 2) ok = mbarrier_wait_bounded(&sm.pv_done[pb], ((i - 2) >> 1) & 1, DT_STATUS, DT_SPIN, a.status);
      if (!ok) break;
      t5_fence_after();
      // validity of entry j of this tile for this row: a range [lo, hi) of j
      int lo, hi;
      if (i < nct) { lo = 0; hi = nvis - i * DT_KT; }
      else {
        const int w0 = wrow0 + (i - nct) * DT_KT;                  // window row of entry 0
        lo = tw - a.win_size + 1 - w0; hi = tw + 1 - w0;
        if (!active) hi = lo;
      }
      lo = max(lo, 0); hi = min(hi, DT_KT);
      any_valid = any_valid || hi > lo;
      uint8_t* prow = reinterpret_cast<uint8_t*>(sm.p[pb]) + r * 128;
      uint32_t sv[2][32];                                            // both halves of the score row requested at once
      t5_ld32(tS + 64u * pb + lane_base, sv[0]);
      t5_ld32(tS + 64u * pb + lane_base + 32, sv[1]);
      t5_wait_ld();
      const bool full = __all_sync(0xffffffffu, lo == 0 && hi == DT_KT);   // interior tile: no entry of any row masked
      float la = 0.f, lb = 0.f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {                               // 8 keys = one 16-byte chunk of the P row
          uint32_t o4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j0 = 32 * half + 8 * c + 2 * e;
            float p0 = ex2_fast(fmaf(__uint_as_float(sv[half][8 * c + 2 * e]), qs2, -sh2));
            float p1 = ex2_fast(fmaf(__uint_as_float(sv[half][8 * c + 2 * e + 1]), qs2, -sh2));
            if (!full) {
              p0 = (j0 >= lo && j0 < hi) ? p0 : 0.f;
              p1 = (j0 + 1 >= lo && j0 + 1 < hi) ? p1 : 0.f;
            }
            la += p0;
            lb += p1;
            __nv_bfloat162 hp = __floats2bfloat162_rn(p0, p1);
            o4[e] = *reinterpret_cast<uint32_t*>(&hp);
          }
          const int ch = 4 * half + c;
          *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
      }
      l += la + lb;
      t5_fence_async_smem();                                        // the MMA reads P through the async proxy
      t5_fence_before();
      __syncwarp();
      if (lane == 0) mbarrier_arrive(&sm.p_full[pb]);
    }
    // ---- epilogue ---------------------------------------------------------------------------------------------------
    if (ok && ntiles > 0) ok = mbarrier_wait_bounded(&sm.o_full, 0, DT_STATUS, DT_SPIN, a.status);
    t5_fence_after();
    if (a.sink && h < a.nh) l += __expf(sink - shift);
    const float inv = (any_valid && l > 0.f) ? 1.f / l : 0.f;
    bf16* orow = a.out + ((int64_t)b * a.T + t) * ((int64_t)a.nh * DT_C) + h * DT_C;
#pragma unroll 1
    for (int c0 = 0; c0 < DT_C; c0 += 32) {
      uint32_t ov[32];
      if (ok && ntiles > 0) { t5_ld32(tO + lane_base + c0, ov); t5_wait_ld(); }
      else {
#pragma unroll
        for (int j = 0; j < 32; ++j) ov[j] = 0u;
      }
      if (active && ok) {
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint32_t o4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 hp = __floats2bfloat162_rn(__uint_as_float(ov[8 * v4 + 2 * e]) * inv, __uint_as_float(ov[8 * v4 + 2 * e + 1]) * inv);
            o4[e] = *reinterpret_cast<uint32_t*>(&hp);
          }
          *reinterpret_cast<uint4*>(orow + c0 + 8 * v4) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
      }
    }
    t5_fence_before();
  }
  __syncthreads();
  if (warp == 4) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
  }
}

// ---- host ---------------------------------------------------------------------------------------------------------
typedef CUresult (*PFN_dt_encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int kch_make_tensor_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                                uint32_t box_rows, uint32_t box_cols);
int kch_make_tensor_map_qtile_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint32_t nh, uint64_t ld_elems,
                                   uint32_t box_heads, uint32_t box_rows);

// KCH_OK when launched; -100 when the shape is not this kernel's
int kch_attend_dense_tc5(const bf16* q, int64_t q_ld, int B, int T, int nh, const bf16* comp, int64_t comp_batch_rows,
                         int n_comp, int m, int64_t t0, int nvis_fixed, const bf16* win, int64_t win_ld,
                         int64_t win_batch_rows, int win_size, int win_t0, const void* sink, int sink_dtype, float scale,
                         bf16* out, cudaStream_t s) {
  if (nh < 1 || nh > 16 || T < 1 || B < 1) return -100;
  if ((q_ld % 8) != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return -100;
  if (comp && ((uintptr_t)comp & 15)) return -100;
  if (win && (((uintptr_t)win & 15) || (win_ld % 8) != 0)) return -100;
  if ((int64_t)B * T > 0x7FFFFFF0LL || (int64_t)B * comp_batch_rows > 0x7FFFFFF0LL || (int64_t)B * win_batch_rows > 0x7FFFFFF0LL) return -100;
  const bool has_comp = comp != nullptr && n_comp > 0, has_win = win != nullptr && win_size > 0;
  if (!has_comp && !has_win) return -100;
  CUtensorMap qmap, cmap, wmap;
  if (kch_make_tensor_map_qtile_bf16(&qmap, q, (uint64_t)B * T, (uint32_t)nh, (uint64_t)q_ld, 16, DT_Q) != KCH_OK) return -100;
  // a map that is not used still has to be a valid object: point it at the other operand
  const bf16* cbase = has_comp ? comp : win;
  const uint64_t crows = has_comp ? (uint64_t)B * comp_batch_rows : (uint64_t)B * win_batch_rows;
  const uint64_t cld = has_comp ? DT_C : (uint64_t)win_ld;
  if (kch_make_tensor_map_2d_bf16(&cmap, cbase, crows, DT_C, cld, DT_KT, 64) != KCH_OK) return -100;
  const bf16* wbase = has_win ? win : comp;
  const uint64_t wrows = has_win ? (uint64_t)B * win_batch_rows : (uint64_t)B * comp_batch_rows;
  const uint64_t wld = has_win ? (uint64_t)win_ld : DT_C;
  if (kch_make_tensor_map_2d_bf16(&wmap, wbase, wrows, DT_C, wld, DT_KT, 64) != KCH_OK) return -100;
  DtArgs a;
  a.B = B; a.T = T; a.nh = nh; a.n_comp = has_comp ? n_comp : 0; a.m = m; a.nvis_fixed = nvis_fixed; a.t0 = t0;
  a.comp_batch_rows = comp_batch_rows; a.win_batch_rows = win_batch_rows; a.win_size = has_win ? win_size : 0; a.win_t0 = win_t0;
  a.has_comp = has_comp ? 1 : 0; a.has_win = has_win ? 1 : 0;
  a.sink = sink; a.sink_dtype = sink_dtype; a.scale = scale; a.out = out;
  a.status = kch_status_device_ptr();
  KCH_REQUIRE(a.status != nullptr, "kch_attend: cannot resolve the device status word");
  const size_t smem = sizeof(DtSmem) + 1024;
  KCH_CUDA_OK(cudaFuncSetAttribute(attn_dense_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int64_t ctas = (int64_t)B * ((T + DT_Q - 1) / DT_Q);
  attn_dense_tc5_kernel<<<(unsigned)ctas, DT_THREADS, smem, s>>>(qmap, cmap, wmap, a);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
