// Lightning-indexer logits of a one-token step on tcgen05 (CSADecodingCache.forward_step, ops_decoding_cache.py:891-1000
// after csa_lightning_indexer, ops_csa.py:503-554):
//   logit[b, r] = sum_h w[b,h] relu(scale * q_h[b] . k[b,r] / ||k[b,r]||),   q_h normalised when asked.
// At batch 64 and 128 K tokens of context this is the largest stream of the step (268 MB of stored bf16 keys), with
// next to no arithmetic: the kernel's job is to keep HBM requests in flight.  Keys therefore never pass through
// registers: a producer thread brings tiles of 128 key rows (16 KB) through a ring of TMA stages, one thread issues
// the MMAs, and the only per-row work of the four epilogue warps is reading 24 accumulator columns.
//   A operand: the key tile as it lies in memory (exact bf16), 128 rows x K = 64.
//   B operand: the query of this batch entry, fp32, split in three bf16 terms (hi + mid + lo carries 24 bits of
//              mantissa); row `term * 8 + head` of a 32-row tile, so the products are exact and every sum is fp32.
//   D:         128 rows x 32 fp32 columns in tensor memory, two buffers, so the epilogue of a tile overlaps the MMAs
//              of the next one.
// A CTA takes 1024 rows of one batch entry; three CTAs share an SM (ring of 4 x 16 KB each).
// Every wait is bounded (status word, see kch_device_status).  No multicast.
#include <cuda.h>
#include <stdlib.h>

#include "kch_common.cuh"
#include "tc5_utils.cuh"

#define IXD_ROWS 1024
#define IXD_TILE 128
#define IXD_STAGES 4
#define IXD_THREADS 192
#define IXD_SPIN (1u << 24)

struct IxdSmem {
  alignas(1024) bf16 k[IXD_STAGES][IXD_TILE * 64];
  alignas(1024) bf16 qb[32 * 64];          // rows term * 8 + head, 128-byte swizzle; rows 24..31 zero
  float sq[8 * 64];
  float sw[8];
  alignas(8) uint64_t full[IXD_STAGES];
  uint64_t empty[IXD_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem;
};

__global__ void __launch_bounds__(IXD_THREADS, 3)
decode_indexer_tc5_kernel(const __grid_constant__ CUtensorMap kmap, const void* __restrict__ q, int q_dtype, int64_t q_ld,
                          const float* __restrict__ norms, const void* __restrict__ w, int w_dtype, int64_t w_ld,
                          float* __restrict__ logits, int64_t cap, int64_t n_ld, int HI, int normalize, float scale, int m,
                          const int32_t* __restrict__ ctr, unsigned int* status) {
  extern __shared__ uint8_t ixd_raw[];
  IxdSmem& sm = *reinterpret_cast<IxdSmem*>(((uintptr_t)ixd_raw + 1023) & ~(uintptr_t)1023);
  const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nvis = min(ctr[KCH_CTR_TOKENS] / m, ctr[KCH_CTR_N_BLOCKS]);
  const int r0 = blockIdx.x * IXD_ROWS;
  if (r0 >= nvis) return;                                      // the whole CTA, before any barrier or allocation
  const int ntiles = min(IXD_ROWS / IXD_TILE, (nvis - r0 + IXD_TILE - 1) / IXD_TILE);

  if (tid == 0) {
    for (int s = 0; s < IXD_STAGES; ++s) { mbarrier_init(&sm.full[s], 1); mbarrier_init(&sm.empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbarrier_init(&sm.acc_full[i], 1); mbarrier_init(&sm.acc_empty[i], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // the first round of the ring needs nothing but the barriers: the key stream starts before the query is staged
    for (int t = 0; t < min(ntiles, IXD_STAGES); ++t) {
      mbarrier_expect_tx(&sm.full[t], IXD_TILE * 64 * 2);
      t5_tma_load_2d(sm.k[t], &kmap, 0, (int)((int64_t)b * cap + r0 + t * IXD_TILE), &sm.full[t]);
    }
  }
  // ---- the query: normalised fp32 in shared memory, then its three bf16 terms as the B tile ----------------------
  for (int h = warp; h < 8; h += IXD_THREADS / 32) {
    float v0 = 0.f, v1 = 0.f;
    if (h < HI) { v0 = ld_any(q, (int64_t)b * q_ld + h * 64 + lane, q_dtype); v1 = ld_any(q, (int64_t)b * q_ld + h * 64 + 32 + lane, q_dtype); }
    if (normalize) {
      const float nrm = fmaxf(sqrtf(warp_sum(v0 * v0 + v1 * v1)), 1e-12f);
      v0 /= nrm; v1 /= nrm;
    }
    sm.sq[h * 64 + lane] = v0; sm.sq[h * 64 + 32 + lane] = v1;
    if (lane == 0) sm.sw[h] = h < HI ? (w ? ld_any(w, (int64_t)b * w_ld + h, w_dtype) : 1.f) : 0.f;
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr_u32(&sm.tmem)), "r"(64) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  __syncthreads();
  // 32 rows x 8 chunks of 16 bytes: row = term * 8 + head, chunk c holds elements 8c .. 8c+7 of that head's term
  for (int i = tid; i < 32 * 8; i += IXD_THREADS) {
    const int row = i >> 3, ch = i & 7, term = row >> 3, h = row & 7;
    uint32_t o[4] = {0u, 0u, 0u, 0u};
    if (term < 3) {
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float x0 = sm.sq[h * 64 + ch * 8 + 2 * p], x1 = sm.sq[h * 64 + ch * 8 + 2 * p + 1];
        const uint32_t hi = cvt_bf16x2(x0, x1);
        const float e0 = x0 - __uint_as_float(hi << 16), e1 = x1 - __uint_as_float(hi & 0xFFFF0000u);
        const uint32_t mid = cvt_bf16x2(e0, e1);
        const uint32_t lo = cvt_bf16x2(e0 - __uint_as_float(mid << 16), e1 - __uint_as_float(mid & 0xFFFF0000u));
        o[p] = term == 0 ? hi : (term == 1 ? mid : lo);
      }
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.qb) + row * 128 + ((ch ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  t5_fence_async_smem();                                       // the MMA reads this tile through the async proxy
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem = sm.tmem;

  if (warp == 4) {
    // ------------------------------ producer: key tiles ------------------------------------------------------------
    if (lane == 0) {
      for (int t = IXD_STAGES; t < ntiles; ++t) {              // the first round was issued at the top
        const int s = t % IXD_STAGES;
        if (!mbarrier_wait_bounded(&sm.empty[s], ((t / IXD_STAGES) & 1) ^ 1, KCH_STATUS_INDEXER_DECODE, IXD_SPIN, status)) break;
        mbarrier_expect_tx(&sm.full[s], IXD_TILE * 64 * 2);
        t5_tma_load_2d(sm.k[s], &kmap, 0, (int)((int64_t)b * cap + r0 + t * IXD_TILE), &sm.full[s]);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer -----------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = t5_idesc(32);
      const uint64_t bdesc = t5_desc(smem_addr_u32(sm.qb));
      for (int t = 0; t < ntiles; ++t) {
        const int s = t % IXD_STAGES, acc = t & 1;
        if (t >= 2 && !mbarrier_wait_bounded(&sm.acc_empty[acc], ((t >> 1) & 1) ^ 1, KCH_STATUS_INDEXER_DECODE, IXD_SPIN, status)) break;
        if (!mbarrier_wait_bounded(&sm.full[s], (t / IXD_STAGES) & 1, KCH_STATUS_INDEXER_DECODE, IXD_SPIN, status)) break;
        t5_fence_after();
        const uint64_t adesc = t5_desc(smem_addr_u32(sm.k[s]));
#pragma unroll
        for (int k = 0; k < 4; ++k) t5_mma(tmem + acc * 32, adesc + 2 * k, bdesc + 2 * k, idesc, k ? 1u : 0u);
        t5_commit(&sm.empty[s]);
        t5_commit(&sm.acc_full[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue: one key row per thread --------------------------------------------------
    const float* nb = norms + (int64_t)b * cap;
    float* lg = logits + (int64_t)b * n_ld;
    float wh[8];
#pragma unroll
    for (int h = 0; h < 8; ++h) wh[h] = sm.sw[h];
    // the norms of all this thread's rows first: one round trip for the CTA instead of one per tile
    float nv[IXD_ROWS / IXD_TILE];
#pragma unroll
    for (int t = 0; t < IXD_ROWS / IXD_TILE; ++t) {
      const int row = r0 + t * IXD_TILE + warp * 32 + lane;
      nv[t] = (normalize && row < nvis) ? nb[row] : 1.f;
    }
    bool ok = true;
#pragma unroll
    for (int t = 0; t < IXD_ROWS / IXD_TILE; ++t) {
      if (t < ntiles && ok) {
        const int acc = t & 1;
        const int row = r0 + t * IXD_TILE + warp * 32 + lane;
        ok = mbarrier_wait_bounded(&sm.acc_full[acc], (t >> 1) & 1, KCH_STATUS_INDEXER_DECODE, IXD_SPIN, status);
        if (ok) {
          t5_fence_after();
          uint32_t r[32];
          t5_ld32(tmem + ((uint32_t)(warp * 32) << 16) + acc * 32, r);
          t5_wait_ld();
          t5_fence_before();
          __syncwarp();
          if (lane == 0) mbarrier_arrive(&sm.acc_empty[acc]);
          float o = 0.f;
#pragma unroll
          for (int h = 0; h < 8; ++h) {
            const float c = (__uint_as_float(r[h]) + __uint_as_float(r[8 + h])) + __uint_as_float(r[16 + h]);
            o += fmaxf(c / nv[t] * scale, 0.f) * wh[h];
          }
          if (row < nvis) lg[row] = o;
        }
      }
    }
  }
  t5_fence_before();
  __syncthreads();
  if (warp == 4) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64) : "memory");
  }
}

int kch_make_tensor_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                                uint32_t box_rows, uint32_t box_cols);

// KCH_OK when launched; -100 when the shape is not this kernel's (bf16 keys of 64 channels, at most 8 indexer heads)
int kch_decode_indexer_logits_tc5(const void* q, int q_dtype, int64_t q_ld, const void* keys, const float* norms,
                                  const void* w, int w_dtype, int64_t w_ld, float* logits, int B, int64_t cap, int64_t n_ld,
                                  int HI, int normalize, float scale, int m, const int32_t* ctr, cudaStream_t s) {
  if (HI > 8 || ((uintptr_t)keys & 15) || (int64_t)B * cap > 0x7FFFFFFFLL) return -100;
  CUtensorMap kmap;
  if (kch_make_tensor_map_2d_bf16(&kmap, keys, (uint64_t)B * (uint64_t)cap, 64, 64, IXD_TILE, 64) != KCH_OK) return -100;
  unsigned int* status = kch_status_device_ptr();
  KCH_REQUIRE(status != nullptr, "kch_decode_indexer_topk: cannot resolve the device status word");
  const size_t smem = sizeof(IxdSmem) + 1024;
  KCH_CUDA_OK(cudaFuncSetAttribute(decode_indexer_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((cap + IXD_ROWS - 1) / IXD_ROWS), (unsigned)B);
  decode_indexer_tc5_kernel<<<grid, IXD_THREADS, smem, s>>>(kmap, q, q_dtype, q_ld, norms, w, w_dtype, w_ld, logits, cap, n_ld, HI,
                                                           normalize, scale, m, ctr, status);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
