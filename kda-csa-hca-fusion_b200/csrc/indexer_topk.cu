// Lightning indexer and exact top-k selection  (csa_lightning_indexer, ops_csa.py:503-554).
//   logits[t,n] = sum_h w[t,h] * relu(scale * q[t,h] . k[n])      fp32 FMA throughout
//   block n is visible to the query at absolute position t iff n < (t+1)/m
//   select the min(topk, n_blocks) largest visible logits; slots without a visible block are -1
// Tie rule: equal logits are taken in ascending block index (the reference leaves tie order to
// its array library).  Selection is an exact 4x8-bit radix select on the order-preserving integer
// image of the fp32 logits, so the selected SET is a pure function of the logits.
#include <math.h>
#include <stdlib.h>

#include <atomic>

#include "mma_utils.cuh"

// ---------------------------------------------------------------------------------------
// Logits: 64 queries x 64 blocks per CTA, 16x16 threads, 4x4 outputs per thread.
// q: [B,T,HI,DI] fp32, k: [B,n,DI] fp32 (both already normalised when cosine scoring is on).
// ---------------------------------------------------------------------------------------
#define IDX_TQ 64
#define IDX_TN 64
#define IDX_DK 32

__global__ void __launch_bounds__(256)
indexer_logits_kernel(const float* __restrict__ q, const float* __restrict__ k,
                      const float* __restrict__ w, float* __restrict__ logits, int T, int n, int HI,
                      int DI, int64_t n_ld, float scale, int m, int64_t t0, int nvis_fixed,
                      int64_t k_bstride) {
  const int nt = blockIdx.x, qt = blockIdx.y, b = blockIdx.z;
  const int tq0 = qt * IDX_TQ, n0 = nt * IDX_TN;
  // visibility of the last query of the tile bounds the useful block range
  int tlast = min(T, tq0 + IDX_TQ) - 1;
  int64_t vis_last = nvis_fixed >= 0 ? nvis_fixed : (m > 0 ? (t0 + tlast + 1) / m : n);
  if (n0 >= vis_last) return;
  __shared__ float sq[IDX_DK][IDX_TQ + 1];
  __shared__ float sk[IDX_DK][IDX_TN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float out[4][4] = {};
  for (int h = 0; h < HI; ++h) {
    float acc[4][4] = {};
    for (int d0 = 0; d0 < DI; d0 += IDX_DK) {
      for (int idx = threadIdx.x; idx < IDX_TQ * IDX_DK; idx += 256) {
        int r = idx / IDX_DK, d = idx % IDX_DK;
        int t = tq0 + r;
        sq[d][r] = (t < T && d0 + d < DI) ? q[(((int64_t)b * T + t) * HI + h) * DI + d0 + d] : 0.f;
      }
      for (int idx = threadIdx.x; idx < IDX_TN * IDX_DK; idx += 256) {
        int r = idx / IDX_DK, d = idx % IDX_DK;
        int nn = n0 + r;
        sk[d][r] = (nn < n && d0 + d < DI) ? k[(int64_t)b * k_bstride + (int64_t)nn * DI + d0 + d] : 0.f;
      }
      __syncthreads();
#pragma unroll 8
      for (int d = 0; d < IDX_DK; ++d) {
        float qa[4], ka[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { qa[i] = sq[d][ty * 4 + i]; ka[i] = sk[d][tx * 4 + i]; }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qa[i], ka[j], acc[i][j]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int t = tq0 + ty * 4 + i;
      float wh = 1.f;
      if (w) wh = t < T ? w[((int64_t)b * T + t) * HI + h] : 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) out[i][j] = fmaf(fmaxf(acc[i][j] * scale, 0.f), wh, out[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int t = tq0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int nn = n0 + tx * 4 + j;
      if (nn < n) logits[((int64_t)b * T + t) * n_ld + nn] = out[i][j];
    }
  }
}

// ---------------------------------------------------------------------------------------
// Tensor-core logits for DI = 64: 64 queries x 128 blocks per CTA, 4 warps (16 queries each).
// fp32-grade accuracy from bf16 tensor cores: both operands are split into three bf16 terms
// (hi + mid + lo = 24 bits of mantissa) and the six products that matter are accumulated in fp32:
//   q.k ~= hi.hi + hi.mid + mid.hi + mid.mid + hi.lo + lo.hi      (dropped terms < 2^-24 |q||k|)
// so the selection boundary rule (picks exact wherever the gap exceeds 1e-6 relative) still holds.
// ---------------------------------------------------------------------------------------
#define IM_TQ 64
#define IM_TN 128
#define IM_D 64

__device__ __forceinline__ void split3_pair(float x0, float x1, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  hi = cvt_bf16x2(x0, x1);
  const float r0 = x0 - __uint_as_float(hi << 16), r1 = x1 - __uint_as_float(hi & 0xFFFF0000u);
  mid = cvt_bf16x2(r0, r1);
  lo = cvt_bf16x2(r0 - __uint_as_float(mid << 16), r1 - __uint_as_float(mid & 0xFFFF0000u));
}

// Three-term split of fp32 rows into three bf16 row arrays (row r of batch b read at x + b*bstride + r*64).
__global__ void split3_rows_kernel(const float* __restrict__ x, int64_t rows_per_batch, int64_t bstride, int64_t rows,
                                   bf16* __restrict__ hi, bf16* __restrict__ mid, bf16* __restrict__ lo) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one 8-element chunk
  if (i >= rows * 8) return;
  const int64_t r = i >> 3;
  const int ch = (int)(i & 7);
  const float4* p = reinterpret_cast<const float4*>(x + (r / rows_per_batch) * bstride + (r % rows_per_batch) * IM_D + 8 * ch);
  const float4 a = p[0], c = p[1];
  uint32_t h[4], m[4], l[4];
  split3_pair(a.x, a.y, h[0], m[0], l[0]); split3_pair(a.z, a.w, h[1], m[1], l[1]);
  split3_pair(c.x, c.y, h[2], m[2], l[2]); split3_pair(c.z, c.w, h[3], m[3], l[3]);
  *reinterpret_cast<uint4*>(hi + i * 8) = make_uint4(h[0], h[1], h[2], h[3]);
  *reinterpret_cast<uint4*>(mid + i * 8) = make_uint4(m[0], m[1], m[2], m[3]);
  *reinterpret_cast<uint4*>(lo + i * 8) = make_uint4(l[0], l[1], l[2], l[3]);
}

__device__ __forceinline__ void cpa16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

struct IdxSplit {            // pre-split operands (PRE = true); rows are 64 bf16
  const bf16 *qh, *qm, *ql;  // [B*T*HI][64]
  const bf16 *kh, *km, *kl;  // [B*n][64]
  const bf16* qraw;          // QRAW: un-normalised bf16 queries, token t of batch b at qraw + (b*T+t)*q_ld, head h at +64h
  int64_t q_ld;
  int q_normalize;           // QRAW: divide each head's dot products by max(||q_h||, 1e-12)
};

// PRE = false: operands are split inside the kernel (no extra workspace); PRE = true: the three bf16 terms
// were prepared once by split3_rows_kernel and are streamed in with cp.async (query tiles double-buffered).
// QRAW (with PRE): the queries are bf16 as the projection wrote them, so they are exact single-term operands;
// their L2 norm is taken from the fragments and divides the finished dot product.  Three products per k-step
// (q x key hi/mid/lo) instead of six, and no split pass over the queries.
template <bool PRE, bool QRAW = false>
__global__ void __launch_bounds__(128)
indexer_logits_mma_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ w,
                          IdxSplit sp, float* __restrict__ logits, int T, int n, int HI, int64_t n_ld, float scale,
                          int m, int64_t t0, int nvis_fixed, int64_t k_bstride) {
  extern __shared__ __align__(128) uint8_t sm[];
  const int nt0 = blockIdx.x * IM_TN, tq0 = blockIdx.y * IM_TQ, b = blockIdx.z;
  const int tlast = min(T, tq0 + IM_TQ) - 1;
  const int64_t vis_last = nvis_fixed >= 0 ? nvis_fixed : (m > 0 ? (t0 + tlast + 1) / m : n);
  if (nt0 >= vis_last) return;
  uint8_t* kt = sm;                        // 3 x [128][64] bf16 (hi, mid, lo), 128-byte rows, swizzled
  uint8_t* qt = sm + 3 * IM_TN * 128;      // (PRE: 2 x) 3 x [64][64] bf16; QRAW: 2 x [64][64] bf16
  constexpr int QT_BYTES = (QRAW ? 1 : 3) * IM_TQ * 128;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g4 = lane >> 2, j4 = lane & 3;

  auto stage_q = [&](int h, int buf) {
    uint8_t* dstb = qt + buf * QT_BYTES;
    for (int idx = tid; idx < IM_TQ * 8; idx += 128) {
      const int r = idx >> 3, ch = idx & 7;
      const int t = tq0 + r;
      const uint32_t off = swz<128>(r, ch);
      if constexpr (QRAW) {
        const int64_t src = ((int64_t)b * T + (t < T ? t : 0)) * sp.q_ld + h * IM_D + 8 * ch;
        cpa16(smem_addr_u32(dstb + off), sp.qraw + src, t < T ? 16 : 0);
      } else if constexpr (PRE) {
        const int64_t src = ((((int64_t)b * T + (t < T ? t : 0)) * HI + h) * IM_D + 8 * ch);
        const int bytes = t < T ? 16 : 0;
        cpa16(smem_addr_u32(dstb + off), sp.qh + src, bytes);
        cpa16(smem_addr_u32(dstb + IM_TQ * 128 + off), sp.qm + src, bytes);
        cpa16(smem_addr_u32(dstb + 2 * IM_TQ * 128 + off), sp.ql + src, bytes);
      } else {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
        if (t < T) {
          const float4* p = reinterpret_cast<const float4*>(q + (((int64_t)b * T + t) * HI + h) * IM_D + 8 * ch);
          x = p[0]; y = p[1];
        }
        uint32_t hi[4], mid[4], lo[4];
        split3_pair(x.x, x.y, hi[0], mid[0], lo[0]); split3_pair(x.z, x.w, hi[1], mid[1], lo[1]);
        split3_pair(y.x, y.y, hi[2], mid[2], lo[2]); split3_pair(y.z, y.w, hi[3], mid[3], lo[3]);
        *reinterpret_cast<uint4*>(dstb + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(dstb + IM_TQ * 128 + off) = make_uint4(mid[0], mid[1], mid[2], mid[3]);
        *reinterpret_cast<uint4*>(dstb + 2 * IM_TQ * 128 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
    }
    if constexpr (PRE) asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // stage the key tile once
  for (int idx = tid; idx < IM_TN * 8; idx += 128) {
    const int r = idx >> 3, ch = idx & 7;
    const int nn = nt0 + r;
    const uint32_t off = swz<128>(r, ch);
    if constexpr (PRE) {
      const int64_t src = ((int64_t)b * n + (nn < n ? nn : 0)) * IM_D + 8 * ch;
      const int bytes = nn < n ? 16 : 0;
      cpa16(smem_addr_u32(kt + off), sp.kh + src, bytes);
      cpa16(smem_addr_u32(kt + IM_TN * 128 + off), sp.km + src, bytes);
      cpa16(smem_addr_u32(kt + 2 * IM_TN * 128 + off), sp.kl + src, bytes);
    } else {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
      if (nn < n) {
        const float4* p = reinterpret_cast<const float4*>(k + (int64_t)b * k_bstride + (int64_t)nn * IM_D + 8 * ch);
        x = p[0]; y = p[1];
      }
      uint32_t hi[4], mid[4], lo[4];
      split3_pair(x.x, x.y, hi[0], mid[0], lo[0]); split3_pair(x.z, x.w, hi[1], mid[1], lo[1]);
      split3_pair(y.x, y.y, hi[2], mid[2], lo[2]); split3_pair(y.z, y.w, hi[3], mid[3], lo[3]);
      *reinterpret_cast<uint4*>(kt + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(kt + IM_TN * 128 + off) = make_uint4(mid[0], mid[1], mid[2], mid[3]);
      *reinterpret_cast<uint4*>(kt + 2 * IM_TN * 128 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
  }
  if constexpr (PRE) stage_q(0, 0);     // joins the key tile's copies in the first commit group
  float out[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { out[i][0] = out[i][1] = out[i][2] = out[i][3] = 0.f; }
  const uint32_t kth = smem_addr_u32(kt), ktm = kth + IM_TN * 128, ktl = ktm + IM_TN * 128;
  const int r0 = tq0 + 16 * warp + g4, r1 = r0 + 8;
  for (int h = 0; h < HI; ++h) {
    int buf = 0;
    if constexpr (PRE) {
      buf = h & 1;
      if (h + 1 < HI) {
        stage_q(h + 1, buf ^ 1);          // the other buffer was released by the barrier ending head h-1
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();
    } else {
      __syncthreads();     // previous head's fragments are in registers; the query tile may be overwritten
      stage_q(h, 0);
      __syncthreads();
    }
    const uint32_t qth = smem_addr_u32(qt + buf * QT_BYTES), qtm = qth + IM_TQ * 128, qtl = qtm + IM_TQ * 128;
    uint32_t ah[4][4], am[4][4], al[4][4];
    float qs0 = scale, qs1 = scale;        // scale / ||q|| of rows r0, r1 (QRAW)
    {
      const int arow = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t o = swz<128>(arow, 2 * ks + (lane >> 4));
        ldmatrix_x4(qth + o, ah[ks][0], ah[ks][1], ah[ks][2], ah[ks][3]);
        if constexpr (!QRAW) {
          ldmatrix_x4(qtm + o, am[ks][0], am[ks][1], am[ks][2], am[ks][3]);
          ldmatrix_x4(qtl + o, al[ks][0], al[ks][1], al[ks][2], al[ks][3]);
        }
      }
      if constexpr (QRAW) {
        if (sp.q_normalize) {
          // registers 0,2 of a fragment hold row g4 (r0), registers 1,3 row g4+8 (r1); a quad covers a row
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {
              const float x = __uint_as_float(ah[ks][rr] << 16), y = __uint_as_float(ah[ks][rr] & 0xFFFF0000u);
              if (rr & 1) s1 = fmaf(x, x, fmaf(y, y, s1)); else s0 = fmaf(x, x, fmaf(y, y, s0));
            }
          }
          s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
          s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
          qs0 = scale / fmaxf(sqrtf(s0), 1e-12f);
          qs1 = scale / fmaxf(sqrtf(s1), 1e-12f);
        }
      }
    }
    float w0 = 1.f, w1 = 1.f;
    if (w) {
      w0 = r0 < T ? w[((int64_t)b * T + r0) * HI + h] : 0.f;
      w1 = r1 < T ? w[((int64_t)b * T + r1) * HI + h] : 0.f;
    }
    // two 8-block column tiles at a time: two independent accumulator chains per warp
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int qd = 0; qd < 2; ++qd) {
        uint32_t bh[2][4], bm[2][4], bl[2][4];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t o = swz<128>(8 * (2 * np + u) + (lane & 7), 4 * qd + (lane >> 3));
          ldmatrix_x4(kth + o, bh[u][0], bh[u][1], bh[u][2], bh[u][3]);
          ldmatrix_x4(ktm + o, bm[u][0], bm[u][1], bm[u][2], bm[u][3]);
          ldmatrix_x4(ktl + o, bl[u][0], bl[u][1], bl[u][2], bl[u][3]);
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int ks = 2 * qd + kk;
          if constexpr (QRAW) {
            mma_bf16_16816(acc[0], ah[ks], bl[0][2 * kk], bl[0][2 * kk + 1]);
            mma_bf16_16816(acc[1], ah[ks], bl[1][2 * kk], bl[1][2 * kk + 1]);
            mma_bf16_16816(acc[0], ah[ks], bm[0][2 * kk], bm[0][2 * kk + 1]);
            mma_bf16_16816(acc[1], ah[ks], bm[1][2 * kk], bm[1][2 * kk + 1]);
            mma_bf16_16816(acc[0], ah[ks], bh[0][2 * kk], bh[0][2 * kk + 1]);
            mma_bf16_16816(acc[1], ah[ks], bh[1][2 * kk], bh[1][2 * kk + 1]);
            continue;
          }
          // smallest terms first; the two column tiles alternate so consecutive MMAs are independent
          mma_bf16_16816(acc[0], al[ks], bh[0][2 * kk], bh[0][2 * kk + 1]);
          mma_bf16_16816(acc[1], al[ks], bh[1][2 * kk], bh[1][2 * kk + 1]);
          mma_bf16_16816(acc[0], ah[ks], bl[0][2 * kk], bl[0][2 * kk + 1]);
          mma_bf16_16816(acc[1], ah[ks], bl[1][2 * kk], bl[1][2 * kk + 1]);
          mma_bf16_16816(acc[0], am[ks], bm[0][2 * kk], bm[0][2 * kk + 1]);
          mma_bf16_16816(acc[1], am[ks], bm[1][2 * kk], bm[1][2 * kk + 1]);
          mma_bf16_16816(acc[0], am[ks], bh[0][2 * kk], bh[0][2 * kk + 1]);
          mma_bf16_16816(acc[1], am[ks], bh[1][2 * kk], bh[1][2 * kk + 1]);
          mma_bf16_16816(acc[0], ah[ks], bm[0][2 * kk], bm[0][2 * kk + 1]);
          mma_bf16_16816(acc[1], ah[ks], bm[1][2 * kk], bm[1][2 * kk + 1]);
          mma_bf16_16816(acc[0], ah[ks], bh[0][2 * kk], bh[0][2 * kk + 1]);
          mma_bf16_16816(acc[1], ah[ks], bh[1][2 * kk], bh[1][2 * kk + 1]);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int nt = 2 * np + u;
        out[nt][0] = fmaf(fmaxf(acc[u][0] * qs0, 0.f), w0, out[nt][0]);
        out[nt][1] = fmaf(fmaxf(acc[u][1] * qs0, 0.f), w0, out[nt][1]);
        out[nt][2] = fmaf(fmaxf(acc[u][2] * qs1, 0.f), w1, out[nt][2]);
        out[nt][3] = fmaf(fmaxf(acc[u][3] * qs1, 0.f), w1, out[nt][3]);
      }
    }
    if constexpr (PRE) __syncthreads();   // every warp is done with this head's query buffer
  }
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const int nn = nt0 + 8 * nt + 2 * j4;
    if (r0 < T) {
      float* p = logits + ((int64_t)b * T + r0) * n_ld + nn;
      if (nn + 1 < n) *reinterpret_cast<float2*>(p) = make_float2(out[nt][0], out[nt][1]);
      else if (nn < n) p[0] = out[nt][0];
    }
    if (r1 < T) {
      float* p = logits + ((int64_t)b * T + r1) * n_ld + nn;
      if (nn + 1 < n) *reinterpret_cast<float2*>(p) = make_float2(out[nt][2], out[nt][3]);
      else if (nn < n) p[0] = out[nt][2];
    }
  }
}

static inline int64_t align256(int64_t x) { return (x + 255) & ~255LL; }

// logits launcher shared by both entry points: tensor cores for DI == 64, CUDA cores otherwise.
// `split_ws` (optional, split_bytes long) holds the pre-split operands when it is large enough.
static int64_t indexer_split_bytes(int B, int T, int n_blocks, int HI, int DI) {
  if (DI != IM_D) return 0;
  return 3 * (align256((int64_t)B * T * HI * IM_D * 2) + align256((int64_t)B * n_blocks * IM_D * 2));
}

static int64_t indexer_ksplit_bytes(int B, int n_blocks) { return 3 * align256((int64_t)B * n_blocks * IM_D * 2); }

// tcgen05 form of the logits (gemm_tcgen05.cu)
bool kch_indexer_logits_tcgen05_ok(int B, int T, int n, int HI, int64_t q_ld, const void* q);
int kch_indexer_logits_tcgen05(const void* q, int64_t q_ld, int q_normalize, const void* kh, const void* km,
                               const void* kl, const float* w, float* coef, float* logits, int B, int T, int n, int HI,
                               int64_t n_ld, float scale, int m, int64_t t0, int n_visible, cudaStream_t s);

// `qraw` (optional): un-normalised bf16 queries read in place (token stride q_ld); then q_idx is not used.
static int launch_indexer_logits(const float* q_idx, const float* k_idx, const float* w_idx, float* logits, int B,
                                 int T, int n_blocks, int HI, int DI, int64_t n_ld, float scale, int m, int64_t t0,
                                 int n_visible, int64_t k_batch_stride, void* split_ws, int64_t split_bytes,
                                 cudaStream_t s, const bf16* qraw = nullptr, int64_t q_ld = 0, int q_normalize = 0) {
  const int64_t kbs = k_batch_stride > 0 ? k_batch_stride : (int64_t)n_blocks * DI;
  static const bool force_simt = [] { const char* e = getenv("KCH_INDEXER"); return e && e[0] == 's'; }();
  if (qraw) {
    KCH_REQUIRE(DI == IM_D && (((uintptr_t)qraw | (uintptr_t)k_idx) & 15) == 0 && (q_ld % 8) == 0 && (kbs % 4) == 0,
                "kch_indexer_topk_ex: bf16 queries need c_I == 64, 16-byte aligned operands and q_ld %% 8 == 0");
    KCH_REQUIRE(split_ws && split_bytes >= indexer_ksplit_bytes(B, n_blocks) && (((uintptr_t)split_ws) & 15) == 0,
                "kch_indexer_topk_ex: workspace too small for the split keys");
    dim3 g((n_blocks + IM_TN - 1) / IM_TN, (T + IM_TQ - 1) / IM_TQ, B);
    const int64_t krows = (int64_t)B * n_blocks, kb = align256(krows * IM_D * 2);
    uint8_t* p = (uint8_t*)split_ws;
    bf16* kh = (bf16*)p; bf16* km = (bf16*)(p + kb); bf16* kl = (bf16*)(p + 2 * kb);
    split3_rows_kernel<<<(unsigned)ceil_div64(krows * 8, 256), 256, 0, s>>>(k_idx, n_blocks, kbs, krows, kh, km, kl);
    KCH_LAUNCH_OK();
    // tcgen05 path (query tiles of 128 rows, tensor-memory accumulators) when the shape allows and the workspace
    // also holds the per-(query, head) coefficients; else the mma.sync kernel below
    const int64_t coef_off = 3 * kb, coef_bytes = (int64_t)B * T * HI * 4;
    // (that kernel folds `scale` into the coefficient outside the relu, which equals relu(scale * q.k) only for
    // scale >= 0; a negative scale takes the mma.sync kernel, which applies it inside)
    if (scale >= 0.f && kch_indexer_logits_tcgen05_ok(B, T, n_blocks, HI, q_ld, qraw) &&
        split_bytes >= coef_off + coef_bytes)
      return kch_indexer_logits_tcgen05(qraw, q_ld, q_normalize, kh, km, kl, w_idx, (float*)(p + coef_off), logits, B, T,
                                        n_blocks, HI, n_ld, scale, m, t0, n_visible, s);
    IdxSplit sp = {};
    sp.kh = kh; sp.km = km; sp.kl = kl; sp.qraw = qraw; sp.q_ld = q_ld; sp.q_normalize = q_normalize;
    const int smem = 3 * IM_TN * 128 + 2 * IM_TQ * 128;
    KCH_CUDA_OK(cudaFuncSetAttribute(indexer_logits_mma_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    indexer_logits_mma_kernel<true, true><<<g, 128, smem, s>>>(nullptr, k_idx, w_idx, sp, logits, T, n_blocks, HI, n_ld, scale,
                                                               m, t0, n_visible, kbs);
    KCH_LAUNCH_OK();
    return KCH_OK;
  }
  const bool aligned = (((uintptr_t)q_idx | (uintptr_t)k_idx) & 15) == 0 && (kbs % 4) == 0;
  if (!force_simt && DI == IM_D && aligned) {
    dim3 g((n_blocks + IM_TN - 1) / IM_TN, (T + IM_TQ - 1) / IM_TQ, B);
    IdxSplit sp = {};
    if (split_ws && split_bytes >= indexer_split_bytes(B, T, n_blocks, HI, DI) && (((uintptr_t)split_ws) & 15) == 0) {
      const int64_t qrows = (int64_t)B * T * HI, krows = (int64_t)B * n_blocks;
      const int64_t qb = align256(qrows * IM_D * 2), kb = align256(krows * IM_D * 2);
      uint8_t* p = (uint8_t*)split_ws;
      bf16* qh = (bf16*)p; bf16* qm = (bf16*)(p + qb); bf16* ql = (bf16*)(p + 2 * qb);
      bf16* kh = (bf16*)(p + 3 * qb); bf16* km = (bf16*)(p + 3 * qb + kb); bf16* kl = (bf16*)(p + 3 * qb + 2 * kb);
      split3_rows_kernel<<<(unsigned)ceil_div64(qrows * 8, 256), 256, 0, s>>>(q_idx, qrows, 0, qrows, qh, qm, ql);
      KCH_LAUNCH_OK();
      split3_rows_kernel<<<(unsigned)ceil_div64(krows * 8, 256), 256, 0, s>>>(k_idx, n_blocks, kbs, krows, kh, km, kl);
      KCH_LAUNCH_OK();
      sp.qh = qh; sp.qm = qm; sp.ql = ql; sp.kh = kh; sp.km = km; sp.kl = kl;
      const int smem = 3 * IM_TN * 128 + 2 * 3 * IM_TQ * 128;
      KCH_CUDA_OK(cudaFuncSetAttribute(indexer_logits_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      indexer_logits_mma_kernel<true><<<g, 128, smem, s>>>(q_idx, k_idx, w_idx, sp, logits, T, n_blocks, HI, n_ld, scale,
                                                           m, t0, n_visible, kbs);
    } else {
      const int smem = 3 * (IM_TN + IM_TQ) * 128;
      KCH_CUDA_OK(cudaFuncSetAttribute(indexer_logits_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      indexer_logits_mma_kernel<false><<<g, 128, smem, s>>>(q_idx, k_idx, w_idx, sp, logits, T, n_blocks, HI, n_ld, scale,
                                                            m, t0, n_visible, kbs);
    }
  } else {
    dim3 g1((n_blocks + IDX_TN - 1) / IDX_TN, (T + IDX_TQ - 1) / IDX_TQ, B);
    indexer_logits_kernel<<<g1, 256, 0, s>>>(q_idx, k_idx, w_idx, logits, T, n_blocks, HI, DI, n_ld, scale, m, t0,
                                              n_visible, kbs);
  }
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// ---------------------------------------------------------------------------------------
// Selection: one CTA per query row.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f2ord(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// inclusive-exclusive block scan helper over 256 threads: returns exclusive prefix of `v`,
// total in *total.  `buf` has 9 words.
__device__ __forceinline__ int block_excl_scan(int v, int* buf, int* total) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += y;
  }
  if (lane == 31) buf[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int x = lane < 8 ? buf[lane] : 0;
    int xi = x;
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, xi, o);
      if (lane >= o) xi += y;
    }
    if (lane < 8) buf[lane] = xi - x;
    if (lane == 7) buf[8] = xi;
  }
  __syncthreads();
  int res = buf[warp] + inc - v;
  *total = buf[8];
  __syncthreads();
  return res;
}

// the same scan over NT threads (NT / 32 <= 32 warps); `buf` has 34 words
template <int NT>
__device__ __forceinline__ int block_excl_scan_n(int v, int* buf, int* total) {
  constexpr int NW = NT / 32;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += y;
  }
  if (lane == 31) buf[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int x = lane < NW ? buf[lane] : 0;
    int xi = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, xi, o);
      if (lane >= o) xi += y;
    }
    if (lane < NW) buf[lane] = xi - x;
    if (lane == 31) buf[33] = xi;
  }
  __syncthreads();
  int res = buf[warp] + inc - v;
  *total = buf[33];
  __syncthreads();
  return res;
}

// NT threads per row: 256 for the rows of a prefill, 1024 for the few long rows of a decode step
template <int NT>
__global__ void __launch_bounds__(NT)
topk_select_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int T, int n,
                   int64_t n_ld, int topk, int m, int64_t t0, int nvis_fixed, int sorted, int cache_cap,
                   const int32_t* __restrict__ ctr = nullptr, int ctr_m = 1) {
  if (ctr) {   // decode step: row count and visible prefix come from the cache's device counters
    n = ctr[KCH_CTR_N_BLOCKS];
    nvis_fixed = min(ctr[KCH_CTR_TOKENS] / ctr_m, n);
  }
  // dynamic shared memory: [cache_cap floats: the row's visible logits] [sort keys, only when sorted]
  extern __shared__ __align__(16) uint8_t sel_smem[];
  float* srow = reinterpret_cast<float*>(sel_smem);
  unsigned long long* ssort = reinterpret_cast<unsigned long long*>(sel_smem + (size_t)cache_cap * 4);
  const int64_t row = blockIdx.x;  // b*T + t
  const int t = (int)(row % T);
  const float* lg = logits + row * n_ld;
  int32_t* orow = out + row * topk;
  int64_t nv64 = nvis_fixed >= 0 ? nvis_fixed : (m > 0 ? (t0 + t + 1) / m : n);
  const int nv = (int)(nv64 < n ? nv64 : n);
  const int ksel = topk < n ? topk : n;
  const int tid = threadIdx.x;
  __shared__ int hist[256];
  __shared__ int sbuf[34];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  int nsel;
  if (nv <= ksel) {
    for (int i = tid; i < topk; i += NT) orow[i] = i < nv ? i : -1;
    nsel = nv;
  } else {
    // Thread t owns the contiguous index range [t*E, (t+1)*E): ordered compaction then needs one
    // block scan in total.  The row is staged in shared memory transposed (element k of thread t at
    // k*NT + t) so that those strided-by-E reads are bank-conflict free.
    const int E = (nv + NT - 1) / NT;
    const bool cached = E * NT <= cache_cap;
    if (cached) {
      for (int i = tid; i < nv; i += NT) srow[(i % E) * NT + i / E] = lg[i];
      __syncthreads();
    }
    const int i0 = tid * E;
    const int cnt_mine = max(0, min(E, nv - i0));
    auto val = [&](int k) -> float { return cached ? srow[k * NT + tid] : lg[i0 + k]; };
    uint32_t prefix = 0, pmask = 0;
    int need = ksel;  // how many still to take from the current prefix class
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int k = 0; k < cnt_mine; ++k) {
        uint32_t u = f2ord(val(k));
        if ((u & pmask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1);
      }
      __syncthreads();
      // thread t looks at bin 255-t: an exclusive scan gives the population of all higher bins
      const int bin = 255 - tid;
      const int cnt = tid < 256 ? hist[bin] : 0;
      int tot;
      const int cum = block_excl_scan_n<NT>(cnt, sbuf, &tot);
      if (tid < 256 && cum < need && cum + cnt >= need) {
        s_prefix = prefix | ((uint32_t)bin << shift);
        s_need = need - cum;
      }
      __syncthreads();
      prefix = s_prefix;
      need = s_need;
      pmask |= 0xFFu << shift;
    }
    // prefix = key of the k-th largest logit; `need` of the entries equal to it are taken,
    // lowest index first; everything strictly greater is taken.
    const int n_gt = ksel - need;
    int c_gt = 0, c_eq = 0;
    for (int k = 0; k < cnt_mine; ++k) {
      uint32_t u = f2ord(val(k));
      c_gt += (u > prefix);
      c_eq += (u == prefix);
    }
    int tot_gt, tot_eq;
    int p_gt = block_excl_scan_n<NT>(c_gt, sbuf, &tot_gt);
    int p_eq = block_excl_scan_n<NT>(c_eq, sbuf, &tot_eq);
    for (int k = 0; k < cnt_mine; ++k) {
      uint32_t u = f2ord(val(k));
      if (u > prefix) orow[p_gt++] = i0 + k;
      else if (u == prefix) { if (p_eq < need) orow[n_gt + p_eq] = i0 + k; ++p_eq; }
    }
    for (int i = ksel + tid; i < topk; i += NT) orow[i] = -1;
    nsel = ksel;
  }
  if (!sorted) return;
  // descending by logit, ascending block index among equals (bitonic sort on 64-bit keys)
  __syncthreads();
  int P = 1;
  while (P < nsel) P <<= 1;
  for (int i = tid; i < P; i += NT) {
    unsigned long long key = 0ull;
    if (i < nsel) {
      int id = orow[i];
      key = ((unsigned long long)f2ord(lg[id]) << 32) | (uint32_t)(0x7FFFFFFF - id);
    }
    ssort[i] = key;
  }
  __syncthreads();
  for (int size = 2; size <= P; size <<= 1)
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < P; i += NT) {
        int j = i ^ stride;
        if (j > i) {
          unsigned long long a = ssort[i], c = ssort[j];
          bool desc = (i & size) == 0;
          if (desc ? (a < c) : (a > c)) { ssort[i] = c; ssort[j] = a; }
        }
      }
      __syncthreads();
    }
  for (int i = tid; i < nsel; i += NT) orow[i] = 0x7FFFFFFF - (int)(uint32_t)(ssort[i] & 0xFFFFFFFFu);
}

// Radix select of one row with SLOTS keys per thread in registers (E <= SLOTS elements owned by each thread).
template <int EPT>
__device__ __forceinline__ void select_row_regs(const float* __restrict__ lg, int32_t* __restrict__ orow, int nv, int ksel,
                                                int E, int64_t n_ld, int* hist, int* sbuf, uint32_t* s_prefix_p,
                                                int* s_need_p) {
  const int tid = threadIdx.x;
  uint32_t& s_prefix = *s_prefix_p;
  int& s_need = *s_need_p;
    const int i0 = tid * E;
    const int cnt_mine = max(0, min(E, nv - i0));
    uint32_t u[EPT];
#pragma unroll
    for (int k4 = 0; k4 < EPT / 4; ++k4) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (4 * k4 < E && i0 + 4 * k4 < n_ld) v = *reinterpret_cast<const float4*>(lg + i0 + 4 * k4);   // row pad is readable
      u[4 * k4] = f2ord(v.x); u[4 * k4 + 1] = f2ord(v.y); u[4 * k4 + 2] = f2ord(v.z); u[4 * k4 + 3] = f2ord(v.w);
    }
    uint32_t prefix = 0, pmask = 0;
    int need = ksel;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      hist[tid] = 0;
      __syncthreads();
#pragma unroll
      for (int k = 0; k < EPT; ++k)
        if (k < cnt_mine && (u[k] & pmask) == prefix) atomicAdd(&hist[(u[k] >> shift) & 255], 1);
      __syncthreads();
      const int bin = 255 - tid;
      const int cnt = hist[bin];
      int tot;
      const int cum = block_excl_scan(cnt, sbuf, &tot);
      if (cum < need && cum + cnt >= need) {
        s_prefix = prefix | ((uint32_t)bin << shift);
        s_need = need - cum;
      }
      __syncthreads();
      prefix = s_prefix;
      need = s_need;
      pmask |= 0xFFu << shift;
    }
    const int n_gt = ksel - need;
    int c_gt = 0, c_eq = 0;
#pragma unroll
    for (int k = 0; k < EPT; ++k)
      if (k < cnt_mine) { c_gt += (u[k] > prefix); c_eq += (u[k] == prefix); }
    int tot_gt, tot_eq;
    int p_gt = block_excl_scan(c_gt, sbuf, &tot_gt);
    int p_eq = block_excl_scan(c_eq, sbuf, &tot_eq);
#pragma unroll
    for (int k = 0; k < EPT; ++k)
      if (k < cnt_mine) {
        if (u[k] > prefix) orow[p_gt++] = i0 + k;
        else if (u[k] == prefix) { if (p_eq < need) orow[n_gt + p_eq] = i0 + k; ++p_eq; }
      }
}

// Register variant for rows of up to 256*EPT logits (the prefill case: n_blocks <= 8192): thread t owns the
// contiguous index range [t*E, (t+1)*E), E = ceil(nv/256) rounded up to 4, and keeps the order-preserving keys of
// its logits in registers for all four radix passes, the counting and the ordered compaction: one 16-byte-vector
// read of the row, no shared-memory staging.  Same selection rule and output as topk_select_kernel.
template <int EPT>
__global__ void __launch_bounds__(256)
topk_select_reg_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int T, int n, int64_t n_ld,
                       int topk, int m, int64_t t0, int nvis_fixed, int sorted) {
  extern __shared__ __align__(16) uint8_t sel_smem[];
  unsigned long long* ssort = reinterpret_cast<unsigned long long*>(sel_smem);
  const int64_t row = blockIdx.x;
  const int t = (int)(row % T);
  const float* lg = logits + row * n_ld;
  int32_t* orow = out + row * topk;
  int64_t nv64 = nvis_fixed >= 0 ? nvis_fixed : (m > 0 ? (t0 + t + 1) / m : n);
  const int nv = (int)(nv64 < n ? nv64 : n);
  const int ksel = topk < n ? topk : n;
  const int tid = threadIdx.x;
  __shared__ int hist[256];
  __shared__ int sbuf[9];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  int nsel;
  if (nv <= ksel) {
    for (int i = tid; i < topk; i += 256) orow[i] = i < nv ? i : -1;
    nsel = nv;
  } else {
    // slots per thread follow this row's visible length, not the longest row of the launch
    const int E = (((nv + 255) >> 8) + 3) & ~3;          // <= EPT by the host's choice of EPT
    if (EPT > 8 && E <= 8) select_row_regs<8>(lg, orow, nv, ksel, E, n_ld, hist, sbuf, &s_prefix, &s_need);
    else if (EPT > 16 && E <= 16) select_row_regs<(EPT > 16 ? 16 : EPT)>(lg, orow, nv, ksel, E, n_ld, hist, sbuf, &s_prefix, &s_need);
    else select_row_regs<EPT>(lg, orow, nv, ksel, E, n_ld, hist, sbuf, &s_prefix, &s_need);
    for (int i = ksel + tid; i < topk; i += 256) orow[i] = -1;
    nsel = ksel;
  }
  if (!sorted) return;
  __syncthreads();
  int P = 1;
  while (P < nsel) P <<= 1;
  for (int i = tid; i < P; i += 256) {
    unsigned long long key = 0ull;
    if (i < nsel) {
      int id = orow[i];
      key = ((unsigned long long)f2ord(lg[id]) << 32) | (uint32_t)(0x7FFFFFFF - id);
    }
    ssort[i] = key;
  }
  __syncthreads();
  for (int size = 2; size <= P; size <<= 1)
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < P; i += 256) {
        int j = i ^ stride;
        if (j > i) {
          unsigned long long a = ssort[i], c = ssort[j];
          bool desc = (i & size) == 0;
          if (desc ? (a < c) : (a > c)) { ssort[i] = c; ssort[j] = a; }
        }
      }
      __syncthreads();
    }
  for (int i = tid; i < nsel; i += 256) orow[i] = 0x7FFFFFFF - (int)(uint32_t)(ssort[i] & 0xFFFFFFFFu);
}

// Long rows of a decode step (one query per sequence over tens of thousands of cached blocks): a thread-block
// cluster of SC_CTAS CTAs per row instead of one CTA.  (Shared-memory atomics on a few hot bins are not the cost of
// these passes: aggregating the increments of a warp with match.any first made the select 10 - 25 % slower.)  CTA r owns the contiguous index range
// [r * seg, (r + 1) * seg) with its keys in registers (as topk_select_reg_kernel); each radix pass builds a
// 256-bin histogram per CTA, and every CTA sums the SC_CTAS histograms through distributed shared memory, so all
// of them agree on the threshold without a broadcast.  The histogram is double-buffered: one cluster barrier per
// pass.  Same selection rule and output as topk_select_kernel (ties: lowest block index first, because rank
// order is index order); output order is unspecified.  Row length and visible prefix come from the cache's
// device counters.
#define SC_CTAS 8
__device__ __forceinline__ uint32_t sc_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void sc_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ int sc_ld_remote(const int* local, uint32_t rank) {
  uint32_t addr = (uint32_t)__cvta_generic_to_shared(local), remote;
  int v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}

template <int EPT>
__global__ void __launch_bounds__(256)
topk_select_cluster_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int64_t n_ld, int topk,
                           const int32_t* __restrict__ ctr, int ctr_m) {
  const int n = ctr[KCH_CTR_N_BLOCKS];
  const int nv = min(ctr[KCH_CTR_TOKENS] / ctr_m, n);
  const int b = blockIdx.y, tid = threadIdx.x;
  const uint32_t rank = sc_cluster_rank();
  const float* lg = logits + (int64_t)b * n_ld;
  int32_t* orow = out + (int64_t)b * topk;
  const int ksel = topk < n ? topk : n;
  if (nv <= ksel) {                                       // uniform over the cluster: nobody reaches a barrier
    if (rank == 0) for (int i = tid; i < topk; i += 256) orow[i] = i < nv ? i : -1;
    return;
  }
  __shared__ int hist[2][256];
  __shared__ int sbuf[9];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  __shared__ int s_tot[2];
  // slots per thread: this row's visible length over SC_CTAS x 256 threads, rounded up to 4 (<= EPT by the host's choice)
  const int E = (((nv + SC_CTAS * 256 - 1) / (SC_CTAS * 256)) + 3) & ~3;
  const int i0 = ((int)rank * 256 + tid) * E;
  const int cnt_mine = max(0, min(E, nv - i0));
  uint32_t u[EPT];
#pragma unroll
  for (int k4 = 0; k4 < EPT / 4; ++k4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (4 * k4 < E && i0 + 4 * k4 < n_ld) v = *reinterpret_cast<const float4*>(lg + i0 + 4 * k4);   // row pad is readable
    u[4 * k4] = f2ord(v.x); u[4 * k4 + 1] = f2ord(v.y); u[4 * k4 + 2] = f2ord(v.z); u[4 * k4 + 3] = f2ord(v.w);
  }
  uint32_t prefix = 0, pmask = 0;
  int need = ksel;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    int* h = hist[pass & 1];
    h[tid] = 0;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < EPT; ++k)
      if (k < cnt_mine && (u[k] & pmask) == prefix) atomicAdd(&h[(u[k] >> shift) & 255], 1);
    sc_cluster_sync();                                    // every CTA's histogram of this pass is complete
    const int bin = 255 - tid;
    int cnt = 0;
#pragma unroll
    for (uint32_t r = 0; r < SC_CTAS; ++r) cnt += sc_ld_remote(&h[bin], r);
    int tot;
    const int cum = block_excl_scan(cnt, sbuf, &tot);
    if (cum < need && cum + cnt >= need) {
      s_prefix = prefix | ((uint32_t)bin << shift);
      s_need = need - cum;
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    pmask |= 0xFFu << shift;
  }
  // ordered compaction: everything above the threshold, then `need` of the entries equal to it, lowest index first
  const int n_gt = ksel - need;
  int c_gt = 0, c_eq = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k)
    if (k < cnt_mine) { c_gt += (u[k] > prefix); c_eq += (u[k] == prefix); }
  int tot_gt, tot_eq;
  int p_gt = block_excl_scan(c_gt, sbuf, &tot_gt);
  int p_eq = block_excl_scan(c_eq, sbuf, &tot_eq);
  if (tid == 0) { s_tot[0] = tot_gt; s_tot[1] = tot_eq; }
  sc_cluster_sync();
  for (uint32_t r = 0; r < rank; ++r) { p_gt += sc_ld_remote(&s_tot[0], r); p_eq += sc_ld_remote(&s_tot[1], r); }
#pragma unroll
  for (int k = 0; k < EPT; ++k)
    if (k < cnt_mine) {
      if (u[k] > prefix) orow[p_gt++] = i0 + k;
      else if (u[k] == prefix) { if (p_eq < need) orow[n_gt + p_eq] = i0 + k; ++p_eq; }
    }
  if (rank == 0) for (int i = ksel + tid; i < topk; i += 256) orow[i] = -1;
  sc_cluster_sync();                                      // nobody leaves while a neighbour may still read its totals
}

static int launch_topk_select_cluster(const float* logits, int32_t* indices, int B, int64_t n_ld, int topk,
                                      const int32_t* counters, int ctr_m, int ept, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = SC_CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(SC_CTAS, (unsigned)B); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = s;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (ept <= 8) KCH_CUDA_OK(cudaLaunchKernelEx(&cfg, topk_select_cluster_kernel<8>, logits, indices, n_ld, topk, counters, ctr_m));
  else if (ept <= 16) KCH_CUDA_OK(cudaLaunchKernelEx(&cfg, topk_select_cluster_kernel<16>, logits, indices, n_ld, topk, counters, ctr_m));
  else KCH_CUDA_OK(cudaLaunchKernelEx(&cfg, topk_select_cluster_kernel<32>, logits, indices, n_ld, topk, counters, ctr_m));
  kch_note_launch(1);
  return KCH_OK;
}

// shared launcher of the selection: register variant when a row fits 256 x 32 logits, else the staged one
static int launch_topk_select(const float* logits, int32_t* indices, int B, int T, int n_blocks, int64_t n_ld, int topk,
                              int m, int64_t t0, int n_visible, int sorted, size_t sort_smem, cudaStream_t s) {
  const unsigned grid = (unsigned)((int64_t)B * T);
  static const bool force_staged = [] { const char* e = getenv("KCH_SELECT"); return e && e[0] == 's'; }();
  const int e_needed = (((n_blocks + 255) >> 8) + 3) & ~3;
  if (!force_staged && e_needed <= 32 && (((uintptr_t)logits) & 15) == 0 && (n_ld % 4) == 0) {
#define SEL_GO(EPT_)                                                                                              \
    do {                                                                                                          \
      if (sort_smem > 48 * 1024)                                                                                  \
        KCH_CUDA_OK(cudaFuncSetAttribute(topk_select_reg_kernel<EPT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sort_smem)); \
      topk_select_reg_kernel<EPT_><<<grid, 256, sort_smem, s>>>(logits, indices, T, n_blocks, n_ld, topk, m, t0, n_visible, sorted); \
    } while (0)
    if (e_needed <= 8) SEL_GO(8);
    else if (e_needed <= 16) SEL_GO(16);
    else SEL_GO(32);
#undef SEL_GO
    KCH_LAUNCH_OK();
    return KCH_OK;
  }
  const int cache_cap = (int)(n_ld <= 16384 ? ((n_ld + 255) & ~255LL) : 0);
  const size_t smem = sort_smem + (size_t)cache_cap * 4;
  KCH_CUDA_OK(cudaFuncSetAttribute(topk_select_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  topk_select_kernel<256><<<grid, 256, smem, s>>>(logits, indices, T, n_blocks, n_ld, topk, m, t0, n_visible, sorted, cache_cap);
  KCH_LAUNCH_OK();
  return KCH_OK;
}

static int64_t indexer_logits_bytes(int B, int T, int n) {
  int64_t n_ld = ((int64_t)n + 3) & ~3LL;
  return align256((int64_t)B * T * n_ld * 4);
}

extern "C" int64_t kch_indexer_workspace_bytes(int B, int T, int n, int HI, int DI) {
  if (B <= 0 || T <= 0 || n <= 0) return 0;
  return indexer_logits_bytes(B, T, n) + indexer_split_bytes(B, T, n, HI, DI);
}

extern "C" int64_t kch_indexer_workspace_bytes_ex(int B, int T, int n, int q_dtype) {
  if (B <= 0 || T <= 0 || n <= 0) return 0;
  if (q_dtype == KCH_BF16)   // logits + three key terms + one coefficient per (query, head), up to 16 heads
    return indexer_logits_bytes(B, T, n) + indexer_ksplit_bytes(B, n) + align256((int64_t)B * T * 16 * 4);
  return indexer_logits_bytes(B, T, n);
}

extern "C" int kch_indexer_topk_ex(const void* q_idx, int q_dtype, int64_t q_ld, int q_normalize, const float* k_idx,
                                   const float* w_idx, int32_t* indices, int B, int T, int n_blocks, int HI, int DI,
                                   int topk, float scale, int m, int64_t t0, int n_visible, int sorted,
                                   int64_t k_batch_stride, void* workspace, int64_t workspace_bytes, void* stream);

extern "C" int kch_indexer_topk(const float* q_idx, const float* k_idx, const float* w_idx,
                                int32_t* indices, int B, int T, int n_blocks, int HI, int DI, int topk,
                                float scale, int m, int64_t t0, int n_visible, int sorted,
                                int64_t k_batch_stride, void* workspace, int64_t workspace_bytes,
                                void* stream) {
  return kch_indexer_topk_ex(q_idx, KCH_F32, (int64_t)HI * DI, 0, k_idx, w_idx, indices, B, T, n_blocks, HI, DI, topk, scale,
                             m, t0, n_visible, sorted, k_batch_stride, workspace, workspace_bytes, stream);
}

extern "C" int kch_indexer_topk_ex(const void* q_idx_any, int q_dtype, int64_t q_ld, int q_normalize, const float* k_idx,
                                   const float* w_idx, int32_t* indices, int B, int T, int n_blocks, int HI, int DI,
                                   int topk, float scale, int m, int64_t t0, int n_visible, int sorted,
                                   int64_t k_batch_stride, void* workspace, int64_t workspace_bytes, void* stream) {
  KCH_REQUIRE(q_dtype == KCH_F32 || q_dtype == KCH_BF16, "kch_indexer_topk_ex: q_dtype=%d", q_dtype);
  KCH_REQUIRE(q_dtype == KCH_BF16 || (q_ld == (int64_t)HI * DI && !q_normalize),
              "kch_indexer_topk_ex: fp32 queries must be dense and already normalised");
  const float* q_idx = q_dtype == KCH_F32 ? (const float*)q_idx_any : nullptr;
  const bf16* q_raw = q_dtype == KCH_BF16 ? (const bf16*)q_idx_any : nullptr;
  KCH_REQUIRE(topk >= 0, "topk=%d must be >= 0 (0 selects zero blocks)", topk);
  KCH_REQUIRE(DI >= 1, "q_idx.shape[-1]=%d must be >= 1 (indexer key dimension c_I must be positive)", DI);
  KCH_REQUIRE(HI >= 1, "nIh=%d must be >= 1 (indexer head count)", HI);
  KCH_REQUIRE(B >= 0 && T >= 0 && n_blocks >= 0, "kch_indexer_topk: B=%d T=%d n=%d", B, T, n_blocks);
  if (B == 0 || T == 0 || topk == 0) return KCH_OK;
  cudaStream_t s = kch_stream(stream);
  if (n_blocks == 0) {
    KCH_CUDA_OK(cudaMemsetAsync(indices, 0xFF, (size_t)B * T * topk * sizeof(int32_t), s));
    return KCH_OK;
  }
  // the logits are mandatory; the pre-split operands are used when the workspace also has room for them
  const int64_t need = indexer_logits_bytes(B, T, n_blocks);     // 256-byte aligned start of the split area
  const int64_t logits_exact = (int64_t)B * T * (((int64_t)n_blocks + 3) & ~3LL) * 4;
  KCH_REQUIRE(workspace && workspace_bytes >= logits_exact, "kch_indexer_topk: workspace %lld < %lld bytes",
              (long long)workspace_bytes, (long long)logits_exact);
  int64_t n_ld = ((int64_t)n_blocks + 3) & ~3LL;
  float* logits = (float*)workspace;
  {
    void* split_ws = workspace_bytes > need ? (void*)((uint8_t*)workspace + need) : nullptr;
    int rc = launch_indexer_logits(q_idx, k_idx, w_idx, logits, B, T, n_blocks, HI, DI, n_ld, scale, m, t0, n_visible,
                                   k_batch_stride, split_ws, workspace_bytes - need, s, q_raw, q_ld, q_normalize);
    if (rc != KCH_OK) return rc;
  }
  size_t smem = 0;
  if (sorted) {
    int ks = topk < n_blocks ? topk : n_blocks;
    int P = 1;
    while (P < ks) P <<= 1;
    KCH_REQUIRE(P <= 8192, "kch_indexer_topk: sorted output supports topk <= 8192 (got %d)", ks);
    smem = (size_t)P * 8;
  }
  return launch_topk_select(logits, indices, B, T, n_blocks, n_ld, topk, m, t0, n_visible, sorted, smem, s);
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some callers cannot obtain device memory at the moment they need the indexer: a decode loop that
// runs inside a serving runtime whose memory pool is frozen after start-up, or a host thread that is
// not allowed to touch the CUDA allocator (cudaMalloc synchronises the whole device and would stall
// every other stream of the server).  kch_indexer_topk needs a logits workspace from such a caller;
// this entry point instead keeps the logits in a fixed array that is part of the loaded library
// image: KCH_INDEXER_STATIC_FLOATS fp32 values (16 MiB) per GPU that loads the library, held until the
// process exits.  That covers B*T*round_up(n_blocks,4) <= 4 Mi, e.g. a batch-64 decode step over 32768
// cached blocks per sequence; larger requests are rejected, not truncated.
//
// The array name is only a host-side handle.  The device address is looked up with
// cudaGetSymbolAddress once per device, on the first call made while that device is current, and cached.
// Make that first call outside any stream capture (symbol lookup is not a capturable operation).
// Every call on a device uses the same array and overwrites whatever the previous call left there; the
// selection only reads logits written by the same call, so nothing has to be cleared in between.  Two
// calls that overlap on the GPU (different streams, no dependency) would race on the array: order them.
// ---------------------------------------------------------------------------------------
#define KCH_INDEXER_STATIC_FLOATS (4u << 20)
static __device__ __align__(256) float g_indexer_static_logits[KCH_INDEXER_STATIC_FLOATS];

static int indexer_static_address(float** out) {
  // one slot per device ordinal; host threads that make their first call on a device at the same time all look
  // the address up and store the same value, so relaxed atomics are enough
  static std::atomic<float*> cached[64];
  int dev = 0;
  KCH_CUDA_OK(cudaGetDevice(&dev));
  KCH_REQUIRE(dev >= 0 && dev < 64, "kch_indexer_topk_static: device ordinal %d out of range", dev);
  float* p = cached[dev].load(std::memory_order_relaxed);
  if (!p) {
    KCH_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_indexer_static_logits));
    cached[dev].store(p, std::memory_order_relaxed);
  }
  *out = p;
  return KCH_OK;
}

extern "C" int64_t kch_indexer_topk_static_capacity(void) { return (int64_t)KCH_INDEXER_STATIC_FLOATS; }

extern "C" int kch_indexer_topk_static(const float* q_idx, const float* k_idx, const float* w_idx,
                                       int32_t* indices, int B, int T, int n_blocks, int HI, int DI, int topk,
                                       float scale, int m, int64_t t0, int n_visible, int64_t k_batch_stride,
                                       void* stream) {
  KCH_REQUIRE(topk >= 0, "topk=%d must be >= 0 (0 selects zero blocks)", topk);
  KCH_REQUIRE(DI >= 1, "q_idx.shape[-1]=%d must be >= 1 (indexer key dimension c_I must be positive)", DI);
  KCH_REQUIRE(HI >= 1, "nIh=%d must be >= 1 (indexer head count)", HI);
  KCH_REQUIRE(B >= 0 && T >= 0 && n_blocks >= 0, "kch_indexer_topk_static: B=%d T=%d n=%d", B, T, n_blocks);
  if (B == 0 || T == 0 || topk == 0) return KCH_OK;
  cudaStream_t s = kch_stream(stream);
  if (n_blocks == 0) {
    KCH_CUDA_OK(cudaMemsetAsync(indices, 0xFF, (size_t)B * T * topk * sizeof(int32_t), s));
    return KCH_OK;
  }
  const int64_t n_ld = ((int64_t)n_blocks + 3) & ~3LL;
  const int64_t need = (int64_t)B * T * n_ld;
  KCH_REQUIRE(need <= (int64_t)KCH_INDEXER_STATIC_FLOATS,
              "kch_indexer_topk_static: B*T*round_up(n_blocks,4) = %lld logits exceed the built-in scratch of %lld; "
              "use kch_indexer_topk with a caller-provided workspace",
              (long long)need, (long long)KCH_INDEXER_STATIC_FLOATS);
  float* logits = nullptr;
  int rc = indexer_static_address(&logits);
  if (rc != KCH_OK) return rc;
  rc = launch_indexer_logits(q_idx, k_idx, w_idx, logits, B, T, n_blocks, HI, DI, n_ld, scale, m, t0, n_visible,
                             k_batch_stride, nullptr, 0, s);
  if (rc != KCH_OK) return rc;
  return launch_topk_select(logits, indices, B, T, n_blocks, n_ld, topk, m, t0, n_visible, 0, 0, s);
}

// ---------------------------------------------------------------------------------------
// Decode step: one indexer query per sequence against that sequence's stored keys.
// A memory-bound matrix-vector product: every visible key row is read once in its storage type
// (bf16 or fp32; DI*2 bytes per row at bf16) together with its fp32 norm (the reference normalises the
// stored keys with F.normalize, ops_decoding_cache.py:919-924; here q . key is divided by the norm) and
// scored against the HI query heads held in shared memory.  The visible prefix comes from the
// cache's device counters.  VEC path: 16-byte loads, DI/EPL lanes per row; otherwise one warp per row.
// ---------------------------------------------------------------------------------------
#define DIX_ROWS 1024   // key rows per CTA
#define DIX_MAX_HD 1024 // HI*DI floats of query held in shared memory

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
decode_indexer_logits_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ld, const T* __restrict__ keys,
                             const float* __restrict__ norms, const void* __restrict__ w, int w_dtype, int64_t w_ld,
                             float* __restrict__ logits, int64_t cap, int64_t n_ld,
                             int HI, int DI, int normalize, float scale, int m, const int32_t* __restrict__ ctr) {
  const int b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvis = min(ctr[KCH_CTR_TOKENS] / m, ctr[KCH_CTR_N_BLOCKS]);
  const int r0 = blockIdx.x * DIX_ROWS;
  if (r0 >= nvis) return;
  const int r1 = min(nvis, r0 + DIX_ROWS);
  __shared__ __align__(16) float sq[DIX_MAX_HD];
  __shared__ float sw[64];
  // the query of this sequence, L2-normalised per head when cosine scoring is on (one warp per head)
  for (int h = warp; h < HI; h += 8) {
    float ss = 0.f;
    for (int d = lane; d < DI; d += 32) { float v = ld_any(q, (int64_t)b * q_ld + h * DI + d, q_dtype); sq[h * DI + d] = v; ss += v * v; }
    if (normalize) {
      const float nrm = fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
      for (int d = lane; d < DI; d += 32) sq[h * DI + d] /= nrm;
    }
    if (lane == 0) sw[h] = w ? ld_any(w, (int64_t)b * w_ld + h, w_dtype) : 1.f;
  }
  __syncthreads();
  const T* kb = keys + (int64_t)b * cap * DI;
  const float* nb = norms + (int64_t)b * cap;
  float* lg = logits + (int64_t)b * n_ld;
  if (VEC) {
    constexpr int EPL = 16 / (int)sizeof(T);          // elements per lane
    const int LPR = DI / EPL;                          // lanes per row (power of two <= 32)
    const int rpp = 256 / LPR;                         // rows per pass of the CTA
    const int sub = tid % LPR, rloc = tid / LPR;
    // uniform trip count keeps the shuffles converged; four rows per thread are loaded before any is scored
    for (int rb = r0 + rloc; rb < r0 + DIX_ROWS; rb += 4 * rpp) {
      uint4 raw[4];
      float dv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = rb + u * rpp;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        dv[u] = 1.f;
        if (r < r1) {
          raw[u] = *reinterpret_cast<const uint4*>(kb + (int64_t)r * DI + sub * EPL);
          if (normalize) dv[u] = nb[r];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = rb + u * rpp;
        float kv[EPL];
        if (sizeof(T) == 2) {
          const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            kv[(2 * i) % EPL] = __uint_as_float(w4[i] << 16);
            kv[(2 * i + 1) % EPL] = __uint_as_float(w4[i] & 0xFFFF0000u);
          }
        } else {
          kv[0] = __uint_as_float(raw[u].x); kv[1] = __uint_as_float(raw[u].y);
          kv[2 % EPL] = __uint_as_float(raw[u].z); kv[3 % EPL] = __uint_as_float(raw[u].w);
        }
        float out = 0.f;
        for (int h = 0; h < HI; ++h) {
          const float* qh = sq + h * DI + sub * EPL;
          float p = 0.f;
#pragma unroll
          for (int i = 0; i < EPL; ++i) p = fmaf(qh[i], kv[i], p);
          for (int off = LPR >> 1; off > 0; off >>= 1) p += __shfl_xor_sync(0xffffffffu, p, off);
          // the key's norm divides the finished dot product (the reference divides the key element by element:
          // the same value up to one rounding of the logit)
          out = fmaf(fmaxf(p / dv[u] * scale, 0.f), sw[h], out);
        }
        if (r < r1 && sub == 0) lg[r] = out;
      }
    }
  } else {
    for (int r = r0 + warp; r < r1; r += 8) {
      const float dv = normalize ? nb[r] : 1.f;
      float out = 0.f;
      for (int h = 0; h < HI; ++h) {
        float p = 0.f;
        for (int d = lane; d < DI; d += 32) p = fmaf(sq[h * DI + d], ldf(kb + (int64_t)r * DI + d) / dv, p);
        p = warp_sum(p);
        out = fmaf(fmaxf(p * scale, 0.f), sw[h], out);
      }
      if (lane == 0) lg[r] = out;
    }
  }
}

// Tensor-core form of the same product for bf16 keys with DI = 64 and up to 8 indexer heads.  Sixteen key rows
// are the M rows of mma.sync m16n8k16 and the heads its N columns; the query is split in three bf16 terms
// (24 bits of mantissa) while the stored keys are exact bf16, so every product is exact and the sum is
// fp32-grade.  A key row is 128 bytes: four lanes read it with 16-byte loads (fully coalesced, no shared
// memory); the contraction index is permuted so that those 8 consecutive elements are the A fragments of two
// k-steps, and the query fragments are built once with the same permutation.
__global__ void __launch_bounds__(256, 3)      // three CTAs per SM: the key stream wants warps in flight, not registers
decode_indexer_logits_mma_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ld, const bf16* __restrict__ keys,
                                 const float* __restrict__ norms, const void* __restrict__ w, int w_dtype, int64_t w_ld,
                                 float* __restrict__ logits, int64_t cap, int64_t n_ld, int HI, int normalize,
                                 float scale, int m, const int32_t* __restrict__ ctr) {
  constexpr int DI = 64;
  const int b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int nvis = min(ctr[KCH_CTR_TOKENS] / m, ctr[KCH_CTR_N_BLOCKS]);
  const int r0 = blockIdx.x * DIX_ROWS;
  if (r0 >= nvis) return;
  __shared__ float sq[8 * DI];
  __shared__ float sw[8];
  {
    const int h = warp;                                        // 8 warps, 8 head slots
    float v0 = 0.f, v1 = 0.f;
    if (h < HI) { v0 = ld_any(q, (int64_t)b * q_ld + h * DI + lane, q_dtype); v1 = ld_any(q, (int64_t)b * q_ld + h * DI + 32 + lane, q_dtype); }
    if (normalize) {
      const float nrm = fmaxf(sqrtf(warp_sum(v0 * v0 + v1 * v1)), 1e-12f);
      v0 /= nrm; v1 /= nrm;
    }
    sq[h * DI + lane] = v0; sq[h * DI + 32 + lane] = v1;
    if (lane == 0) sw[h] = h < HI ? (w ? ld_any(w, (int64_t)b * w_ld + h, w_dtype) : 1.f) : 0.f;
  }
  __syncthreads();
  // B fragments (head g is column g) of the four k-steps, three terms each: logical k-step 2c+s' holds the
  // query elements 32c + 8t + 4s' + {0,1} (b0) and + {2,3} (b1), matching the key chunk a lane loads
  uint32_t qb[4][3][2];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    const int k0 = (ks >> 1) * 32 + 8 * t + 4 * (ks & 1);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t hi, mid, lo;
      split3_pair(sq[g * DI + k0 + 2 * half], sq[g * DI + k0 + 2 * half + 1], hi, mid, lo);
      qb[ks][0][half] = hi; qb[ks][1][half] = mid; qb[ks][2][half] = lo;
    }
  }
  const float w0 = sw[2 * t], w1 = sw[2 * t + 1];             // this thread's output columns are heads 2t, 2t+1
  const bf16* kb = keys + (int64_t)b * cap * DI;
  const float* nb = norms + (int64_t)b * cap;
  float* lg = logits + (int64_t)b * n_ld;
  const int wr0 = r0 + warp * (DIX_ROWS / 8);                 // 128 rows per warp, 8 groups of 16
#pragma unroll 1
  for (int gi = 0; gi < 8; gi += 2) {
    uint4 raw[2][4];                                           // [group][row g chunk 0/1, row g+8 chunk 0/1]
    float nv[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int rg = wr0 + (gi + u) * 16;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = rg + g + 8 * hh;
        raw[u][2 * hh] = raw[u][2 * hh + 1] = make_uint4(0u, 0u, 0u, 0u);
        nv[u][hh] = 1.f;
        if (row < nvis) {
          const uint4* rp = reinterpret_cast<const uint4*>(kb + (int64_t)row * DI);
          raw[u][2 * hh] = rp[t];
          raw[u][2 * hh + 1] = rp[4 + t];
          if (normalize) nv[u][hh] = nb[row];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int rg = wr0 + (gi + u) * 16;
      if (rg >= nvis) break;                                   // warp-uniform
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      // a0 = row g, first pair; a1 = row g+8, first pair; a2 = row g, second pair; a3 = row g+8, second pair
      const uint32_t lo_row[8] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w, raw[u][1].x, raw[u][1].y, raw[u][1].z, raw[u][1].w};
      const uint32_t hi_row[8] = {raw[u][2].x, raw[u][2].y, raw[u][2].z, raw[u][2].w, raw[u][3].x, raw[u][3].y, raw[u][3].z, raw[u][3].w};
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t af[4] = {lo_row[2 * ks], hi_row[2 * ks], lo_row[2 * ks + 1], hi_row[2 * ks + 1]};
#pragma unroll
        for (int term = 0; term < 3; ++term) mma_bf16_16816(c, af, qb[ks][term][0], qb[ks][term][1]);
      }
      // c0,c1: row rg+g, heads 2t, 2t+1;  c2,c3: row rg+g+8
      float o0 = fmaxf(c[0] / nv[u][0] * scale, 0.f) * w0 + fmaxf(c[1] / nv[u][0] * scale, 0.f) * w1;
      float o1 = fmaxf(c[2] / nv[u][1] * scale, 0.f) * w0 + fmaxf(c[3] / nv[u][1] * scale, 0.f) * w1;
      o0 += __shfl_xor_sync(0xffffffffu, o0, 1); o0 += __shfl_xor_sync(0xffffffffu, o0, 2);
      o1 += __shfl_xor_sync(0xffffffffu, o1, 1); o1 += __shfl_xor_sync(0xffffffffu, o1, 2);
      if (t == 0) {
        if (rg + g < nvis) lg[rg + g] = o0;
        if (rg + g + 8 < nvis) lg[rg + g + 8] = o1;
      }
    }
  }
}

int kch_decode_indexer_logits_tc5(const void* q, int q_dtype, int64_t q_ld, const void* keys, const float* norms,
                                  const void* w, int w_dtype, int64_t w_ld, float* logits, int B, int64_t cap, int64_t n_ld,
                                  int HI, int normalize, float scale, int m, const int32_t* ctr, cudaStream_t s);

extern "C" int64_t kch_decode_indexer_workspace_bytes(int B, int64_t capacity) {
  if (B < 1 || capacity < 1) return 0;
  return (int64_t)B * ((capacity + 3) & ~3LL) * 4;
}

extern "C" int kch_decode_indexer_topk(const void* q_idx, int q_dtype, int64_t q_ld, const void* keys, int k_dtype,
                                       const float* k_norms, const void* w, int w_dtype, int64_t w_ld,
                                       int32_t* idx_out, int B, int64_t capacity, int HI, int DI,
                                       int topk, int normalize, float scale, int m, const int32_t* counters,
                                       void* workspace, int64_t workspace_bytes, void* stream) {
  KCH_REQUIRE(topk >= 1, "kch_decode_indexer_topk: topk=%d must be >= 1", topk);
  KCH_REQUIRE(DI >= 1 && HI >= 1 && HI <= 64 && (int64_t)HI * DI <= DIX_MAX_HD,
              "kch_decode_indexer_topk: nIh=%d c_I=%d (needs nIh <= 64, nIh*c_I <= 1024)", HI, DI);
  KCH_REQUIRE(B >= 1 && capacity >= 1 && m >= 1, "kch_decode_indexer_topk: B=%d capacity=%lld m=%d", B, (long long)capacity, m);
  KCH_REQUIRE(k_dtype == KCH_F32 || k_dtype == KCH_BF16, "kch_decode_indexer_topk: k_dtype=%d", k_dtype);
  KCH_REQUIRE((q_dtype == KCH_F32 || q_dtype == KCH_BF16) && (!w || w_dtype == KCH_F32 || w_dtype == KCH_BF16),
              "kch_decode_indexer_topk: q_dtype=%d w_dtype=%d", q_dtype, w_dtype);
  KCH_REQUIRE(q_ld >= (int64_t)HI * DI && (!w || w_ld >= HI), "kch_decode_indexer_topk: q_ld=%lld w_ld=%lld",
              (long long)q_ld, (long long)w_ld);
  KCH_REQUIRE(q_idx && keys && idx_out && counters && (!normalize || k_norms), "kch_decode_indexer_topk: null operand");
  KCH_REQUIRE(workspace && workspace_bytes >= kch_decode_indexer_workspace_bytes(B, capacity),
              "kch_decode_indexer_topk: workspace %lld < %lld bytes", (long long)workspace_bytes,
              (long long)kch_decode_indexer_workspace_bytes(B, capacity));
  cudaStream_t s = kch_stream(stream);
  const int64_t n_ld = (capacity + 3) & ~3LL;
  float* logits = (float*)workspace;
  dim3 grid((unsigned)((capacity + DIX_ROWS - 1) / DIX_ROWS), B);
  const int epl = k_dtype == KCH_BF16 ? 8 : 4;
  const int lpr = DI % epl == 0 ? DI / epl : 0;
  const bool vec = lpr >= 1 && lpr <= 32 && (lpr & (lpr - 1)) == 0 && ((uintptr_t)keys & 15) == 0;
#define GO(T_, V_) decode_indexer_logits_kernel<T_, V_><<<grid, 256, 0, s>>>(q_idx, q_dtype, q_ld, (const T_*)keys, k_norms, \
      w, w_dtype, w_ld, logits, capacity, n_ld, HI, DI, normalize, scale, m, counters)
  static const bool force_simt = [] { const char* e = getenv("KCH_INDEXER_DECODE"); return e && e[0] == 's'; }();
  // (KCH_INDEXER_DECODE=m keeps the mma.sync kernel, =s the scalar one, for comparison)
  static const bool force_mma = [] { const char* e = getenv("KCH_INDEXER_DECODE"); return e && e[0] == 'm'; }();
  int tc5_rc = -100;
  if (!force_simt && !force_mma && k_dtype == KCH_BF16 && DI == 64 && HI <= 8)
    tc5_rc = kch_decode_indexer_logits_tc5(q_idx, q_dtype, q_ld, keys, k_norms, w, w_dtype, w_ld, logits, B, capacity, n_ld, HI,
                                           normalize, scale, m, counters, s);
  if (tc5_rc != -100) {
    if (tc5_rc != KCH_OK) return tc5_rc;
  } else {
    if (!force_simt && k_dtype == KCH_BF16 && DI == 64 && HI <= 8 && ((uintptr_t)keys & 15) == 0)
      decode_indexer_logits_mma_kernel<<<grid, 256, 0, s>>>(q_idx, q_dtype, q_ld, (const bf16*)keys, k_norms, w, w_dtype, w_ld,
                                                            logits, capacity, n_ld, HI, normalize, scale, m, counters);
    else if (k_dtype == KCH_BF16) { if (vec) GO(bf16, true); else GO(bf16, false); }
    else { if (vec) GO(float, true); else GO(float, false); }
    KCH_LAUNCH_OK();
  }
#undef GO
  // rows of up to 8 x 256 x 32 logits: a cluster of eight CTAs per row (KCH_SELECT_DECODE=s keeps one CTA per row)
  static const bool one_cta = [] { const char* e = getenv("KCH_SELECT_DECODE"); return e && e[0] == 's'; }();
  const int e_needed = (int)((((capacity + SC_CTAS * 256 - 1) / (SC_CTAS * 256)) + 3) & ~3LL);
  if (!one_cta && e_needed <= 32 && (((uintptr_t)logits) & 15) == 0)
    return launch_topk_select_cluster(logits, idx_out, B, n_ld, topk, counters, m, e_needed, s);
  // the whole row of logits is staged in shared memory when it fits (one CTA per SM at the largest size)
  const int cache_cap = (int)(n_ld <= 49152 ? ((n_ld + 1023) & ~1023LL) : 0);
  KCH_CUDA_OK(cudaFuncSetAttribute(topk_select_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, cache_cap * 4));
  topk_select_kernel<1024><<<(unsigned)B, 1024, (size_t)cache_cap * 4, s>>>(logits, idx_out, 1, (int)capacity, n_ld, topk, m, 0,
                                                                            -1, 0, cache_cap, counters, m);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
