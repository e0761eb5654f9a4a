// Chunked KDA (naive_chunk_kda, ops_kda.py:340-536) on tensor cores for the production geometry:
// bf16 inputs, K = V = 128, chunks of 64 tokens.  Same mathematics as the fp32 CUDA-core kernels in
// kda.cu; every tensor-core product uses a two-term bf16 split of both operands (hi*hi + lo*hi + hi*lo,
// ~16 bits of mantissa) with fp32 accumulation, so results stay within fp32 round-off of the exact form.
//
// Stage 1, kda_prepare_mma_kernel (one CTA per (batch, value head, chunk), fully parallel):
//   gamma = cumsum(g).  A[i,j] = beta_i sum_k k_i k_j e^{gamma_i - gamma_j} and Aqk are built in 16x16
//   blocks; the exponent difference is factored around a reference row that lies between j and i (the
//   last row of the column block, or the middle row of a diagonal block), so both factors stay
//   representable for every log-decay down to -10 per token.  (I+A)^-1 by block forward substitution,
//   then w = T diag(beta) (e^gamma k) and u = T diag(beta) v as tensor-core products.  Everything the
//   sequential stage needs is written as ready-to-use shared-memory images (swizzled bf16 hi/lo tiles).
// Stage 2, kda_scan_mma_kernel (one CTA per (batch, value head, 64 value columns), sequential in chunks):
//   the state slice S^T [64 v x 128 k] lives in fp32 MMA accumulators for the whole sequence; a producer
//   warp streams the chunk's tiles with 1-D TMA bulk copies through a 12-stage mbarrier ring:
//     vt^T = u^T - S^T w^T ;  o^T = S^T qg^T + vt^T Aqk^T ;  S^T <- S^T diag(dl) + vt^T kg
//   Accumulator fragments are re-used directly as A operands (their column index is the next product's
//   contraction index), so the state never leaves registers.
#include <math.h>
#include <stdlib.h>

#include "mma_utils.cuh"

#define KM_K 128
#define KM_V 128
#define KM_C 64
#define KM_TILE 16384          // one [64][128] bf16 tile
#define KM_OFF_WHI 0
#define KM_OFF_WLO 16384
#define KM_OFF_QHI 32768
#define KM_OFF_QLO 49152
#define KM_OFF_AQK 65536       // hi [64][64] bf16 then lo
#define KM_OFF_KHI 81920
#define KM_OFF_KLO 98304
#define KM_OFF_U 114688        // per 64-column slice: u^T [64 v][64 tok] fp32, then dl [128] fp32
#define KM_U_SLICE 16896
#define KM_CHUNK_BYTES (KM_OFF_U + (KM_V / 64) * KM_U_SLICE)
#define KM_STAGES 12
#define KM_STAGE_BYTES KM_U_SLICE
#define KM_SPIN (1u << 26)

// =====================================================================================
// Stage 1
// =====================================================================================
struct PrepArgs {
  const bf16 *q, *k, *v, *g, *beta;
  uint8_t* ws;
  int T, H, HV, NT;                  // T: tokens from the first chunk of this launch to the end of the sequence
  int Tb;                            // tokens between consecutive batch entries (the whole sequence length)
  float scale, g_min;
  float gate_scale;                  // != 0: g holds the gate's pre-activation x; the decay is -softplus(x) * gate_scale
  int umma;                          // 1: operand tiles in the tcgen05 layout (see kda_scan_tc5.cu) instead of the ldmatrix one
  int64_t ld_qk, ld_v, ld_g, ld_b;   // elements between consecutive tokens
};

// shared-memory map of the prepare kernel (bytes)
#define PS_GLD 136                              // gamma row stride (floats): fragment-pattern reads are conflict-free
#define PS_G 0                                  // gamma fp32 [64][136]            34816
#define PS_A (PS_G + 34816)                     // A fp32 [64][68]                 17408
#define PS_T (PS_A + 17408)                     // (I+A)^-1 fp32 [64][68]          17408
#define PS_ST (PS_T + 17408)                    // first 24576 bytes of the e^gamma k tiles (see PS_EK)
#define PS_Q (PS_ST + 24576)                    // Aqk fp32 [64][68]               17408
#define PS_BETA (PS_Q + 17408)                  // beta [64], scratch P [3][16][17]
#define PS_TOTAL (PS_BETA + 256 + 3 * 16 * 17 * 4)
#define PS_LD 68
#define PS_KLD 136                              // row stride of the bf16 k / q tiles (elements)
#define PS_KQ PS_T                              // k then q tile [64][136] bf16, 2 x 17408 bytes (over T + ST)
// aliases (valid after the producers of the aliased regions are dead)
#define PS_EK PS_ST                             // e^gamma k hi [64][128] bf16 then lo   (over ST + Q)
#define PS_V PS_G                               // v bf16 [64][128]                     (over gamma, first half)
#define PS_TB (PS_G + 16384)                    // T diag(beta) hi [64][64] bf16 then lo (over gamma, second half)
#define PS_U PS_A                               // u^T staging 2 x [64][64] fp32        (over A + T)

#define KM_LOG2E 1.4426950408889634f

// One chunk on the mma.sync path; `sm` needs PS_TOTAL bytes, 128-byte aligned.  Any log-decay down to the clamp.
__device__ __forceinline__ void kda_prepare_chunk_mma(const PrepArgs& a, uint8_t* sm, const int n, const int hv, const int b) {
  float* sG = reinterpret_cast<float*>(sm + PS_G);     // gamma in log2 units: exp(x) == ex2_fast(x')
  float* sA = reinterpret_cast<float*>(sm + PS_A);
  float* sT = reinterpret_cast<float*>(sm + PS_T);
  float* sQ = reinterpret_cast<float*>(sm + PS_Q);
  float* sbeta = reinterpret_cast<float*>(sm + PS_BETA);
  float* sP = sbeta + 64;
  const int G = a.HV / a.H, h = hv / G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g4 = lane >> 2, j4 = lane & 3;
  const int t0 = n * KM_C;
  const int64_t bh = (int64_t)b * a.HV + hv;
  uint8_t* wsc = a.ws + (bh * a.NT + n) * (int64_t)KM_CHUNK_BYTES;
  auto qk_off = [&](int i) { return ((int64_t)b * a.Tb + t0 + i) * a.ld_qk + (int64_t)h * KM_K; };
  auto g_off = [&](int i) { return ((int64_t)b * a.Tb + t0 + i) * a.ld_g + (int64_t)hv * KM_K; };
  auto v_off = [&](int i) { return ((int64_t)b * a.Tb + t0 + i) * a.ld_v + (int64_t)hv * KM_V; };
  auto load8 = [&](const bf16* p, bool ok, float (&out)[8]) {
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (ok) raw = *reinterpret_cast<const uint4*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int x = 0; x < 8; ++x) out[x] = __bfloat162float(e[x]);
  };

  // ---- clamped log-decay into shared memory (log2 units), then the running sum per channel --------
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = tid + 256 * it, i = idx >> 4, ch = idx & 15;
    float gv[8];
    load8(a.g + g_off(i) + 8 * ch, t0 + i < a.T, gv);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      float gx = gv[x];
      if (a.gate_scale != 0.f) {
        // the gate activation of the layer (ops_fused.py:575-578) with its bf16 rounding points, as the GEMM
        // epilogue would have applied it: round(-round(softplus(x)) * scale)
        const float sp = __bfloat162float(__float2bfloat16_rn(gx > 20.f ? gx : __logf(1.0f + __expf(gx))));
        gx = __bfloat162float(__float2bfloat16_rn(-sp * a.gate_scale));
      }
      gv[x] = (t0 + i < a.T) ? fmaxf(gx, a.g_min) * KM_LOG2E : 0.f;
    }
    float4* dst = reinterpret_cast<float4*>(sG + i * PS_GLD + 8 * ch);
    dst[0] = make_float4(gv[0], gv[1], gv[2], gv[3]);
    dst[1] = make_float4(gv[4], gv[5], gv[6], gv[7]);
  }
  if (tid < KM_C) sbeta[tid] = (t0 + tid < a.T) ? __bfloat162float(a.beta[((int64_t)b * a.Tb + t0 + tid) * a.ld_b + hv]) : 0.f;
  for (int idx = tid; idx < KM_C * PS_LD; idx += 256) { sA[idx] = 0.f; sQ[idx] = 0.f; }
  // Every elementwise stage below maps thread -> (row r0 + 16*s, 8-channel chunk c8) with r0 = tid/16 and
  // c8 = tid%16, so the k and q values a thread ever needs are these 4 x 8: keep them in registers.
  const int r0 = tid >> 4, c8 = tid & 15;
  uint4 kreg[4], qreg[4];
#pragma unroll
  for (int s4 = 0; s4 < 4; ++s4) {
    const int i = r0 + 16 * s4;
    kreg[s4] = make_uint4(0u, 0u, 0u, 0u);
    qreg[s4] = make_uint4(0u, 0u, 0u, 0u);
    if (t0 + i < a.T) {
      kreg[s4] = *reinterpret_cast<const uint4*>(a.k + qk_off(i) + 8 * c8);
      qreg[s4] = *reinterpret_cast<const uint4*>(a.q + qk_off(i) + 8 * c8);
    }
  }
  // the same rows as bf16 tiles in shared memory for the fragment-pattern reads of the A / Aqk stage (row stride
  // 136 elements: conflict-free); they live over T and the e^gamma k area, both unused until that stage is over
  bf16* sKt = reinterpret_cast<bf16*>(sm + PS_KQ);
  bf16* sQt = sKt + KM_C * PS_KLD;
#pragma unroll
  for (int s4 = 0; s4 < 4; ++s4) {
    const int i = r0 + 16 * s4;
    *reinterpret_cast<uint4*>(sKt + i * PS_KLD + 8 * c8) = kreg[s4];
    *reinterpret_cast<uint4*>(sQt + i * PS_KLD + 8 * c8) = qreg[s4];
  }
  auto unpack8 = [](const uint4& raw, float (&out)[8]) {
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int x = 0; x < 8; ++x) out[x] = __bfloat162float(e[x]);
  };
  __syncthreads();
  {
    // running sum over the 64 rows: two 32-row segments per channel in parallel, then the second segment adds
    // the first one's total (independent adds)
    const int cch = tid & (KM_K - 1), seg = tid >> 7;
    float acc = 0.f;
#pragma unroll 8
    for (int i = 32 * seg; i < 32 * seg + 32; ++i) {
      acc += sG[i * PS_GLD + cch];
      sG[i * PS_GLD + cch] = acc;
    }
    __syncthreads();
    if (seg == 1) {
      const float base = sG[31 * PS_GLD + cch];
#pragma unroll 8
      for (int i = 32; i < 64; ++i) sG[i * PS_GLD + cch] += base;
    }
  }
  __syncthreads();

  // ---- A and Aqk, block by block ------------------------------------------------------------------
  // 40 independent warp tasks (block pair, 8-column half, contraction half): a warp builds its operand fragments in
  // registers, straight in the mma.sync layout, from gamma (shared memory) and the bf16 rows of k / q (L1), so
  // the whole stage needs no staging tiles and no block barrier.  Row operand: x_i e^{gamma_i - gamma_ref};
  // column operand: k_j e^{gamma_ref - gamma_j}; ref is the middle row of a diagonal block, else the last row of
  // the column block, which keeps both factors representable for every log-decay down to -10 per token.
  {
    const int pa[10] = {0, 1, 2, 3, 1, 2, 3, 2, 3, 3};
    const int pb[10] = {0, 1, 2, 3, 0, 1, 2, 0, 1, 0};
    auto lo16 = [](uint32_t u) { return __uint_as_float(u << 16); };
    auto hi16 = [](uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); };
    for (int task = warp; task < 40; task += 8) {
      // task = (block pair, 8-column half, half of the contraction): A and Aqk together, since they share the
      // column operand and every decay factor; the two contraction halves meet through shared-memory adds
      const int p = task >> 2, nt = (task >> 1) & 1, khalf = task & 1;
      const int ba = pa[p], bb = pb[p];
      const int refrow = (ba == bb) ? (16 * ba + 8) : (16 * bb + 15);
      const int i0 = 16 * ba + g4, i1 = i0 + 8;          // accumulator / row-operand rows of this thread
      const int jn = 16 * bb + 8 * nt + g4;              // the k row that is column g4 of the column operand
      const bf16* k0p = sKt + i0 * PS_KLD;
      const bf16* k1p = sKt + i1 * PS_KLD;
      const bf16* q0p = sQt + i0 * PS_KLD;
      const bf16* q1p = sQt + i1 * PS_KLD;
      const bf16* cjp = sKt + jn * PS_KLD;
      const float* gref = sG + refrow * PS_GLD;
      const float* gi0 = sG + i0 * PS_GLD;
      const float* gi1 = sG + i1 * PS_GLD;
      const float* gj = sG + jn * PS_GLD;
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f}, d2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int ks = 4 * khalf; ks < 4 * khalf + 4; ++ks) {
        uint32_t ah[4], al[4], qh[4], ql[4], bh[2], bl[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {             // k index pairs 16ks + 2j4 (+8)
          const int kk = 16 * ks + 8 * half + 2 * j4;
          const float2 gr = *reinterpret_cast<const float2*>(gref + kk);
          const float2 g0 = *reinterpret_cast<const float2*>(gi0 + kk);
          const float2 g1 = *reinterpret_cast<const float2*>(gi1 + kk);
          const float2 gc = *reinterpret_cast<const float2*>(gj + kk);
          const uint32_t x0 = *reinterpret_cast<const uint32_t*>(k0p + kk);
          const uint32_t x1 = *reinterpret_cast<const uint32_t*>(k1p + kk);
          const uint32_t y0 = *reinterpret_cast<const uint32_t*>(q0p + kk);
          const uint32_t y1 = *reinterpret_cast<const uint32_t*>(q1p + kk);
          const uint32_t xc = *reinterpret_cast<const uint32_t*>(cjp + kk);
          const float e0x = ex2_fast(g0.x - gr.x), e0y = ex2_fast(g0.y - gr.y);
          const float e1x = ex2_fast(g1.x - gr.x), e1y = ex2_fast(g1.y - gr.y);
          split2_bf16(lo16(x0) * e0x, hi16(x0) * e0y, ah[2 * half], al[2 * half]);
          split2_bf16(lo16(x1) * e1x, hi16(x1) * e1y, ah[2 * half + 1], al[2 * half + 1]);
          split2_bf16(lo16(y0) * a.scale * e0x, hi16(y0) * a.scale * e0y, qh[2 * half], ql[2 * half]);
          split2_bf16(lo16(y1) * a.scale * e1x, hi16(y1) * a.scale * e1y, qh[2 * half + 1], ql[2 * half + 1]);
          split2_bf16(lo16(xc) * ex2_fast(gr.x - gc.x), hi16(xc) * ex2_fast(gr.y - gc.y), bh[half], bl[half]);
        }
        mma_bf16_16816(c0, ah, bh[0], bh[1]);
        mma_bf16_16816(d0, qh, bh[0], bh[1]);
        mma_bf16_16816(c1, al, bh[0], bh[1]);
        mma_bf16_16816(d1, ql, bh[0], bh[1]);
        mma_bf16_16816(c2, ah, bl[0], bl[1]);
        mma_bf16_16816(d2, qh, bl[0], bl[1]);
      }
      const int jc = 16 * bb + 8 * nt + 2 * j4;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = (e & 2) ? i1 : i0, jj = jc + (e & 1);
        if (jj < i) atomicAdd(&sA[i * PS_LD + jj], (c0[e] + (c1[e] + c2[e])) * sbeta[i]);
        if (jj <= i) atomicAdd(&sQ[i * PS_LD + jj], d0[e] + (d1[e] + d2[e]));
      }
    }
  }
  __syncthreads();

  // ---- Aqk -> workspace as swizzled bf16 hi/lo tiles [64][64] --------------------------------------
  for (int idx = tid; idx < KM_C * 8; idx += 256) {
    const int i = idx >> 3, ch = idx & 7;
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) split2_bf16(sQ[i * PS_LD + 8 * ch + 2 * e], sQ[i * PS_LD + 8 * ch + 2 * e + 1], hi[e], lo[e]);
    const uint32_t off = swz<128>(i, ch);
    *reinterpret_cast<uint4*>(wsc + KM_OFF_AQK + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4*>(wsc + KM_OFF_AQK + 8192 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
  __syncthreads();   // sQ is dead from here: the e^gamma k tiles may overwrite it

  // ---- qg, kg (workspace), e^gamma k (shared), dl ------------------------------------------------------
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = tid + 256 * it, i = idx >> 4, ch = idx & 15;
    float kf[8], qf[8], gm[8], gl[8];
    unpack8(kreg[it], kf);
    unpack8(qreg[it], qf);
    {
      const float4* p4 = reinterpret_cast<const float4*>(sG + i * PS_GLD + 8 * ch);
      float4 x = p4[0], y = p4[1];
      gm[0] = x.x; gm[1] = x.y; gm[2] = x.z; gm[3] = x.w; gm[4] = y.x; gm[5] = y.y; gm[6] = y.z; gm[7] = y.w;
      p4 = reinterpret_cast<const float4*>(sG + (KM_C - 1) * PS_GLD + 8 * ch);
      x = p4[0]; y = p4[1];
      gl[0] = x.x; gl[1] = x.y; gl[2] = x.z; gl[3] = x.w; gl[4] = y.x; gl[5] = y.y; gl[6] = y.z; gl[7] = y.w;
    }
    uint32_t qh[4], ql[4], kh[4], kl[4], eh[4], el[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float e0 = ex2_fast(gm[2 * e]), e1 = ex2_fast(gm[2 * e + 1]);
      split2_bf16(qf[2 * e] * a.scale * e0, qf[2 * e + 1] * a.scale * e1, qh[e], ql[e]);
      split2_bf16(kf[2 * e] * ex2_fast(gl[2 * e] - gm[2 * e]), kf[2 * e + 1] * ex2_fast(gl[2 * e + 1] - gm[2 * e + 1]), kh[e], kl[e]);
      split2_bf16(kf[2 * e] * e0, kf[2 * e + 1] * e1, eh[e], el[e]);
    }
    const uint32_t off = swz<256>(i, ch);
    if (a.umma) {
      // tcgen05 operand layout: 64-channel panels of 128-byte rows under the 128-byte swizzle.  Rows 0..63 of a
      // [w; qg] panel hold w, rows 64..127 hold qg (hi panels at 0, lo panels at 32768); kg keeps tokens as rows
      // (the state update reads it as an MN-major operand).
      const uint32_t pan = (uint32_t)(ch >> 3), inner = swz<128>(i, ch & 7);
      *reinterpret_cast<uint4*>(wsc + pan * 16384u + 8192u + inner) = make_uint4(qh[0], qh[1], qh[2], qh[3]);
      *reinterpret_cast<uint4*>(wsc + 32768u + pan * 16384u + 8192u + inner) = make_uint4(ql[0], ql[1], ql[2], ql[3]);
      *reinterpret_cast<uint4*>(wsc + KM_OFF_KHI + pan * 8192u + inner) = make_uint4(kh[0], kh[1], kh[2], kh[3]);
      *reinterpret_cast<uint4*>(wsc + KM_OFF_KLO + pan * 8192u + inner) = make_uint4(kl[0], kl[1], kl[2], kl[3]);
    } else {
      *reinterpret_cast<uint4*>(wsc + KM_OFF_QHI + off) = make_uint4(qh[0], qh[1], qh[2], qh[3]);
      *reinterpret_cast<uint4*>(wsc + KM_OFF_QLO + off) = make_uint4(ql[0], ql[1], ql[2], ql[3]);
      *reinterpret_cast<uint4*>(wsc + KM_OFF_KHI + off) = make_uint4(kh[0], kh[1], kh[2], kh[3]);
      *reinterpret_cast<uint4*>(wsc + KM_OFF_KLO + off) = make_uint4(kl[0], kl[1], kl[2], kl[3]);
    }
    *reinterpret_cast<uint4*>(sm + PS_EK + off) = make_uint4(eh[0], eh[1], eh[2], eh[3]);
    *reinterpret_cast<uint4*>(sm + PS_EK + KM_TILE + off) = make_uint4(el[0], el[1], el[2], el[3]);
  }
  if (tid < KM_K) {
    const float dl = ex2_fast(sG[(KM_C - 1) * PS_GLD + tid]);
    if (a.umma) {
      reinterpret_cast<float*>(wsc + KM_OFF_U + 32768)[tid] = dl;
    } else {
#pragma unroll
      for (int s = 0; s < KM_V / 64; ++s)
        reinterpret_cast<float*>(wsc + KM_OFF_U + s * KM_U_SLICE + 16384)[tid] = dl;
    }
  }

  // ---- (I + A)^-1 by block forward substitution (fp32, CUDA cores) ------------------------------------
  // blocks above the diagonal are zero (the area held the k / q tiles until now); nothing else writes them
  for (int idx = tid; idx < 6 * 256; idx += 256) {
    const int bi = idx >> 8, r = (idx >> 4) & 15, cc = idx & 15;
    const int ub_a[6] = {0, 0, 0, 1, 1, 2}, ub_b[6] = {1, 2, 3, 2, 3, 3};
    sT[(16 * ub_a[bi] + r) * PS_LD + 16 * ub_b[bi] + cc] = 0.f;
  }
  // diagonal 16x16 blocks: four lanes per (block, column); lane q keeps the solved entries x_s with s = q (mod 4)
  // in registers and contributes their part of each row's dot product, two shuffles complete it
  {
    const int col = tid >> 2, q4 = tid & 3;
    const int blk = col >> 4, cc = col & 15, base = 16 * blk;
    float xs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      float acc = 0.f;
#pragma unroll
      for (int m4 = 0; m4 < 4; ++m4) {
        const int sidx = 4 * m4 + q4;
        if (sidx < r && sidx >= cc) acc = fmaf(sA[(base + r) * PS_LD + base + sidx], xs[m4], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      const float x = (r == cc) ? 1.f : (r > cc ? -acc : 0.f);
      if ((r & 3) == q4) xs[r >> 2] = x;
      if (q4 == 0) sT[(base + r) * PS_LD + base + cc] = x;
    }
  }
  __syncthreads();
  // off-diagonal blocks, by distance d from the diagonal:  T_ab = -T_aa (sum_{b<=c<a} A_ac T_cb)
  for (int d = 1; d < 4; ++d) {
    const int nblk = 4 - d;
    for (int idx = tid; idx < nblk * 256; idx += 256) {
      const int bi = idx >> 8, r = (idx >> 4) & 15, cc = idx & 15;
      const int ba = bi + d, bb = bi;
      float acc = 0.f;
      for (int cblk = bb; cblk < ba; ++cblk)
#pragma unroll 4
        for (int s = 0; s < 16; ++s)
          acc = fmaf(sA[(16 * ba + r) * PS_LD + 16 * cblk + s], sT[(16 * cblk + s) * PS_LD + 16 * bb + cc], acc);
      sP[(bi * 16 + r) * 17 + cc] = acc;
    }
    __syncthreads();
    for (int idx = tid; idx < nblk * 256; idx += 256) {
      const int bi = idx >> 8, r = (idx >> 4) & 15, cc = idx & 15;
      const int ba = bi + d, bb = bi;
      float acc = 0.f;
#pragma unroll 4
      for (int s = 0; s <= r; ++s) acc = fmaf(sT[(16 * ba + r) * PS_LD + 16 * ba + s], sP[(bi * 16 + s) * 17 + cc], acc);
      sT[(16 * ba + r) * PS_LD + 16 * bb + cc] = -acc;
    }
    __syncthreads();
  }
  // T diag(beta) as swizzled bf16 hi/lo tiles (over the dead gamma buffer), v tile next to it
  for (int idx = tid; idx < KM_C * 8; idx += 256) {
    const int i = idx >> 3, ch = idx & 7;
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int jj = 8 * ch + 2 * e;
      split2_bf16(sT[i * PS_LD + jj] * sbeta[jj], sT[i * PS_LD + jj + 1] * sbeta[jj + 1], hi[e], lo[e]);
    }
    const uint32_t off = swz<128>(i, ch);
    *reinterpret_cast<uint4*>(sm + PS_TB + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4*>(sm + PS_TB + 8192 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = tid + 256 * it, i = idx >> 4, ch = idx & 15;
    uint4 vr = make_uint4(0u, 0u, 0u, 0u);
    if (t0 + i < a.T) vr = *reinterpret_cast<const uint4*>(a.v + v_off(i) + 8 * ch);
    *reinterpret_cast<uint4*>(sm + PS_V + swz<256>(i, ch)) = vr;
  }
  __syncthreads();

  // ---- w = Tb (e^gamma k), u = Tb v : warp = (16-row tile, half of the 128 columns); lower-triangular k-steps ----
  const int mt = warp & 3, nh = warp >> 2;
  float wacc[8][4], uacc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) { wacc[i][0] = wacc[i][1] = wacc[i][2] = wacc[i][3] = 0.f; uacc[i][0] = uacc[i][1] = uacc[i][2] = uacc[i][3] = 0.f; }
  {
    const uint32_t tbh = smem_addr_u32(sm + PS_TB), tbl = tbh + 8192;
    const uint32_t ekh = smem_addr_u32(sm + PS_EK), ekl = ekh + KM_TILE, vv = smem_addr_u32(sm + PS_V);
    const int arow = 16 * mt + (lane & 7) + ((lane >> 3) & 1) * 8;
    for (int ks = 0; ks <= mt; ++ks) {
      uint32_t ah[4], al[4];
      const uint32_t oa = swz<128>(arow, 2 * ks + (lane >> 4));
      ldmatrix_x4(tbh + oa, ah[0], ah[1], ah[2], ah[3]);
      ldmatrix_x4(tbl + oa, al[0], al[1], al[2], al[3]);
      const int brow = 16 * ks + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dpl = 0; dpl < 4; ++dpl) {
        const uint32_t ob = swz<256>(brow, 2 * (4 * nh + dpl) + (lane >> 4));
        uint32_t h0, h1, h2, h3, l0, l1, l2, l3, v0, v1, v2, v3;
        ldmatrix_x4_trans(ekh + ob, h0, h1, h2, h3);
        ldmatrix_x4_trans(ekl + ob, l0, l1, l2, l3);
        ldmatrix_x4_trans(vv + ob, v0, v1, v2, v3);
        mma_bf16_16816(wacc[2 * dpl], ah, h0, h1);     mma_bf16_16816(wacc[2 * dpl + 1], ah, h2, h3);
        mma_bf16_16816(wacc[2 * dpl], al, h0, h1);     mma_bf16_16816(wacc[2 * dpl + 1], al, h2, h3);
        mma_bf16_16816(wacc[2 * dpl], ah, l0, l1);     mma_bf16_16816(wacc[2 * dpl + 1], ah, l2, l3);
        mma_bf16_16816(uacc[2 * dpl], ah, v0, v1);     mma_bf16_16816(uacc[2 * dpl + 1], ah, v2, v3);
        mma_bf16_16816(uacc[2 * dpl], al, v0, v1);     mma_bf16_16816(uacc[2 * dpl + 1], al, v2, v3);
      }
    }
  }
  // w -> workspace (swizzled hi/lo); u^T -> shared staging (over A and T, dead now) -> workspace
  {
    const int i0 = 16 * mt + g4, i1 = i0 + 8;
    float* us = reinterpret_cast<float*>(sm + PS_U);
#pragma unroll
    for (int ntl = 0; ntl < 8; ++ntl) {
      const int nt = 8 * nh + ntl;
      uint32_t hi, lo;
      split2_bf16(wacc[ntl][0], wacc[ntl][1], hi, lo);
      const uint32_t ow0 = a.umma ? (uint32_t)(nt >> 3) * 16384u + swz<128>(i0, nt & 7) : swz<256>(i0, nt);
      const uint32_t ow1 = a.umma ? (uint32_t)(nt >> 3) * 16384u + swz<128>(i1, nt & 7) : swz<256>(i1, nt);
      const uint32_t wlo = a.umma ? 32768u : (uint32_t)KM_OFF_WLO;
      *reinterpret_cast<uint32_t*>(wsc + KM_OFF_WHI + ow0 + 4 * j4) = hi;
      *reinterpret_cast<uint32_t*>(wsc + wlo + ow0 + 4 * j4) = lo;
      split2_bf16(wacc[ntl][2], wacc[ntl][3], hi, lo);
      *reinterpret_cast<uint32_t*>(wsc + KM_OFF_WHI + ow1 + 4 * j4) = hi;
      *reinterpret_cast<uint32_t*>(wsc + wlo + ow1 + 4 * j4) = lo;
      const int c0 = 8 * nt + 2 * j4;            // value column
      if (a.umma) {
        // u^T as [token / 32][token / 4 % 8][value column][token % 4]: a warp of the scan reads 512 contiguous bytes
        float* s0 = us + ((i0 >> 5) * 8 + ((i0 >> 2) & 7)) * 512 + (i0 & 3) + 4 * c0;
        float* s1 = us + ((i1 >> 5) * 8 + ((i1 >> 2) & 7)) * 512 + (i1 & 3) + 4 * c0;
        s0[0] = uacc[ntl][0];
        s0[4] = uacc[ntl][1];
        s1[0] = uacc[ntl][2];
        s1[4] = uacc[ntl][3];
      } else {
        float* s0 = us + (c0 >> 6) * 4096 + (c0 & 63) * 64;
        s0[i0] = uacc[ntl][0];
        s0[64 + i0] = uacc[ntl][1];
        s0[i1] = uacc[ntl][2];
        s0[64 + i1] = uacc[ntl][3];
      }
    }
  }
  __syncthreads();
  {
    const float4* us4 = reinterpret_cast<const float4*>(sm + PS_U);
#pragma unroll
    for (int s = 0; s < KM_V / 64; ++s) {
      float4* dst = reinterpret_cast<float4*>(wsc + KM_OFF_U + s * (a.umma ? 16384 : KM_U_SLICE));
      for (int idx = tid; idx < 1024; idx += 256) dst[idx] = us4[s * 1024 + idx];
    }
  }
}

__global__ void __launch_bounds__(256, 2) kda_prepare_mma_kernel(PrepArgs a) {
  extern __shared__ __align__(128) uint8_t sm[];
  kda_prepare_chunk_mma(a, sm, blockIdx.x, blockIdx.y, blockIdx.z);
}

#include "kda_prepare_tc5.cuh"

// =====================================================================================
// Stage 2
// =====================================================================================
struct ScanArgs {
  const uint8_t* ws;
  const float* S0;
  bf16* o;
  float* S_out;
  unsigned int* status;
  int T, HV, NT;
};

#define SC_OSTAGE (KM_STAGES * KM_STAGE_BYTES)          // 4 warps x [64 tok][16 v] bf16
#define SC_BARS (SC_OSTAGE + 4 * 64 * 16 * 2)
#define SC_TOTAL (SC_BARS + 2 * KM_STAGES * 8)

__global__ void __launch_bounds__(160, 1) kda_scan_mma_kernel(ScanArgs a) {
  extern __shared__ __align__(1024) uint8_t sm[];
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + SC_BARS);
  uint64_t* empty = full + KM_STAGES;
  const int vs = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g4 = lane >> 2, j4 = lane & 3;
  const int64_t bh = (int64_t)b * a.HV + hv;
  const uint8_t* wsb = a.ws + bh * a.NT * (int64_t)KM_CHUNK_BYTES;
  if (threadIdx.x == 0) {
    for (int s = 0; s < KM_STAGES; ++s) { mbarrier_init(&full[s], 1); mbarrier_init(&empty[s], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 4) {
    // ---------------- producer: one elected lane streams 8 tiles per chunk ----------------
    if (lane == 0) {
      const uint32_t src_off[8] = {KM_OFF_WHI, KM_OFF_WLO, KM_OFF_QHI, KM_OFF_QLO,
                                   (uint32_t)(KM_OFF_U + vs * KM_U_SLICE), KM_OFF_AQK, KM_OFF_KHI, KM_OFF_KLO};
      uint32_t it = 0;
      bool ok = true;
      for (int n = 0; n < a.NT && ok; ++n) {
        const uint8_t* src = wsb + (int64_t)n * KM_CHUNK_BYTES;
        for (int tl = 0; tl < 8; ++tl, ++it) {
          const uint32_t s = it % KM_STAGES, ph = (it / KM_STAGES) & 1;
          if (!mbarrier_wait_bounded(&empty[s], ph ^ 1, 11, KM_SPIN, a.status)) { ok = false; break; }
          const uint32_t bytes = (tl == 4) ? KM_U_SLICE : KM_TILE;
          mbarrier_expect_tx(&full[s], bytes);
          bulk_copy_g2s(sm + s * KM_STAGE_BYTES, src + src_off[tl], bytes, &full[s]);
        }
      }
      if (!ok) {   // let copies already issued land before the CTA retires
        for (uint32_t back = 0; back < KM_STAGES && back < it; ++back) {
          const uint32_t jt = it - 1 - back;
          mbarrier_wait_bounded(&full[jt % KM_STAGES], (jt / KM_STAGES) & 1, 12, 1u << 20, a.status);
        }
      }
    }
    return;
  }

  // ---------------- consumers: warp w owns value columns vs*64 + 16w .. +15 ----------------
  const int vrow = vs * 64 + 16 * warp;            // global value column of accumulator row 0
  float sacc[16][4];                               // S^T rows (v) g4, g4+8; cols (k) 8nt + 2j4, +1
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const int kc = 8 * nt + 2 * j4;
    if (a.S0) {
      const float* s0 = a.S0 + bh * (KM_K * KM_V);
      sacc[nt][0] = s0[(int64_t)kc * KM_V + vrow + g4];
      sacc[nt][1] = s0[(int64_t)(kc + 1) * KM_V + vrow + g4];
      sacc[nt][2] = s0[(int64_t)kc * KM_V + vrow + g4 + 8];
      sacc[nt][3] = s0[(int64_t)(kc + 1) * KM_V + vrow + g4 + 8];
    } else {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
    }
  }
  bf16* ost = reinterpret_cast<bf16*>(sm + SC_OSTAGE) + warp * (64 * 16);
  bool ok = true;
  auto wait_tile = [&](uint32_t it) -> uint32_t {
    const uint32_t s = it % KM_STAGES;
    if (ok && !mbarrier_wait_bounded(&full[s], (it / KM_STAGES) & 1, 13, KM_SPIN, a.status)) ok = false;
    return smem_addr_u32(sm + s * KM_STAGE_BYTES);
  };
  auto release_tile = [&](uint32_t it) {
    __syncwarp();
    if (lane == 0) mbarrier_arrive(&empty[it % KM_STAGES]);
  };

  for (int n = 0; n < a.NT && ok; ++n) {
    const uint32_t it0 = (uint32_t)n * 8;
    // ======== phase 1: -(S^T w^T) and S^T qg^T =========================================================
    const uint32_t whi = wait_tile(it0 + 0), wlo = wait_tile(it0 + 1), qhi = wait_tile(it0 + 2), qlo = wait_tile(it0 + 3);
    if (!ok) break;
    float accw[8][4], accq[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { accw[i][0] = accw[i][1] = accw[i][2] = accw[i][3] = 0.f; accq[i][0] = accq[i][1] = accq[i][2] = accq[i][3] = 0.f; }
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
      uint32_t ah[2][4], al[2][4];
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int n0 = 4 * qd + 2 * kk;
        split2_bf16(sacc[n0][0], sacc[n0][1], ah[kk][0], al[kk][0]);
        split2_bf16(sacc[n0][2], sacc[n0][3], ah[kk][1], al[kk][1]);
        split2_bf16(sacc[n0 + 1][0], sacc[n0 + 1][1], ah[kk][2], al[kk][2]);
        split2_bf16(sacc[n0 + 1][2], sacc[n0 + 1][3], ah[kk][3], al[kk][3]);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const uint32_t off = swz<256>(8 * nt + (lane & 7), 4 * qd + (lane >> 3));
        // the w and q products are independent accumulator chains: alternate them so that consecutive MMAs
        // never wait on each other's result
        uint32_t h0, h1, h2, h3, l0, l1, l2, l3, g0, g1, g2, g3, m0, m1, m2, m3;
        ldmatrix_x4(whi + off, h0, h1, h2, h3);
        ldmatrix_x4(qhi + off, g0, g1, g2, g3);
        ldmatrix_x4(wlo + off, l0, l1, l2, l3);
        ldmatrix_x4(qlo + off, m0, m1, m2, m3);
        mma_bf16_16816(accw[nt], ah[0], h0, h1); mma_bf16_16816(accq[nt], ah[0], g0, g1);
        mma_bf16_16816(accw[nt], ah[1], h2, h3); mma_bf16_16816(accq[nt], ah[1], g2, g3);
        mma_bf16_16816(accw[nt], al[0], h0, h1); mma_bf16_16816(accq[nt], al[0], g0, g1);
        mma_bf16_16816(accw[nt], al[1], h2, h3); mma_bf16_16816(accq[nt], al[1], g2, g3);
        mma_bf16_16816(accw[nt], ah[0], l0, l1); mma_bf16_16816(accq[nt], ah[0], m0, m1);
        mma_bf16_16816(accw[nt], ah[1], l2, l3); mma_bf16_16816(accq[nt], ah[1], m2, m3);
      }
    }
    release_tile(it0 + 0); release_tile(it0 + 1); release_tile(it0 + 2); release_tile(it0 + 3);
    // ======== vt^T = u^T - S^T w^T, kept as split A fragments for the next two products ================
    const uint32_t ut_addr = wait_tile(it0 + 4);
    if (!ok) break;
    const float* ut = reinterpret_cast<const float*>(sm + (it0 + 4) % KM_STAGES * KM_STAGE_BYTES);
    (void)ut_addr;
    uint32_t vh[4][4], vl[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int nt = 2 * ks + half;
        const float2 u0 = *reinterpret_cast<const float2*>(ut + (16 * warp + g4) * 64 + 8 * nt + 2 * j4);
        const float2 u1 = *reinterpret_cast<const float2*>(ut + (16 * warp + g4 + 8) * 64 + 8 * nt + 2 * j4);
        split2_bf16(u0.x - accw[nt][0], u0.y - accw[nt][1], vh[ks][2 * half], vl[ks][2 * half]);
        split2_bf16(u1.x - accw[nt][2], u1.y - accw[nt][3], vh[ks][2 * half + 1], vl[ks][2 * half + 1]);
      }
    }
    // ======== phase 2: o^T = S^T qg^T + vt^T Aqk^T ====================================================
    const uint32_t aqh = wait_tile(it0 + 5);
    if (!ok) break;
    const uint32_t aql = aqh + 8192;
#pragma unroll
    for (int qd = 0; qd < 2; ++qd) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (8 * nt + 7 < 32 * qd) continue;          // block entirely above the diagonal: zeros
        const uint32_t off = swz<128>(8 * nt + (lane & 7), 4 * qd + (lane >> 3));
        uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
        ldmatrix_x4(aqh + off, h0, h1, h2, h3);
        ldmatrix_x4(aql + off, l0, l1, l2, l3);
        mma_bf16_16816(accq[nt], vh[2 * qd], h0, h1); mma_bf16_16816(accq[nt], vh[2 * qd + 1], h2, h3);
        mma_bf16_16816(accq[nt], vl[2 * qd], h0, h1); mma_bf16_16816(accq[nt], vl[2 * qd + 1], h2, h3);
        mma_bf16_16816(accq[nt], vh[2 * qd], l0, l1); mma_bf16_16816(accq[nt], vh[2 * qd + 1], l2, l3);
      }
    }
    release_tile(it0 + 5);
    // o^T fragments -> [tok][16 v] bf16 staging -> 32-byte row segments of o[b, t, hv, :]
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int tk = 8 * nt + 2 * j4;
      ost[tk * 16 + g4] = __float2bfloat16_rn(accq[nt][0]);
      ost[(tk + 1) * 16 + g4] = __float2bfloat16_rn(accq[nt][1]);
      ost[tk * 16 + g4 + 8] = __float2bfloat16_rn(accq[nt][2]);
      ost[(tk + 1) * 16 + g4 + 8] = __float2bfloat16_rn(accq[nt][3]);
    }
    __syncwarp();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int tk = lane + 32 * half;
      const int t = n * KM_C + tk;
      if (t < a.T) {
        const uint4* src = reinterpret_cast<const uint4*>(ost + tk * 16);
        uint4* dst = reinterpret_cast<uint4*>(a.o + (((int64_t)b * a.T + t) * a.HV + hv) * KM_V + vrow);
        dst[0] = src[0];
        dst[1] = src[1];
      }
    }
    __syncwarp();
    // ======== phase 3: S^T <- S^T diag(dl) + vt^T kg ====================================================
    {
      const float* dl = ut + 4096;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const float2 d = *reinterpret_cast<const float2*>(dl + 8 * nt + 2 * j4);
        sacc[nt][0] *= d.x; sacc[nt][1] *= d.y; sacc[nt][2] *= d.x; sacc[nt][3] *= d.y;
      }
    }
    release_tile(it0 + 4);
    const uint32_t khi = wait_tile(it0 + 6), klo = wait_tile(it0 + 7);
    if (!ok) break;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int brow = 16 * ks + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const uint32_t off = swz<256>(brow, 2 * dp + (lane >> 4));
        uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
        ldmatrix_x4_trans(khi + off, h0, h1, h2, h3);
        ldmatrix_x4_trans(klo + off, l0, l1, l2, l3);
        mma_bf16_16816(sacc[2 * dp], vh[ks], h0, h1); mma_bf16_16816(sacc[2 * dp + 1], vh[ks], h2, h3);
        mma_bf16_16816(sacc[2 * dp], vl[ks], h0, h1); mma_bf16_16816(sacc[2 * dp + 1], vl[ks], h2, h3);
        mma_bf16_16816(sacc[2 * dp], vh[ks], l0, l1); mma_bf16_16816(sacc[2 * dp + 1], vh[ks], l2, l3);
      }
    }
    release_tile(it0 + 6); release_tile(it0 + 7);
  }
  if (a.S_out && ok) {
    float* so = a.S_out + bh * (KM_K * KM_V);
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const int kc = 8 * nt + 2 * j4;
      so[(int64_t)kc * KM_V + vrow + g4] = sacc[nt][0];
      so[(int64_t)(kc + 1) * KM_V + vrow + g4] = sacc[nt][1];
      so[(int64_t)kc * KM_V + vrow + g4 + 8] = sacc[nt][2];
      so[(int64_t)(kc + 1) * KM_V + vrow + g4 + 8] = sacc[nt][3];
    }
  }
}

// ---- host -------------------------------------------------------------------------------------------
bool kch_kda_scan_tc5_enabled();      // kda_scan_tc5.cu
int kch_kda_scan_tc5(const void* workspace, const float* initial_state, void* o, float* final_state, int B, int T,
                     int Tb, int HV, int NT, unsigned int* status, cudaStream_t s);

bool kch_kda_mma_supported(int K, int V, int chunk_size, float g_clamp_min, int dtype) {
  static const bool force_generic = [] { const char* e = getenv("KCH_KDA"); return e && e[0] == 'g'; }();
  return !force_generic && dtype == KCH_BF16 && K == KM_K && V == KM_V && chunk_size == KM_C && g_clamp_min >= -10.0f;
}

// chunk records, then one fp32 state per (batch, head): the carry between the segments of a long sequence
int64_t kch_kda_mma_workspace_bytes(int B, int T, int HV) {
  int64_t NT = (T + KM_C - 1) / KM_C;
  return (int64_t)B * HV * NT * KM_CHUNK_BYTES + (int64_t)B * HV * KM_K * KM_V * 4;
}

// Side stream and events of the segmented driver below (one set per device, created on first use).
#define KM_MAX_SEG 8
struct KmSideStream {
  cudaStream_t hp = nullptr;
  cudaEvent_t prep_done[KM_MAX_SEG] = {};
  cudaEvent_t scan_done = nullptr;
};
static int km_side_stream(KmSideStream** out) {
  static KmSideStream per_dev[16];
  int dev = 0;
  KCH_CUDA_OK(cudaGetDevice(&dev));
  KCH_REQUIRE(dev >= 0 && dev < 16, "kch_kda_chunk: device ordinal %d", dev);
  KmSideStream& ss = per_dev[dev];
  if (!ss.hp) {
    int least = 0, greatest = 0;
    KCH_CUDA_OK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    KCH_CUDA_OK(cudaStreamCreateWithPriority(&ss.hp, cudaStreamNonBlocking, greatest));
    for (int i = 0; i < KM_MAX_SEG; ++i) KCH_CUDA_OK(cudaEventCreateWithFlags(&ss.prep_done[i], cudaEventDisableTiming));
    KCH_CUDA_OK(cudaEventCreateWithFlags(&ss.scan_done, cudaEventDisableTiming));
  }
  *out = &ss;
  return KCH_OK;
}

int kch_kda_chunk_mma(const void* q, const void* k, const void* v, const void* g, const void* beta,
                      const float* initial_state, void* o, float* final_state, int B, int T, int H, int HV,
                      float scale, float g_clamp_min, int64_t ld_qk, int64_t ld_v, int64_t ld_g, int64_t ld_beta,
                      void* workspace, int64_t workspace_bytes, void* stream, float gate_scale) {
  const int NT = (T + KM_C - 1) / KM_C;
  KCH_REQUIRE(workspace && workspace_bytes >= kch_kda_mma_workspace_bytes(B, T, HV),
              "kch_kda_chunk: workspace %lld < %lld bytes", (long long)workspace_bytes,
              (long long)kch_kda_mma_workspace_bytes(B, T, HV));
  KCH_REQUIRE(((uintptr_t)workspace & 15) == 0, "kch_kda_chunk: workspace must be 16-byte aligned");
  unsigned int* status = kch_status_device_ptr();
  KCH_REQUIRE(status != nullptr, "kch_kda_chunk: cannot resolve the device status word");
  cudaStream_t s = kch_stream(stream);
  PrepArgs pa;
  pa.q = (const bf16*)q; pa.k = (const bf16*)k; pa.v = (const bf16*)v; pa.g = (const bf16*)g; pa.beta = (const bf16*)beta;
  pa.ws = (uint8_t*)workspace; pa.T = T; pa.Tb = T; pa.H = H; pa.HV = HV; pa.NT = NT; pa.scale = scale; pa.g_min = g_clamp_min; pa.gate_scale = gate_scale;
  pa.umma = kch_kda_scan_tc5_enabled() ? 1 : 0;
  pa.ld_qk = ld_qk; pa.ld_v = ld_v; pa.ld_g = ld_g; pa.ld_b = ld_beta;
  // 16-byte vector loads: token strides and base pointers must be multiples of 8 elements / 16 bytes
  KCH_REQUIRE((ld_qk % 8) == 0 && (ld_v % 8) == 0 && (ld_g % 8) == 0 &&
              ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)g) & 15) == 0),
              "kch_kda_chunk: q/k/v/g must be 16-byte aligned with token strides that are multiples of 8 elements");
  static const bool prep_mma = [] { const char* e = getenv("KCH_KDA_PREPARE"); return e && e[0] == 'm'; }();
  // Long sequences in segments: the sequential stage holds 64 SMs (one CTA per batch entry and head) for a dependent
  // chain, the parallel stage wants all of them for independent chunks.  Segment i + 1 is prepared on the caller's
  // stream while segment i is scanned on a high-priority side stream (its CTAs take their SMs first at the moment both
  // become runnable; the prepare CTAs fill the rest), the state travels between segments through global memory.
  // (KCH_KDA_SEGMENTS=1 runs the two stages one after the other, for comparison.)
  static const int seg_env = [] { const char* e = getenv("KCH_KDA_SEGMENTS"); return e ? atoi(e) : 0; }();
  int nsegs = seg_env > 0 ? seg_env : (NT >= 64 ? 4 : 1);
  if (nsegs > KM_MAX_SEG) nsegs = KM_MAX_SEG;
  if (nsegs > NT) nsegs = NT > 0 ? NT : 1;
  if (pa.umma && !prep_mma && nsegs > 1) {
    KmSideStream* ss = nullptr;
    int rc = km_side_stream(&ss);
    if (rc != KCH_OK) return rc;
    const int per = (NT + nsegs - 1) / nsegs;
    float* carry = final_state ? final_state
                               : reinterpret_cast<float*>((uint8_t*)workspace + (int64_t)B * HV * NT * KM_CHUNK_BYTES);
    auto seg_args = [&](int i, PrepArgs& sp, int& n0, int& cnt) {
      n0 = i * per;
      cnt = NT - n0 < per ? NT - n0 : per;
      const int64_t tok = (int64_t)n0 * KM_C;
      sp = pa;
      sp.q = pa.q + tok * ld_qk; sp.k = pa.k + tok * ld_qk; sp.v = pa.v + tok * ld_v; sp.g = pa.g + tok * ld_g;
      sp.beta = pa.beta + tok * ld_beta;
      sp.ws = pa.ws + (int64_t)B * HV * n0 * KM_CHUNK_BYTES;
      sp.T = T - (int)tok; sp.NT = cnt;
    };
    PrepArgs sp;
    int n0, cnt;
    seg_args(0, sp, n0, cnt);
    rc = launch_kda_prepare_tc5(sp, B, status, s);
    if (rc != KCH_OK) return rc;
    KCH_CUDA_OK(cudaEventRecord(ss->prep_done[0], s));
    for (int i = 0; i < nsegs && i * per < NT; ++i) {
      seg_args(i, sp, n0, cnt);
      const bool last = (i + 1) * per >= NT;
      KCH_CUDA_OK(cudaStreamWaitEvent(ss->hp, ss->prep_done[i], 0));
      rc = kch_kda_scan_tc5(sp.ws, i == 0 ? initial_state : carry, (bf16*)o + (int64_t)n0 * KM_C * HV * KM_V,
                            last ? final_state : carry, B, sp.T, T, HV, cnt, status, ss->hp);
      if (rc != KCH_OK) return rc;
      if (!last) {
        PrepArgs np;
        int m0, mc;
        seg_args(i + 1, np, m0, mc);
        rc = launch_kda_prepare_tc5(np, B, status, s);
        if (rc != KCH_OK) return rc;
        KCH_CUDA_OK(cudaEventRecord(ss->prep_done[i + 1], s));
      }
    }
    KCH_CUDA_OK(cudaEventRecord(ss->scan_done, ss->hp));
    KCH_CUDA_OK(cudaStreamWaitEvent(s, ss->scan_done, 0));
    return KCH_OK;
  }
  if (pa.umma && !prep_mma) {
    int rc = launch_kda_prepare_tc5(pa, B, status, s);
    if (rc != KCH_OK) return rc;
  } else {
    KCH_CUDA_OK(cudaFuncSetAttribute(kda_prepare_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_TOTAL));
    kda_prepare_mma_kernel<<<dim3(NT, HV, B), 256, PS_TOTAL, s>>>(pa);
    KCH_LAUNCH_OK();
  }
  if (pa.umma) return kch_kda_scan_tc5(workspace, initial_state, o, final_state, B, T, T, HV, NT, status, s);
  ScanArgs sa;
  sa.ws = (const uint8_t*)workspace; sa.S0 = initial_state; sa.o = (bf16*)o; sa.S_out = final_state; sa.status = status;
  sa.T = T; sa.HV = HV; sa.NT = NT;
  KCH_CUDA_OK(cudaFuncSetAttribute(kda_scan_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SC_TOTAL));
  kda_scan_mma_kernel<<<dim3(KM_V / 64, HV, B), 160, SC_TOTAL, s>>>(sa);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
