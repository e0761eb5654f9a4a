// Stage 1 of chunked KDA (naive_chunk_kda, ops_kda.py:388-424 and the per-chunk operands of 509-535) on the
// fifth-generation tensor cores.  Included by kda_mma.cu after kda_prepare_chunk_mma, which stays the path for
// chunks whose decay is too strong for the factorisation below.
//
// With gamma_i[k] the running log-decay inside the chunk (<= 0, log2 units here) every product of the stage is a
// plain matrix product of four element-wise images of k and q:
//     EK = k 2^gamma      QG = scale q 2^gamma      Y = k 2^-gamma      KG = k 2^(gamma_last - gamma)
//     A   = beta_i * tril_-1(EK Y^T)      Aqk = tril(QG Y^T)          one MMA:  [EK; QG] (M = 128) x Y^T (N = 64), K = 128
//     T   = (I + A)^-1 diag(beta)         (fp32, CUDA cores: 16 x 16 diagonal solves + block products)
//     w^T = EK^T T^T                      u^T = V^T T^T               two MMAs: M = 128 channels, N = 64 tokens, K = 64
// 2^-gamma grows as the chunk decays, so the factorisation is used only while gamma_last >= -PT_GMAX for every
// channel (2^96 is far inside the bf16 / fp32 exponent range; the model's gate, -0.1 softplus, stays within a few
// units); entries above the diagonal may overflow but are never read.  Otherwise the CTA runs the mma.sync path,
// which re-centres the exponents per 16 x 16 block.  Each product is hi*hi + lo*hi + hi*lo of two-term bf16 splits
// with fp32 accumulation in tensor memory, as everywhere in the KDA kernels.
//
// Data movement: g, k, q are read once by the threads that turn them into operand images (registers -> swizzled
// shared-memory tiles, the QG / KG images also straight to the chunk record); V arrives through a tensor map
// (cp.async.bulk.tensor, 128-byte swizzle) while the triangular solve runs; w leaves through shared memory as bulk
// copies; u^T and Aqk are written from the tensor-memory epilogues.  EK serves twice: K-major as the row operand of
// the first product, MN-major (the same bytes) as the A operand of the second.
#pragma once
#include <cudaTypedefs.h>

#include "tc5_utils.cuh"

#define PT_AIMG 0                        // [EK; QG] hi: 2 panels of [128 rows][64 ch] bf16 (16384 each), lo at 32768
#define PT_Y 65536                       // Y hi: 2 panels of [64][64] bf16 (8192 each), lo at +16384
#define PT_A PT_Y                        //   after the first product: A fp32 [64][68], T fp32 [64][68] (34816)
#define PT_T (PT_Y + 17408)
#define PT_WST PT_Y                      //   after the second product: w hi panels (2 x 8192), lo panels (2 x 8192)
#define PT_TOT (PT_Y + 34816)            // per 4-row group and channel: sum of the log-decay, fp32 [17][128]
#define PT_BETA (PT_TOT + 17 * 128 * 4)
#define PT_SP (PT_BETA + 256)            // scratch of the block substitution [3][16][17] fp32
#define PT_BARS (PT_SP + 3 * 16 * 17 * 4)
#define PT_TOTAL (PT_BARS + 64)
#define PT_VT (PT_AIMG + 8192)           //   after the first product: V panels over the QG hi rows (16384 apart)
#define PT_TBH (PT_AIMG + 32768 + 8192)  //   T diag(beta) hi [64][64] bf16 over the QG lo rows of panel 0, lo over panel 1
#define PT_TBL (PT_AIMG + 49152 + 8192)
#define PT_DYN 115712                    // two CTAs per SM; the mma.sync path needs PS_TOTAL from the unaligned base
#define PT_GMAX 96.0f
#define PT_SPIN (1u << 24)

static_assert(PT_TOTAL + 1023 <= PT_DYN && PS_TOTAL <= PT_DYN, "shared-memory budget of the prepare kernel");

__global__ void __launch_bounds__(256, 2)
kda_prepare_tc5_kernel(PrepArgs a, const __grid_constant__ CUtensorMap vmap, unsigned int* status) {
  extern __shared__ __align__(128) uint8_t pt_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>(((uintptr_t)pt_raw + 1023) & ~(uintptr_t)1023);
  float* tot = reinterpret_cast<float*>(sm + PT_TOT);
  float* sbeta = reinterpret_cast<float*>(sm + PT_BETA);
  float* sP = reinterpret_cast<float*>(sm + PT_SP);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + PT_BARS);     // 0: first product done, 1: V landed, 2: second product done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  const int n = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int G = a.HV / a.H, h = hv / G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = n * KM_C;
  const int64_t bh = (int64_t)b * a.HV + hv;
  uint8_t* wsc = a.ws + (bh * a.NT + n) * (int64_t)KM_CHUNK_BYTES;
  // thread -> rows 4 rg .. 4 rg + 3, channels 8 c8 .. 8 c8 + 7
  const int rg = tid >> 4, c8 = tid & 15;
  const int64_t tok0 = (int64_t)b * a.Tb + t0 + 4 * rg;

  // ---- all twelve 16-byte loads of this thread's 4 x 8 block (g, k, q) are issued before anything waits on them ---
  uint4 graw[4], kreg[4], qreg[4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    graw[s] = make_uint4(0u, 0u, 0u, 0u);
    kreg[s] = make_uint4(0u, 0u, 0u, 0u);
    qreg[s] = make_uint4(0u, 0u, 0u, 0u);
    if (t0 + 4 * rg + s < a.T) {
      graw[s] = *reinterpret_cast<const uint4*>(a.g + (tok0 + s) * a.ld_g + (int64_t)hv * KM_K + 8 * c8);
      const int64_t off = (tok0 + s) * a.ld_qk + (int64_t)h * KM_K + 8 * c8;
      kreg[s] = *reinterpret_cast<const uint4*>(a.k + off);
      qreg[s] = *reinterpret_cast<const uint4*>(a.q + off);
    }
  }
  // ---- log-decay: activation, clamp, running sum (log2 units) -------------------------------------------------
  float gam[4][8];
  {
    float run[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const bool ok = t0 + 4 * rg + s < a.T;
      const bf16* e = reinterpret_cast<const bf16*>(&graw[s]);
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        float gx = __bfloat162float(e[x]);
        if (a.gate_scale != 0.f) {
          // the gate activation of the layer (ops_fused.py:575-578) with its bf16 rounding points
          const float sp = __bfloat162float(__float2bfloat16_rn(gx > 20.f ? gx : __logf(1.0f + __expf(gx))));
          gx = __bfloat162float(__float2bfloat16_rn(-sp * a.gate_scale));
        }
        run[x] += ok ? fmaxf(gx, a.g_min) * KM_LOG2E : 0.f;
        gam[s][x] = run[x];
      }
    }
    float4* dst = reinterpret_cast<float4*>(tot + rg * 128 + 8 * c8);
    dst[0] = make_float4(run[0], run[1], run[2], run[3]);
    dst[1] = make_float4(run[4], run[5], run[6], run[7]);
  }
  if (tid < KM_C) sbeta[tid] = (t0 + tid < a.T) ? __bfloat162float(a.beta[((int64_t)b * a.Tb + t0 + tid) * a.ld_b + hv]) : 0.f;
  if (tid == 0) {
    mbarrier_init(&bars[0], 1); mbarrier_init(&bars[1], 1); mbarrier_init(&bars[2], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (tid < KM_K) {                                  // exclusive prefix over the 16 row groups, total in row 16
    float run = 0.f;
#pragma unroll
    for (int r = 0; r < 16; ++r) { const float x = tot[r * 128 + tid]; tot[r * 128 + tid] = run; run += x; }
    tot[16 * 128 + tid] = run;
  }
  __syncthreads();
  float pre[8], gl[8];
  {
    const float4* p4 = reinterpret_cast<const float4*>(tot + rg * 128 + 8 * c8);
    const float4 x = p4[0], y = p4[1];
    pre[0] = x.x; pre[1] = x.y; pre[2] = x.z; pre[3] = x.w; pre[4] = y.x; pre[5] = y.y; pre[6] = y.z; pre[7] = y.w;
    const float4* l4 = reinterpret_cast<const float4*>(tot + 16 * 128 + 8 * c8);
    const float4 u = l4[0], v = l4[1];
    gl[0] = u.x; gl[1] = u.y; gl[2] = u.z; gl[3] = u.w; gl[4] = v.x; gl[5] = v.y; gl[6] = v.z; gl[7] = v.w;
  }
  bool strong = false;
#pragma unroll
  for (int x = 0; x < 8; ++x) strong |= !(gl[x] >= -PT_GMAX);
  if (__syncthreads_or(strong)) {                    // uniform: the whole chunk takes the re-centring path
    kda_prepare_chunk_mma(a, pt_raw, n, hv, b);
    return;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // ---- the four operand images of the block ----------------------------------------------------------------------
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int i = 4 * rg + s;
    const bf16* ke = reinterpret_cast<const bf16*>(&kreg[s]);
    const bf16* qe = reinterpret_cast<const bf16*>(&qreg[s]);
    uint32_t ekh[4], ekl[4], qgh[4], qgl[4], yh[4], yl[4], kgh[4], kgl[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ga0 = pre[2 * e] + gam[s][2 * e], ga1 = pre[2 * e + 1] + gam[s][2 * e + 1];
      const float k0 = __bfloat162float(ke[2 * e]), k1 = __bfloat162float(ke[2 * e + 1]);
      const float q0 = __bfloat162float(qe[2 * e]) * a.scale, q1 = __bfloat162float(qe[2 * e + 1]) * a.scale;
      const float d0 = ex2_fast(ga0), d1 = ex2_fast(ga1);
      split2_bf16(k0 * d0, k1 * d1, ekh[e], ekl[e]);
      split2_bf16(q0 * d0, q1 * d1, qgh[e], qgl[e]);
      split2_bf16(k0 * ex2_fast(-ga0), k1 * ex2_fast(-ga1), yh[e], yl[e]);
      split2_bf16(k0 * ex2_fast(gl[2 * e] - ga0), k1 * ex2_fast(gl[2 * e + 1] - ga1), kgh[e], kgl[e]);
    }
    const uint32_t pan = (uint32_t)(c8 >> 3), inner = swz<128>(i, c8 & 7);
    uint8_t* ai = sm + PT_AIMG + pan * 16384u + inner;
    *reinterpret_cast<uint4*>(ai) = make_uint4(ekh[0], ekh[1], ekh[2], ekh[3]);
    *reinterpret_cast<uint4*>(ai + 32768) = make_uint4(ekl[0], ekl[1], ekl[2], ekl[3]);
    *reinterpret_cast<uint4*>(ai + 8192) = make_uint4(qgh[0], qgh[1], qgh[2], qgh[3]);
    *reinterpret_cast<uint4*>(ai + 32768 + 8192) = make_uint4(qgl[0], qgl[1], qgl[2], qgl[3]);
    uint8_t* yi = sm + PT_Y + pan * 8192u + inner;
    *reinterpret_cast<uint4*>(yi) = make_uint4(yh[0], yh[1], yh[2], yh[3]);
    *reinterpret_cast<uint4*>(yi + 16384) = make_uint4(yl[0], yl[1], yl[2], yl[3]);
    // the record of the sequential stage: [w; qg] panels (rows 64..127 are qg), kg panels
    *reinterpret_cast<uint4*>(wsc + pan * 16384u + 8192u + inner) = make_uint4(qgh[0], qgh[1], qgh[2], qgh[3]);
    *reinterpret_cast<uint4*>(wsc + 32768u + pan * 16384u + 8192u + inner) = make_uint4(qgl[0], qgl[1], qgl[2], qgl[3]);
    *reinterpret_cast<uint4*>(wsc + KM_OFF_KHI + pan * 8192u + inner) = make_uint4(kgh[0], kgh[1], kgh[2], kgh[3]);
    *reinterpret_cast<uint4*>(wsc + KM_OFF_KLO + pan * 8192u + inner) = make_uint4(kgl[0], kgl[1], kgl[2], kgl[3]);
  }
  if (tid < KM_K) reinterpret_cast<float*>(wsc + KM_OFF_U + 32768)[tid] = ex2_fast(tot[16 * 128 + tid]);
  t5_fence_async_smem();
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t ai32 = smem_addr_u32(sm + PT_AIMG);

  // ---- [A ; Aqk] raw = [EK; QG] Y^T ---------------------------------------------------------------------------------
  if (tid == 0) {
    const uint32_t yb = smem_addr_u32(sm + PT_Y), id64 = t5_idesc(64);
#pragma unroll
    for (int term = 0; term < 3; ++term) {
      const uint32_t abase = ai32 + (term == 1 ? 32768u : 0u), bbase = yb + (term == 2 ? 16384u : 0u);
#pragma unroll
      for (int pan = 0; pan < 2; ++pan)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          t5_mma(tmem, t5_desc(abase + pan * 16384u) + 2 * ks, t5_desc(bbase + pan * 8192u) + 2 * ks, id64,
                 (term | pan | ks) ? 1u : 0u);
    }
    t5_commit(&bars[0]);
  }
  bool ok = true;
  if (tid == 0) ok = mbarrier_wait_bounded(&bars[0], 0, 61, PT_SPIN, status);   // one poller; the others sleep at the barrier
  ok = __syncthreads_and(ok);
  t5_fence_after();
  const int q4 = warp & 3, hh = warp >> 2;                        // tensor-memory lane quarter, column half
  const uint32_t lane_base = (uint32_t)(32 * q4) << 16;
  float* sA = reinterpret_cast<float*>(sm + PT_A);
  float* sT = reinterpret_cast<float*>(sm + PT_T);
  if (ok) {
    if (tid == 0) {                                               // V tile: the QG rows of the hi panels are free now
      mbarrier_expect_tx(&bars[1], 16384);
      t5_tma_load_2d(sm + PT_VT, &vmap, hv * KM_V, (int)((int64_t)b * a.Tb + t0), &bars[1]);
      t5_tma_load_2d(sm + PT_VT + 16384, &vmap, hv * KM_V + 64, (int)((int64_t)b * a.Tb + t0), &bars[1]);
    }
    uint32_t r[32];
    t5_ld32(tmem + lane_base + 32 * hh, r);
    t5_wait_ld();
    if (q4 < 2) {                                                 // rows of A: beta_i x strictly lower part, fp32
      const int i = 32 * q4 + lane;
      const float bi = sbeta[i];
      float4* dst = reinterpret_cast<float4*>(sA + i * PS_LD + 32 * hh);
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const int jj = 32 * hh + j;
        dst[j >> 2] = make_float4(jj < i ? __uint_as_float(r[j]) * bi : 0.f, jj + 1 < i ? __uint_as_float(r[j + 1]) * bi : 0.f,
                                  jj + 2 < i ? __uint_as_float(r[j + 2]) * bi : 0.f, jj + 3 < i ? __uint_as_float(r[j + 3]) * bi : 0.f);
      }
    } else {                                                      // rows of Aqk: lower part with the diagonal, hi / lo tiles
      const int i = 32 * (q4 - 2) + lane;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int jj = 32 * hh + 8 * c + 2 * e;
          split2_bf16(jj <= i ? __uint_as_float(r[8 * c + 2 * e]) : 0.f, jj + 1 <= i ? __uint_as_float(r[8 * c + 2 * e + 1]) : 0.f,
                      hi[e], lo[e]);
        }
        const uint32_t off = swz<128>(i, 4 * hh + c);
        *reinterpret_cast<uint4*>(wsc + KM_OFF_AQK + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(wsc + KM_OFF_AQK + 8192 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
    }
  }
  __syncthreads();
  if (ok) {
    // ---- T = (I + A)^-1, blocked: [[M00, 0], [M10, M11]]^-1 = [[T00, 0], [-T11 M10 T00, T11]] on two levels ----------
    // All 256 threads work in every phase, and every phase is a short dependent chain: the four 16 x 16 diagonal
    // blocks by substitution (four steps at a time), then the 16 x 16 blocks under them, then the 32 x 32 block.
    // A (row-major, zero at and above the diagonal) is only read; T is built in place in sT, whose upper triangle
    // serves as scratch for the intermediate products and is masked out when T is converted.
    {
      // (a) the diagonal blocks: thread = (block, column, 4 of its 16 rows); the owner of the four rows of a step group
      // solves them locally, the others of its column take the values by shuffle and update their rows.
      const int db = tid >> 6, c = (tid & 63) >> 2, p = tid & 3;
      const float* ab = sA + (16 * db + 4 * p) * PS_LD + 16 * db;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        float4 a4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a4[i] = *reinterpret_cast<const float4*>(ab + i * PS_LD + 4 * kb);
        const bool dg = (c >> 2) == kb;
        const int cj = c & 3;
        const float x0 = ((dg && cj == 0) ? 1.f : 0.f) - v[0];
        const float x1 = fmaf(-a4[1].x, x0, ((dg && cj == 1) ? 1.f : 0.f) - v[1]);
        const float x2 = fmaf(-a4[2].y, x1, fmaf(-a4[2].x, x0, ((dg && cj == 2) ? 1.f : 0.f) - v[2]));
        const float x3 = fmaf(-a4[3].z, x2, fmaf(-a4[3].y, x1, fmaf(-a4[3].x, x0, ((dg && cj == 3) ? 1.f : 0.f) - v[3])));
        const int src = (lane & ~3) | kb;
        const float y0 = __shfl_sync(0xffffffffu, x0, src), y1 = __shfl_sync(0xffffffffu, x1, src),
                    y2 = __shfl_sync(0xffffffffu, x2, src), y3 = __shfl_sync(0xffffffffu, x3, src);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = fmaf(a4[i].w, y3, fmaf(a4[i].z, y2, fmaf(a4[i].y, y1, fmaf(a4[i].x, y0, v[i]))));
        if (p == kb) { v[0] = x0; v[1] = x1; v[2] = x2; v[3] = x3; }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) sT[(16 * db + 4 * p + i) * PS_LD + 16 * db + c] = v[i];
    }
    __syncthreads();
    {
      // (b) blocks (1,0) and (3,2): P = A10 T00 (kept in rows 0..15 of the upper triangle), then T10 = -T11 P;
      // thread = (pair, row, two columns)
      const int pr = tid >> 7, r = (tid & 127) >> 3, q = tid & 7;
      const int K0 = 32 * pr;
      float* pbuf = sT + 16 + 32 * pr + 2 * q;
      float ak[16];
      {
        const float* arow = sA + (K0 + 16 + r) * PS_LD + K0;
#pragma unroll
        for (int kq = 0; kq < 4; ++kq) {
          const float4 t = *reinterpret_cast<const float4*>(arow + 4 * kq);
          ak[4 * kq] = t.x; ak[4 * kq + 1] = t.y; ak[4 * kq + 2] = t.z; ak[4 * kq + 3] = t.w;
        }
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int kq = 0; kq < 16; ++kq) {
          const float2 t = *reinterpret_cast<const float2*>(sT + (K0 + kq) * PS_LD + K0 + 2 * q);
          p0 = fmaf(ak[kq], t.x, p0); p1 = fmaf(ak[kq], t.y, p1);
        }
        *reinterpret_cast<float2*>(pbuf + r * PS_LD) = make_float2(p0, p1);
      }
      __syncthreads();
      {
        const float* trow = sT + (K0 + 16 + r) * PS_LD + K0 + 16;
#pragma unroll
        for (int kq = 0; kq < 4; ++kq) {
          const float4 t = *reinterpret_cast<const float4*>(trow + 4 * kq);
          ak[4 * kq] = t.x; ak[4 * kq + 1] = t.y; ak[4 * kq + 2] = t.z; ak[4 * kq + 3] = t.w;
        }
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int kq = 0; kq < 16; ++kq) {
          const float2 t = *reinterpret_cast<const float2*>(pbuf + kq * PS_LD);
          p0 = fmaf(ak[kq], t.x, p0); p1 = fmaf(ak[kq], t.y, p1);
        }
        *reinterpret_cast<float2*>(sT + (K0 + 16 + r) * PS_LD + K0 + 2 * q) = make_float2(-p0, -p1);
      }
    }
    __syncthreads();
    {
      // (c) the 32 x 32 block: P = A[32.., ..31] T[..31, ..31] (into rows 0..31, columns 32..63), then
      // T[32.., ..31] = -T[32.., 32..] P; thread = (row = lane, four columns = warp).  T[..31, ..31] is lower
      // triangular, so the columns of warp q need k >= 4 q only.
      const int q = warp, r = lane;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const float* arow = sA + (32 + r) * PS_LD;
#pragma unroll 2
      for (int k4 = q; k4 < 8; ++k4) {
        const float4 av = *reinterpret_cast<const float4*>(arow + 4 * k4);
        const float aa[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float4 t = *reinterpret_cast<const float4*>(sT + (4 * k4 + kk) * PS_LD + 4 * q);
          acc[0] = fmaf(aa[kk], t.x, acc[0]); acc[1] = fmaf(aa[kk], t.y, acc[1]);
          acc[2] = fmaf(aa[kk], t.z, acc[2]); acc[3] = fmaf(aa[kk], t.w, acc[3]);
        }
      }
      // (rows 0..15 of that region were the scratch of (b), dead since the barrier above)
      *reinterpret_cast<float4*>(sT + r * PS_LD + 32 + 4 * q) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      __syncthreads();
      float ac2[4] = {0.f, 0.f, 0.f, 0.f};
      const float* trow = sT + (32 + r) * PS_LD + 32;
#pragma unroll
      for (int k4 = 0; k4 < 8; ++k4) {
        float4 av = *reinterpret_cast<const float4*>(trow + 4 * k4);
        if (k4 >= 4 && r < 16) av = make_float4(0.f, 0.f, 0.f, 0.f);   // block (2,3) of T was never written: it is zero
        const float aa[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float4 t = *reinterpret_cast<const float4*>(sT + (4 * k4 + kk) * PS_LD + 32 + 4 * q);
          ac2[0] = fmaf(aa[kk], t.x, ac2[0]); ac2[1] = fmaf(aa[kk], t.y, ac2[1]);
          ac2[2] = fmaf(aa[kk], t.z, ac2[2]); ac2[3] = fmaf(aa[kk], t.w, ac2[3]);
        }
      }
      *reinterpret_cast<float4*>(sT + (32 + r) * PS_LD + 4 * q) = make_float4(-ac2[0], -ac2[1], -ac2[2], -ac2[3]);
    }
    __syncthreads();
    {
      // T diag(beta) into the K-major hi / lo operand tiles (over the QG lo rows): thread = (row, 16 columns)
      const int i = tid >> 2, ch = tid & 3;
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        const int c0 = 16 * ch + 8 * hc;
        const float4 ta = *reinterpret_cast<const float4*>(sT + i * PS_LD + c0), tb = *reinterpret_cast<const float4*>(sT + i * PS_LD + c0 + 4);
        const float4 ba = *reinterpret_cast<const float4*>(sbeta + c0), bb = *reinterpret_cast<const float4*>(sbeta + c0 + 4);
        const float tv[8] = {ta.x * ba.x, ta.y * ba.y, ta.z * ba.z, ta.w * ba.w, tb.x * bb.x, tb.y * bb.y, tb.z * bb.z, tb.w * bb.w};
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          split2_bf16(c0 + 2 * e <= i ? tv[2 * e] : 0.f, c0 + 2 * e + 1 <= i ? tv[2 * e + 1] : 0.f, hi[e], lo[e]);
        const uint32_t off = swz<128>(i, 2 * ch + hc);
        *reinterpret_cast<uint4*>(sm + PT_TBH + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(sm + PT_TBL + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
    }
    t5_fence_async_smem();
  }
  t5_fence_before();
  __syncthreads();
  t5_fence_after();

  // ---- w^T = EK^T Tb^T, u^T = V^T Tb^T (EK and V read as MN-major A operands: rows = tokens, 64-wide panels) -----------
  const uint32_t tW = tmem + 64, tU = tmem + 128;
  if (ok && tid == 0) {
    if (mbarrier_wait_bounded(&bars[1], 0, 62, PT_SPIN, status)) {
      t5_fence_after();
      const uint32_t idm = t5_idesc(64) | (1u << 15);
      const uint32_t tbh = ai32 + (PT_TBH - PT_AIMG), tbl = ai32 + (PT_TBL - PT_AIMG), ekl = ai32 + 32768u,
                     vv = ai32 + (PT_VT - PT_AIMG);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) t5_mma(tW, t5_desc_mn(ai32 + ks * 2048u, 16384u), t5_desc(tbh) + 2 * ks, idm, ks ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) t5_mma(tW, t5_desc_mn(ekl + ks * 2048u, 16384u), t5_desc(tbh) + 2 * ks, idm, 1u);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) t5_mma(tW, t5_desc_mn(ai32 + ks * 2048u, 16384u), t5_desc(tbl) + 2 * ks, idm, 1u);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) t5_mma(tU, t5_desc_mn(vv + ks * 2048u, 16384u), t5_desc(tbh) + 2 * ks, idm, ks ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) t5_mma(tU, t5_desc_mn(vv + ks * 2048u, 16384u), t5_desc(tbl) + 2 * ks, idm, 1u);
    }
    t5_commit(&bars[2]);
  }
  if (ok && tid == 0) ok = mbarrier_wait_bounded(&bars[2], 0, 63, PT_SPIN, status);
  ok = __syncthreads_and(ok);
  t5_fence_after();
  if (ok) {
    uint32_t r[32];
    const int c = 32 * q4 + lane;                                 // channel of w^T / value column of u^T
    t5_ld32(tW + lane_base + 32 * hh, r);
    t5_wait_ld();
    {
      uint8_t* wh = sm + PT_WST + (c >> 6) * 8192;
      uint8_t* wl = wh + 16384;
      const int cc = c & 63;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        bf16 hi, lo;
        split1_bf16(__uint_as_float(r[j]), hi, lo);
        const uint32_t off = swz<128>(32 * hh + j, cc >> 3) + 2 * (cc & 7);
        *reinterpret_cast<bf16*>(wh + off) = hi;
        *reinterpret_cast<bf16*>(wl + off) = lo;
      }
    }
    t5_ld32(tU + lane_base + 32 * hh, r);
    t5_wait_ld();
    {
      // u^T as [token / 32][token / 4 % 8][value column][token % 4]: a warp of the sequential stage reads 512 contiguous bytes
      float4* up = reinterpret_cast<float4*>(wsc + KM_OFF_U) + hh * 8 * 128 + c;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        up[j * 128] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                  __uint_as_float(r[4 * j + 3]));
    }
    t5_fence_async_smem();
  }
  t5_fence_before();
  __syncthreads();
  if (ok && tid == 0) {                                           // w hi / lo panels -> rows 0..63 of the [w; qg] panels
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      t5_bulk_store(wsc + p * 16384, sm + PT_WST + p * 8192, 8192);
      t5_bulk_store(wsc + 32768 + p * 16384, sm + PT_WST + 16384 + p * 8192, 8192);
    }
    t5_bulk_commit();
    t5_bulk_wait_read();
  }
  if (warp == 0) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
  }
}

int kch_make_tensor_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                                uint32_t box_rows, uint32_t box_cols);   // gemm_tcgen05.cu

static int launch_kda_prepare_tc5(const PrepArgs& pa, int B, unsigned int* status, cudaStream_t s) {
  CUtensorMap vmap;
  int rc = kch_make_tensor_map_2d_bf16(&vmap, pa.v, (uint64_t)(B - 1) * pa.Tb + pa.T, (uint64_t)pa.HV * KM_V, (uint64_t)pa.ld_v, 64, 64);
  if (rc != KCH_OK) return rc;
  KCH_CUDA_OK(cudaFuncSetAttribute(kda_prepare_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_DYN));
  KCH_CUDA_OK(cudaFuncSetAttribute(kda_prepare_tc5_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
  kda_prepare_tc5_kernel<<<dim3(pa.NT, pa.HV, B), 256, PT_DYN, s>>>(pa, vmap, status);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
