// Sequential stage of chunked KDA on the fifth-generation tensor cores (tcgen05), state resident in
// tensor memory.  Same arithmetic as kda_scan_mma_kernel (naive_chunk_kda, ops_kda.py:509-535):
//   vt^T = u^T - S^T w^T ;  o^T = S^T qg^T + vt^T Aqk^T ;  S^T <- S^T diag(dl) + vt^T kg
// with every product as hi*hi + lo*hi + hi*lo of two-term bf16 splits and fp32 accumulation.
//
// One CTA per (batch, value head); S^T [128 v x 128 k] fp32 is the accumulator of the update product
// and never leaves tensor memory between chunks.  Per chunk (the dependent chain is S -> D1w -> vt -> S):
//   vector warps : read S^T (tcgen05.ld, one row v per thread), write its bf16 hi / lo images into shared
//                  memory in the MMA operand layout, one 64-channel panel at a time, and write
//                  S^T diag(dl) back (tcgen05.st)
//   MMA thread   : [D1w | D1q] = S^T [w; qg]^T   (M = 128 v, N = 64 + 64 tokens, K = 128 channels), starting on a
//                  panel as soon as the vector warps have finished it
//   vector warps : vt^T = u^T - D1w -> bf16 hi / lo operand tiles, 16 tokens at a time
//   MMA thread   : S^T += vt^T kg (N = 128, kg read as an MN-major operand, i.e. in its natural [token][channel]
//                  layout), then D1q += vt^T Aqk^T (N = 64); K = 64 tokens
//   vector warps : o^T = D1q -> bf16 -> global one chunk later, while the next [D1w | D1q] is being computed
//                  (the [D1w | D1q] block is double-buffered in tensor memory)
// A producer warp streams the chunk's operand tiles (written by the prepare kernel in this layout) with 1-D
// bulk copies.  Every wait is a bounded mbarrier wait that records a status code and leaves the loops.
//
// Workspace record of a chunk in this layout (written by kda_prepare_mma_kernel when PrepArgs::umma is set):
//   0      [w; qg] hi: two 64-channel panels of [128 rows][64] bf16 (rows 0..63 w, 64..127 qg), 128-byte swizzle
//   32768  [w; qg] lo
//   65536  Aqk hi [64][64], lo
//   81920  kg hi: two 64-channel panels of [64 tokens][64] bf16;  98304 kg lo
//   114688 u^T fp32 as [token / 32][token / 4 % 8][v][token % 4], then dl [128] fp32
#include <math.h>
#include <stdlib.h>

#include "mma_utils.cuh"
#include "tc5_utils.cuh"

#define T5_THREADS 320
#define T5_SPIN (1u << 26)
// workspace record of one chunk (offsets shared with kda_mma.cu)
#define T5_OFF_WHI 0
#define T5_OFF_WLO 16384
#define T5_OFF_QHI 32768
#define T5_OFF_QLO 49152
#define T5_OFF_AQK 65536
#define T5_OFF_KHI 81920
#define T5_OFF_KLO 98304
#define T5_OFF_U 114688
#define T5_U_SLICE 16896
#define T5_CHUNK_BYTES (T5_OFF_U + 2 * T5_U_SLICE)

struct T5Args {
  const uint8_t* ws;
  const float* S0;
  bf16* o;
  float* S_out;
  unsigned int* status;
  int T, HV, NT;                     // T: tokens from the first chunk of this launch to the end of the sequence
  int Tb;                            // tokens between consecutive batch entries (the whole sequence length)
};

// shared-memory map (bytes, 1024-aligned operand tiles)
#define T5_SA 0                      // S^T hi: 2 panels [128][64] bf16 (32768), then lo (32768)
#define T5_VA (T5_SA + 65536)        // vt^T hi [128][64] bf16 (16384), lo (16384)
#define T5_TW (T5_VA + 32768)        // w hi, w lo, q hi, q lo: 4 x 16384
#define T5_TK (T5_TW + 65536)        // kg^T hi [128][64] (16384), lo (16384)
#define T5_TA (T5_TK + 32768)        // Aqk hi [64][64] (8192), lo (8192)
#define T5_DL (T5_TA + 16384)        // dl [128] fp32
#define T5_BARS (T5_DL + 512)
#define T5_TOTAL (T5_BARS + 128)

__global__ void __launch_bounds__(T5_THREADS, 1) kda_scan_tc5_kernel(T5Args a) {
  extern __shared__ uint8_t t5_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>(((uintptr_t)t5_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + T5_BARS);
  uint64_t *w_full = bars + 0, *w_empty = bars + 1, *k_full = bars + 2, *k_empty = bars + 3, *sa_ready0 = bars + 4,
           *d1_full = bars + 5, *va_ready0 = bars + 6, *s_full = bars + 7, *o_full = bars + 8, *sa_ready1 = bars + 9,
           *va_ready1 = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  const int hv = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t bh = (int64_t)b * a.HV + hv;
  const uint8_t* wsb = a.ws + bh * a.NT * (int64_t)T5_CHUNK_BYTES;
  constexpr uint32_t TMEM_COLS = 512;          // S^T 128 | [D1w 64 | D1q 64] of even chunks | the same of odd chunks

  if (threadIdx.x == 0) {
    mbarrier_init(w_full, 1); mbarrier_init(w_empty, 1); mbarrier_init(k_full, 1); mbarrier_init(k_empty, 1);
    mbarrier_init(sa_ready0, 8); mbarrier_init(sa_ready1, 8); mbarrier_init(d1_full, 1); mbarrier_init(va_ready0, 8); mbarrier_init(va_ready1, 8); mbarrier_init(s_full, 1); mbarrier_init(o_full, 1);
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
  const uint32_t tS = tmem, tD0 = tmem + 128;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      for (int n = 0; n < a.NT; ++n) {
        const uint8_t* src = wsb + (int64_t)n * T5_CHUNK_BYTES;
        const uint32_t ph = (uint32_t)n & 1;
        if (!mbarrier_wait_bounded(w_empty, ph ^ 1, 41, T5_SPIN, a.status)) break;
        mbarrier_expect_tx(w_full, 4 * 16384 + 512);
        bulk_copy_g2s(sm + T5_TW, src + T5_OFF_WHI, 4 * 16384, w_full);            // [w; qg] hi panels, then lo panels
        bulk_copy_g2s(sm + T5_DL, src + T5_OFF_U + 32768, 512, w_full);            // dl sits behind u^T
        if (!mbarrier_wait_bounded(k_empty, ph ^ 1, 42, T5_SPIN, a.status)) break;
        mbarrier_expect_tx(k_full, 2 * 16384 + 16384);
        bulk_copy_g2s(sm + T5_TK, src + T5_OFF_KHI, 2 * 16384, k_full);            // kg hi, lo
        bulk_copy_g2s(sm + T5_TA, src + T5_OFF_AQK, 16384, k_full);                // Aqk hi, lo
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t id64 = t5_idesc(64), id128 = t5_idesc(128), id128mn = t5_idesc(128) | (1u << 16);
      const uint32_t sa = smem_addr_u32(sm + T5_SA), va = smem_addr_u32(sm + T5_VA), tw = smem_addr_u32(sm + T5_TW),
                     tk = smem_addr_u32(sm + T5_TK), ta = smem_addr_u32(sm + T5_TA);
      for (int n = 0; n < a.NT; ++n) {
        const uint32_t ph = (uint32_t)n & 1;
        const uint32_t tD = tD0 + 128u * ph;                 // [D1w | D1q] of this chunk
        if (!mbarrier_wait_bounded(w_full, ph, 44, T5_SPIN, a.status)) break;
        // [D1w | D1q] = S^T [w; qg]^T: terms (S hi, x hi), (S lo, x hi), (S hi, x lo); one 64-channel panel of
        // S^T at a time, as the vector warps finish it
        bool ok = true;
#pragma unroll
        for (int pan = 0; pan < 2; ++pan) {
          if (!mbarrier_wait_bounded(pan ? sa_ready1 : sa_ready0, ph, 43, T5_SPIN, a.status)) { ok = false; break; }
          t5_fence_after();
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const uint32_t abase = sa + (term == 1 ? 32768u : 0u) + (uint32_t)pan * 16384u;
            const uint32_t bbase = tw + (term == 2 ? 32768u : 0u) + (uint32_t)pan * 16384u;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) t5_mma(tD, t5_desc(abase) + 2 * ks, t5_desc(bbase) + 2 * ks, id128, (pan | term | ks) ? 1u : 0u);
          }
        }
        if (!ok) break;
        t5_commit(d1_full);
        t5_commit(w_empty);
        if (!mbarrier_wait_bounded(k_full, ph, 46, T5_SPIN, a.status)) break;
        // S^T += vt^T kg   (N = 128 channels, kg read in place as an MN-major operand; K = 64 tokens, the 16-token
        // steps {0, 2} first, {1, 3} second, as the vector warps finish them)
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          if (!mbarrier_wait_bounded(part ? va_ready1 : va_ready0, ph, 45, T5_SPIN, a.status)) { ok = false; break; }
          t5_fence_after();
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const uint32_t abase = va + (term == 1 ? 16384u : 0u);
            const uint32_t bbase = tk + (term == 2 ? 16384u : 0u);
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
              const int ks = 2 * k2 + part;
              t5_mma(tS, t5_desc(abase) + 2 * ks, t5_desc_mn(bbase + (uint32_t)ks * 2048u), id128mn, 1u);
            }
          }
        }
        if (!ok) break;
        t5_commit(s_full);
        // D1q += vt^T Aqk^T
#pragma unroll
        for (int term = 0; term < 3; ++term) {
          const uint32_t abase = va + (term == 1 ? 16384u : 0u);
          const uint32_t bbase = ta + (term == 2 ? 8192u : 0u);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) t5_mma(tD + 64, t5_desc(abase) + 2 * ks, t5_desc(bbase) + 2 * ks, id64, 1u);
        }
        t5_commit(o_full);
        t5_commit(k_empty);
      }
    }
  } else {
    // ------------------------------ vector warps ------------------------------
    const int quarter = warp & 3, sub = (warp - 2) >> 2;
    const int v = quarter * 32 + lane;                         // this thread's row of S^T, D1w, D1q
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    uint32_t r[32], r2[32], ro[32];
    // initial state into tensor memory: this warp owns channels 32*sub .. +31 of each 64-channel panel of row v
#pragma unroll
    for (int pan = 0; pan < 2; ++pan) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int kc = 64 * pan + 32 * sub + j;
        r[j] = a.S0 ? __float_as_uint(a.S0[bh * (128 * 128) + (int64_t)kc * 128 + v]) : 0u;
      }
      t5_st32(tS + lane_base + 64 * pan + 32 * sub, r);
    }
    t5_wait_st();
    bool ok = true;
    const float* dl = reinterpret_cast<const float*>(sm + T5_DL);
    for (int n = 0; n < a.NT && ok; ++n) {
      const uint32_t ph = (uint32_t)n & 1;
      const uint8_t* src = wsb + (int64_t)n * T5_CHUNK_BYTES;
      if (n > 0 && !mbarrier_wait_bounded(s_full, ph ^ 1, 47, T5_SPIN, a.status)) { ok = false; break; }
      if (!mbarrier_wait_bounded(w_full, ph, 48, T5_SPIN, a.status)) { ok = false; break; }      // dl has landed
      t5_fence_after();
      // ---- S^T -> bf16 hi / lo operand images, panel 0 then panel 1; S^T diag(dl) back to tensor memory -----------
      t5_ld32(tS + lane_base + 32 * sub, r);
      t5_ld32(tS + lane_base + 64 + 32 * sub, r2);
      t5_wait_ld();
#pragma unroll
      for (int pan = 0; pan < 2; ++pan) {
        uint32_t (&rr)[32] = pan ? r2 : r;
        const int kc0 = 64 * pan + 32 * sub;                   // first channel of these 32 columns
        uint8_t* pan_hi = sm + T5_SA + (size_t)pan * 16384;
        uint8_t* pan_lo = pan_hi + 32768;
#pragma unroll
        for (int q = 0; q < 4; ++q) {                          // four 16-byte chunks of 8 channels
          uint32_t h[4], l[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            split2_bf16(__uint_as_float(rr[8 * q + 2 * e]), __uint_as_float(rr[8 * q + 2 * e + 1]), h[e], l[e]);
          const uint32_t off = swz<128>(v, 4 * sub + q);
          *reinterpret_cast<uint4*>(pan_hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<uint4*>(pan_lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
        }
        t5_fence_async_smem();
        t5_fence_before();
        __syncwarp();
        if (lane == 0) mbarrier_arrive(pan ? sa_ready1 : sa_ready0);
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dl + kc0 + j);
          rr[j] = __float_as_uint(__uint_as_float(rr[j]) * d4.x);
          rr[j + 1] = __float_as_uint(__uint_as_float(rr[j + 1]) * d4.y);
          rr[j + 2] = __float_as_uint(__uint_as_float(rr[j + 2]) * d4.z);
          rr[j + 3] = __float_as_uint(__uint_as_float(rr[j + 3]) * d4.w);
        }
        t5_st32(tS + lane_base + kc0, rr);
      }
      // u^T row v, tokens 32*sub .. +31 (fp32, straight from the workspace)
      float u[32];
      {
        const float4* up = reinterpret_cast<const float4*>(src + T5_OFF_U) + sub * 8 * 128 + v;   // [sub][j][v] float4: coalesced
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float4 x = up[j * 128]; u[4 * j] = x.x; u[4 * j + 1] = x.y; u[4 * j + 2] = x.z; u[4 * j + 3] = x.w; }
      }
      // ---- o^T of the previous chunk -> global: token t, value column v (64 contiguous bytes per warp and token) ----
      if (n > 0) {
        if (!mbarrier_wait_bounded(o_full, ph ^ 1, 52, T5_SPIN, a.status)) { ok = false; break; }
        t5_fence_after();
        t5_ld32(tD0 + 128u * (ph ^ 1) + 64 + lane_base + 32 * sub, ro);
        t5_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int t = (n - 1) * 64 + 32 * sub + j;
          a.o[(((int64_t)b * a.Tb + t) * a.HV + hv) * 128 + v] = __float2bfloat16_rn(__uint_as_float(ro[j]));
        }
      }
      // ---- vt^T = u^T - D1w -> operand images, 16 tokens at a time ---------------------------------------------
      t5_wait_st();                                             // the decayed S^T is in place before the update may start
      if (!mbarrier_wait_bounded(d1_full, ph, 49, T5_SPIN, a.status)) { ok = false; break; }
      t5_fence_after();
      t5_ld32(tD0 + 128u * ph + lane_base + 32 * sub, r);
      t5_wait_ld();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          split2_bf16(u[8 * q + 2 * e] - __uint_as_float(r[8 * q + 2 * e]), u[8 * q + 2 * e + 1] - __uint_as_float(r[8 * q + 2 * e + 1]),
                      h[e], l[e]);
        const uint32_t off = swz<128>(v, 4 * sub + q);
        *reinterpret_cast<uint4*>(sm + T5_VA + off) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(sm + T5_VA + 16384 + off) = make_uint4(l[0], l[1], l[2], l[3]);
        if (q & 1) {
          t5_fence_async_smem();
          t5_fence_before();
          __syncwarp();
          if (lane == 0) mbarrier_arrive(q == 1 ? va_ready0 : va_ready1);
        }
      }
    }
    // the last products must have finished before o^T and the state are read and tensor memory is released
    if (ok && a.NT > 0 && !mbarrier_wait_bounded(s_full, (uint32_t)(a.NT - 1) & 1, 51, T5_SPIN, a.status)) ok = false;
    if (ok && a.NT > 0 && !mbarrier_wait_bounded(o_full, (uint32_t)(a.NT - 1) & 1, 53, T5_SPIN, a.status)) ok = false;
    if (ok && a.NT > 0) {
      t5_fence_after();
      t5_ld32(tD0 + 128u * ((uint32_t)(a.NT - 1) & 1) + 64 + lane_base + 32 * sub, ro);
      t5_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int t = (a.NT - 1) * 64 + 32 * sub + j;
        if (t < a.T) a.o[(((int64_t)b * a.Tb + t) * a.HV + hv) * 128 + v] = __float2bfloat16_rn(__uint_as_float(ro[j]));
      }
      if (a.S_out) {
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          t5_ld32(tS + lane_base + 64 * sub + c0, r);
          t5_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            a.S_out[bh * (128 * 128) + (int64_t)(64 * sub + c0 + j) * 128 + v] = __uint_as_float(r[j]);
        }
      }
    }
  }
  t5_fence_before();
  __syncthreads();
  if (warp == 1) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host ----------------------------------------------------------------------------------------------------
bool kch_kda_scan_tc5_enabled() {
  // default; KCH_KDA_SCAN=m selects the mma.sync scan (kda_scan_mma_kernel) for comparison
  static const bool on = [] { const char* e = getenv("KCH_KDA_SCAN"); return !(e && e[0] == 'm'); }();
  return on;
}

int kch_kda_scan_tc5(const void* workspace, const float* initial_state, void* o, float* final_state, int B, int T,
                     int Tb, int HV, int NT, unsigned int* status, cudaStream_t s) {
  T5Args a;
  a.ws = (const uint8_t*)workspace; a.S0 = initial_state; a.o = (bf16*)o; a.S_out = final_state; a.status = status;
  a.T = T; a.Tb = Tb; a.HV = HV; a.NT = NT;
  const int smem = T5_TOTAL + 1024;
  KCH_CUDA_OK(cudaFuncSetAttribute(kda_scan_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kda_scan_tc5_kernel<<<dim3(HV, B), T5_THREADS, smem, s>>>(a);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
