// KDA: gated delta rule with per-channel log-decay.
//   token recurrence : naive_recurrent_kda (ops_kda.py:222-258)
//   chunked WY form  : naive_chunk_kda     (ops_kda.py:375-424 prepare, 509-535 chain)
// All arithmetic is fp32; inputs are fp32 or bf16; the carried state is fp32 [B,HV,K,V].
#include <math.h>
#include <stdlib.h>

#include "kch_common.cuh"
#include "mma_utils.cuh"

// =====================================================================================
// Token recurrence.  One CTA owns 32 value columns of one (batch, value head); its 4 warps
// split the K rows of the state, which lives in registers for the whole sequence.
// Per token: S <- diag(exp g) S ; S <- S + beta k (v - k^T S)^T ; o = (scale q)^T S.
// Decode (T=1) reads and writes the state exactly once: 2*K*V*4 bytes per (b, hv).
// S0 and S_out may be the same memory: every thread loads its own state elements before the token loop and
// stores the same elements after it.
// =====================================================================================
template <typename T, int KPT>
__global__ void __launch_bounds__(128)
kda_recurrent_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                     const T* __restrict__ g, const T* __restrict__ beta,
                     const float* S0, T* __restrict__ o, float* S_out,
                     int T_, int H, int HV, int K, int V, float scale, float g_min, int64_t ld_qk,
                     int64_t ld_v, int64_t ld_g, int64_t ld_b) {
  const int vb = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int G = HV / H, h = hv / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vcol = vb * 32 + lane;
  const bool vok = vcol < V;
  const int k0 = warp * KPT;
  __shared__ float sk[2][4 * KPT], sq[2][4 * KPT], sg[2][4 * KPT];
  __shared__ float red[4][32], red2[4][32];
  float s[KPT];
  const int64_t sbase = ((int64_t)b * HV + hv) * K * V;
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    int kk = k0 + i;
    s[i] = (S0 && vok && kk < K) ? S0[sbase + (int64_t)kk * V + vcol] : 0.f;
  }
  auto load_tok = [&](int t, int buf) {
    const int64_t qoff = ((int64_t)b * T_ + t) * ld_qk + (int64_t)h * K;
    const int64_t goff = ((int64_t)b * T_ + t) * ld_g + (int64_t)hv * K;
    for (int i = threadIdx.x; i < 4 * KPT; i += 128) {
      bool ok = i < K;
      sk[buf][i] = ok ? ldf(k + qoff + i) : 0.f;
      sq[buf][i] = ok ? ldf(q + qoff + i) * scale : 0.f;
      sg[buf][i] = ok ? expf(fmaxf(ldf(g + goff + i), g_min)) : 1.f;
    }
  };
  if (T_ > 0) load_tok(0, 0);
  __syncthreads();
  for (int t = 0; t < T_; ++t) {
    const int buf = t & 1;
    const int64_t voff = (((int64_t)b * T_ + t) * HV + hv);
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      s[i] *= sg[buf][k0 + i];
      part = fmaf(sk[buf][k0 + i], s[i], part);
    }
    red[warp][lane] = part;
    if (t + 1 < T_) load_tok(t + 1, buf ^ 1);
    __syncthreads();
    float pred = red[0][lane] + red[1][lane] + red[2][lane] + red[3][lane];
    float vv = vok ? ldf(v + ((int64_t)b * T_ + t) * ld_v + (int64_t)hv * V + vcol) : 0.f;
    float delta = ldf(beta + ((int64_t)b * T_ + t) * ld_b + hv) * (vv - pred);
    float op = 0.f;
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      s[i] = fmaf(sk[buf][k0 + i], delta, s[i]);
      op = fmaf(sq[buf][k0 + i], s[i], op);
    }
    red2[warp][lane] = op;
    __syncthreads();
    if (warp == 0 && vok)
      stf(o + voff * V + vcol, red2[0][lane] + red2[1][lane] + red2[2][lane] + red2[3][lane]);
  }
  if (S_out && vok) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      int kk = k0 + i;
      if (kk < K) S_out[sbase + (int64_t)kk * V + vcol] = s[i];
    }
  }
}

// One-token step (T = 1, K = V = 128), the form a decode step takes.  The 64 KB state of one (batch, value head) is
// contiguous: one bulk copy brings it into shared memory (no registers, no per-thread loads: three CTAs per SM keep
// 192 KB of requests in flight), one thread per value column walks its 128 K rows there -- the two contractions over
// K (k^T S and q^T S) are private sums, no exchange between warps -- and one bulk copy writes the state back.  Decay,
// key and scaled query of a K row travel as one float4 broadcast.  The sums are taken in the same order as
// kda_recurrent_kernel (four runs of 32 rows, added left to right), so both kernels return the same bits.
// The wait for the copy is bounded (status word, see kch_device_status).
#define KDS_STATE_BYTES (128 * 128 * 4)
#define KDS_SMEM (KDS_STATE_BYTES + 128 * 16 + 16)
template <typename T>
__global__ void __launch_bounds__(128)
kda_decode_step_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       const T* __restrict__ g, const T* __restrict__ beta, const float* S0, T* __restrict__ o,
                       float* S_out, int H, int HV, float scale, float g_min, int64_t ld_qk, int64_t ld_v,
                       int64_t ld_g, int64_t ld_b, unsigned int* status) {
  constexpr int K = 128, V = 128;
  extern __shared__ __align__(128) uint8_t kds_raw[];
  float* st = reinterpret_cast<float*>(kds_raw);                                   // [K][V]
  float4* sgkq = reinterpret_cast<float4*>(kds_raw + KDS_STATE_BYTES);             // {exp(g), k, scale * q, -} of K row i
  uint64_t* bar = reinterpret_cast<uint64_t*>(kds_raw + KDS_STATE_BYTES + 128 * 16);
  const int hv = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int h = hv / (HV / H);
  const int64_t sbase = ((int64_t)b * HV + hv) * K * V;
  if (tid == 0) {
    mbarrier_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (S0) {
      mbarrier_expect_tx(bar, KDS_STATE_BYTES);
      bulk_copy_g2s(st, S0 + sbase, KDS_STATE_BYTES, bar);
    }
  }
  {
    const int64_t qoff = (int64_t)b * ld_qk + (int64_t)h * K, goff = (int64_t)b * ld_g + (int64_t)hv * K;
    sgkq[tid] = make_float4(expf(fmaxf(ldf(g + goff + tid), g_min)), ldf(k + qoff + tid), ldf(q + qoff + tid) * scale, 0.f);
  }
  const float bt = ldf(beta + (int64_t)b * ld_b + hv);
  const float vv = ldf(v + (int64_t)b * ld_v + (int64_t)hv * V + tid);
  if (!S0) {
    for (int i = 0; i < K; ++i) st[i * V + tid] = 0.f;
  }
  __syncthreads();
  bool ok = true;
  if (S0) ok = mbarrier_wait_bounded(bar, 0, KCH_STATUS_KDA_STEP, 1u << 24, status);
  float* col = st + tid;
  float p[4], r[4];
#pragma unroll
  for (int run = 0; run < 4; ++run) {
    float acc = 0.f;
#pragma unroll 8
    for (int i = 32 * run; i < 32 * run + 32; ++i) {
      const float4 c = sgkq[i];
      acc = fmaf(c.y, col[i * V] * c.x, acc);
    }
    p[run] = acc;
  }
  const float delta = bt * (vv - (p[0] + p[1] + p[2] + p[3]));
#pragma unroll
  for (int run = 0; run < 4; ++run) {
    float acc = 0.f;
#pragma unroll 8
    for (int i = 32 * run; i < 32 * run + 32; ++i) {
      const float4 c = sgkq[i];
      const float sv = fmaf(c.y, delta, col[i * V] * c.x);
      col[i * V] = sv;
      acc = fmaf(c.z, sv, acc);
    }
    r[run] = acc;
  }
  if (ok) stf(o + ((int64_t)b * HV + hv) * V + tid, r[0] + r[1] + r[2] + r[3]);
  if (S_out) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the bulk store reads what the threads wrote
    __syncthreads();
    if (tid == 0 && ok) {
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                   ::"l"(S_out + sbase), "r"(smem_addr_u32(st)), "r"((uint32_t)KDS_STATE_BYTES) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the copy
    }
  }
}

extern "C" int kch_kda_recurrent(const void* q, const void* k, const void* v, const void* g,
                                 const void* beta, const float* initial_state, void* o,
                                 float* final_state, int B, int T, int H, int HV, int K, int V,
                                 float scale, float g_clamp_min, int dtype, int64_t ld_qk, int64_t ld_v,
                                 int64_t ld_g, int64_t ld_beta, void* stream) {
  if (ld_qk <= 0) ld_qk = (int64_t)H * K;
  if (ld_v <= 0) ld_v = (int64_t)HV * V;
  if (ld_g <= 0) ld_g = (int64_t)HV * K;
  if (ld_beta <= 0) ld_beta = HV;
  KCH_REQUIRE(H >= 1, "H=%d must be >= 1", H);
  KCH_REQUIRE(K >= 1, "K=%d must be >= 1", K);
  KCH_REQUIRE(V >= 1, "V=%d must be >= 1", V);
  KCH_REQUIRE(HV >= 1 && HV % H == 0, "HV=%d must be divisible by H=%d (GVA factor)", HV, H);
  KCH_REQUIRE(K <= 256, "K=%d exceeds the supported maximum of 256", K);
  KCH_REQUIRE(B >= 0 && T >= 0, "B=%d T=%d", B, T);
  if (B == 0) return KCH_OK;
  if (T == 0 && !final_state) return KCH_OK;
  dim3 grid((V + 31) / 32, HV, B), block(128);
  cudaStream_t s = kch_stream(stream);
  // (KCH_KDA_DECODE=o keeps the general kernel for the one-token step, for comparison)
  static const bool old_step = [] { const char* e = getenv("KCH_KDA_DECODE"); return e && e[0] == 'o'; }();
  if (T == 1 && K == 128 && V == 128 && !old_step && (((uintptr_t)initial_state | (uintptr_t)final_state) & 15) == 0) {
    unsigned int* status = kch_status_device_ptr();
    KCH_REQUIRE(status != nullptr, "kch_kda_recurrent: cannot resolve the device status word");
    KCH_DISPATCH_FLOAT(dtype, T_, {
      KCH_CUDA_OK(cudaFuncSetAttribute(kda_decode_step_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, KDS_SMEM));
      kda_decode_step_kernel<T_><<<dim3(HV, B), 128, KDS_SMEM, s>>>(
        (const T_*)q, (const T_*)k, (const T_*)v, (const T_*)g, (const T_*)beta, initial_state, (T_*)o, final_state, H, HV,
        scale, g_clamp_min, ld_qk, ld_v, ld_g, ld_beta, status);
    });
    KCH_LAUNCH_OK();
    return KCH_OK;
  }
  int kpt = (K + 3) / 4;
#define GO(T_, KPT)                                                                              \
  kda_recurrent_kernel<T_, KPT><<<grid, block, 0, s>>>((const T_*)q, (const T_*)k, (const T_*)v, \
      (const T_*)g, (const T_*)beta, initial_state, (T_*)o, final_state, T, H, HV, K, V, scale,  \
      g_clamp_min, ld_qk, ld_v, ld_g, ld_beta)
#define GOK(T_)                      \
  do {                               \
    if (kpt <= 4) GO(T_, 4);         \
    else if (kpt <= 8) GO(T_, 8);    \
    else if (kpt <= 16) GO(T_, 16);  \
    else if (kpt <= 32) GO(T_, 32);  \
    else GO(T_, 64);                 \
  } while (0)
  KCH_DISPATCH_FLOAT(dtype, T_, GOK(T_));
#undef GOK
#undef GO
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// =====================================================================================
// Chunked form, stage 1 (fully parallel over chunks): per (b, hv, chunk) compute
//   gamma = cumsum(g), A (strictly lower), Tm = (I+A)^-1 diag(beta),
//   w = Tm (exp(gamma) k), u = Tm v, Aqk (lower incl. diagonal),
//   qg = scale q exp(gamma), kg = k exp(gamma_last - gamma), dl = exp(gamma_last)
// and store them in the workspace for the sequential stage.
// =====================================================================================
#define KDA_CMAX 64

struct KdaChunkWs {
  float *w, *qg, *kg;   // [B,HV,Tp,K]
  float *u;             // [B,HV,Tp,V]
  float *aqk;           // [B,HV,NT,C,C]
  float *dl;            // [B,HV,NT,K]
};

template <typename T>
__global__ void __launch_bounds__(256)
kda_chunk_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                         const T* __restrict__ g, const T* __restrict__ beta, KdaChunkWs ws, int T_,
                         int H, int HV, int K, int V, int C, int NT, float scale, float g_min,
                         int64_t ld_qk, int64_t ld_v, int64_t ld_g, int64_t ld_b) {
  extern __shared__ float smem[];
  const int n = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int G = HV / H, h = hv / G;
  const int tid = threadIdx.x;
  const int KS = K + 1;             // padded row stride
  float* sk = smem;                 // [C][KS]   k
  float* sq = sk + C * KS;          // [C][KS]   scale*q, later exp(gamma)*k
  float* sgam = sq + C * KS;        // [C][KS]   gamma
  float* sA = sgam + C * KS;        // [C][C+1]  A, then Tm
  float* sbeta = sA + C * (C + 1);  // [C]
  const int CS = C + 1;
  const int t0 = n * C;
  for (int idx = tid; idx < C * K; idx += 256) {
    int i = idx / K, kk = idx % K;
    int t = t0 + i;
    float kv = 0.f, qv = 0.f, gv = 0.f;
    if (t < T_) {
      int64_t qoff = ((int64_t)b * T_ + t) * ld_qk + (int64_t)h * K + kk;
      int64_t goff = ((int64_t)b * T_ + t) * ld_g + (int64_t)hv * K + kk;
      kv = ldf(k + qoff);
      qv = ldf(q + qoff) * scale;
      gv = fmaxf(ldf(g + goff), g_min);
    }
    sk[i * KS + kk] = kv;
    sq[i * KS + kk] = qv;
    sgam[i * KS + kk] = gv;
  }
  for (int i = tid; i < C; i += 256) {
    int t = t0 + i;
    sbeta[i] = t < T_ ? ldf(beta + ((int64_t)b * T_ + t) * ld_b + hv) : 0.f;
  }
  __syncthreads();
  // running sum of g over the chunk, one channel per thread
  for (int kk = tid; kk < K; kk += 256) {
    float acc = 0.f;
    for (int i = 0; i < C; ++i) {
      acc += sgam[i * KS + kk];
      sgam[i * KS + kk] = acc;
    }
  }
  __syncthreads();
  const int64_t bh = (int64_t)b * HV + hv;
  const int64_t Tp = (int64_t)NT * C;
  // A[i][j] (i>j) and Aqk[i][j] (i>=j): exact per-channel exponent differences
  float* aqk_out = ws.aqk + (bh * NT + n) * C * C;
  for (int idx = tid; idx < C * C; idx += 256) {
    int i = idx / C, j = idx % C;
    float a = 0.f, aq = 0.f;
    if (j <= i) {
      const float* ki = sk + i * KS;
      const float* kj = sk + j * KS;
      const float* qi = sq + i * KS;
      const float* gi = sgam + i * KS;
      const float* gj = sgam + j * KS;
      for (int kk = 0; kk < K; ++kk) {
        float e = expf(fminf(gi[kk] - gj[kk], 50.f)) * kj[kk];
        a = fmaf(ki[kk], e, a);
        aq = fmaf(qi[kk], e, aq);
      }
    }
    sA[i * CS + j] = (j < i) ? a * sbeta[i] : 0.f;
    aqk_out[idx] = aq;
  }
  __syncthreads();
  // qg, kg, dl to the workspace; sq <- exp(gamma) * k for the w product
  for (int idx = tid; idx < C * K; idx += 256) {
    int i = idx / K, kk = idx % K;
    float gm = sgam[i * KS + kk];
    float gl = sgam[(C - 1) * KS + kk];
    float eg = expf(gm);
    int64_t off = (bh * Tp + t0 + i) * K + kk;
    ws.qg[off] = sq[i * KS + kk] * eg;
    ws.kg[off] = sk[i * KS + kk] * expf(gl - gm);
    if (i == 0) ws.dl[(bh * NT + n) * K + kk] = expf(gl);
  }
  __syncthreads();
  for (int idx = tid; idx < C * K; idx += 256) {
    int i = idx / K, kk = idx % K;
    sq[i * KS + kk] = expf(sgam[i * KS + kk]) * sk[i * KS + kk];
  }
  // (I + A)^-1 by forward substitution; column c is independent of the others
  float* sT = sgam;  // reuse: [C][CS]  (C*CS <= C*KS needs C <= K; guarded on the host)
  __syncthreads();
  for (int c = tid; c < C; c += 256) {
    for (int i = 0; i < C; ++i) {
      float x = (i == c) ? 1.f : 0.f;
      if (i > c) {
        float acc = 0.f;
        for (int j = c; j < i; ++j) acc = fmaf(sA[i * CS + j], sT[j * CS + c], acc);
        x -= acc;
      }
      sT[i * CS + c] = (i >= c) ? x : 0.f;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < C * C; idx += 256) {
    int i = idx / C, j = idx % C;
    sT[i * CS + j] *= sbeta[j];
  }
  __syncthreads();
  // w = Tm (exp(gamma) k)
  for (int idx = tid; idx < C * K; idx += 256) {
    int i = idx / K, kk = idx % K;
    float acc = 0.f;
    for (int j = 0; j <= i; ++j) acc = fmaf(sT[i * CS + j], sq[j * KS + kk], acc);
    ws.w[(bh * Tp + t0 + i) * K + kk] = acc;
  }
  // u = Tm v  (v read straight from global; each element is used by C-j rows)
  for (int idx = tid; idx < C * V; idx += 256) {
    int i = idx / V, vv = idx % V;
    float acc = 0.f;
    for (int j = 0; j <= i; ++j) {
      int t = t0 + j;
      float x = t < T_ ? ldf(v + ((int64_t)b * T_ + t) * ld_v + (int64_t)hv * V + vv) : 0.f;
      acc = fmaf(sT[i * CS + j], x, acc);
    }
    ws.u[(bh * Tp + t0 + i) * V + vv] = acc;
  }
}

// =====================================================================================
// Chunked form, stage 2 (sequential over chunks): one CTA owns 32 value columns of one
// (batch, value head) and keeps that slice of the state in shared memory.
//   vt = u - w S ; o = qg S + Aqk vt ; S <- diag(dl) S + kg^T vt
// =====================================================================================
template <typename T>
__global__ void __launch_bounds__(256)
kda_chunk_scan_kernel(KdaChunkWs ws, const float* __restrict__ S0, T* __restrict__ o,
                      float* __restrict__ S_out, int T_, int HV, int K, int V, int C, int NT) {
  extern __shared__ float smem[];
  const int vb = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int VS = 32;
  const int Kp = (K + 3) & ~3;
  float* sw = smem;                  // [64][Kp]
  float* sqg = sw + KDA_CMAX * Kp;   // [64][Kp]
  float* skg = sqg + KDA_CMAX * Kp;  // [64][Kp]
  float* saqk = skg + KDA_CMAX * Kp; // [64][64]
  float* svt = saqk + KDA_CMAX * KDA_CMAX;  // [64][VS]  u, then vt
  float* sS = svt + KDA_CMAX * VS;   // [Kp][VS]
  float* sdl = sS + Kp * VS;         // [Kp]
  const int64_t bh = (int64_t)b * HV + hv;
  const int64_t Tp = (int64_t)NT * C;
  const int v0 = vb * VS;
  const int64_t sbase = bh * K * V;
  for (int idx = tid; idx < Kp * VS; idx += 256) {
    int kk = idx / VS, vv = idx % VS;
    sS[idx] = (S0 && kk < K && v0 + vv < V) ? S0[sbase + (int64_t)kk * V + v0 + vv] : 0.f;
  }
  // rows >= C of the staging tiles stay zero for the whole kernel
  for (int idx = tid; idx < KDA_CMAX * Kp; idx += 256) { sw[idx] = 0.f; sqg[idx] = 0.f; skg[idx] = 0.f; }
  for (int idx = tid; idx < KDA_CMAX * KDA_CMAX; idx += 256) saqk[idx] = 0.f;
  for (int idx = tid; idx < KDA_CMAX * VS; idx += 256) svt[idx] = 0.f;
  const int ty = tid >> 3, tx = tid & 7;  // rows 2ty,2ty+1 ; cols 4tx..4tx+3
  __syncthreads();
  for (int n = 0; n < NT; ++n) {
    const int64_t row0 = bh * Tp + (int64_t)n * C;
    for (int idx = tid; idx < C * K; idx += 256) {
      int i = idx / K, kk = idx % K;
      int64_t off = (row0 + i) * K + kk;
      sw[i * Kp + kk] = ws.w[off];
      sqg[i * Kp + kk] = ws.qg[off];
      skg[i * Kp + kk] = ws.kg[off];
    }
    for (int idx = tid; idx < C * C; idx += 256)
      saqk[(idx / C) * KDA_CMAX + (idx % C)] = ws.aqk[(bh * NT + n) * C * C + idx];
    for (int idx = tid; idx < C * VS; idx += 256) {
      int i = idx / VS, vv = idx % VS;
      svt[idx] = (v0 + vv < V) ? ws.u[(row0 + i) * V + v0 + vv] : 0.f;
    }
    for (int kk = tid; kk < Kp; kk += 256) sdl[kk] = kk < K ? ws.dl[(bh * NT + n) * K + kk] : 1.f;
    __syncthreads();
    // wS and qS for rows 2ty, 2ty+1
    float aw[2][4] = {}, aq[2][4] = {};
    const int r0 = 2 * ty;
    for (int kk = 0; kk < Kp; ++kk) {
      float4 sv = *reinterpret_cast<const float4*>(sS + kk * VS + 4 * tx);
      float w0 = sw[r0 * Kp + kk], w1 = sw[(r0 + 1) * Kp + kk];
      float q0 = sqg[r0 * Kp + kk], q1 = sqg[(r0 + 1) * Kp + kk];
      aw[0][0] = fmaf(w0, sv.x, aw[0][0]); aw[0][1] = fmaf(w0, sv.y, aw[0][1]);
      aw[0][2] = fmaf(w0, sv.z, aw[0][2]); aw[0][3] = fmaf(w0, sv.w, aw[0][3]);
      aw[1][0] = fmaf(w1, sv.x, aw[1][0]); aw[1][1] = fmaf(w1, sv.y, aw[1][1]);
      aw[1][2] = fmaf(w1, sv.z, aw[1][2]); aw[1][3] = fmaf(w1, sv.w, aw[1][3]);
      aq[0][0] = fmaf(q0, sv.x, aq[0][0]); aq[0][1] = fmaf(q0, sv.y, aq[0][1]);
      aq[0][2] = fmaf(q0, sv.z, aq[0][2]); aq[0][3] = fmaf(q0, sv.w, aq[0][3]);
      aq[1][0] = fmaf(q1, sv.x, aq[1][0]); aq[1][1] = fmaf(q1, sv.y, aq[1][1]);
      aq[1][2] = fmaf(q1, sv.z, aq[1][2]); aq[1][3] = fmaf(q1, sv.w, aq[1][3]);
    }
    // vt = u - wS (in place); every thread touches only its own 2x4 tile
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int cidx = 0; cidx < 4; ++cidx)
        svt[(r0 + r) * VS + 4 * tx + cidx] -= aw[r][cidx];
    __syncthreads();
    // o = qS + Aqk vt
    for (int j = 0; j < C; ++j) {
      float4 vv = *reinterpret_cast<const float4*>(svt + j * VS + 4 * tx);
      float a0 = saqk[r0 * KDA_CMAX + j], a1 = saqk[(r0 + 1) * KDA_CMAX + j];
      aq[0][0] = fmaf(a0, vv.x, aq[0][0]); aq[0][1] = fmaf(a0, vv.y, aq[0][1]);
      aq[0][2] = fmaf(a0, vv.z, aq[0][2]); aq[0][3] = fmaf(a0, vv.w, aq[0][3]);
      aq[1][0] = fmaf(a1, vv.x, aq[1][0]); aq[1][1] = fmaf(a1, vv.y, aq[1][1]);
      aq[1][2] = fmaf(a1, vv.z, aq[1][2]); aq[1][3] = fmaf(a1, vv.w, aq[1][3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int i = r0 + r;
      int t = n * C + i;
      if (i < C && t < T_) {
        T* orow = o + (((int64_t)b * T_ + t) * HV + hv) * V + v0 + 4 * tx;
#pragma unroll
        for (int cidx = 0; cidx < 4; ++cidx)
          if (v0 + 4 * tx + cidx < V) stf(orow + cidx, aq[r][cidx]);
      }
    }
    // S <- diag(dl) S + kg^T vt : thread owns rows kk = 4*ty' .. for a strided set of rows
    for (int kb = (tid >> 3) * 4; kb < Kp; kb += 128) {
      float acc[4][4] = {};
      for (int i = 0; i < C; ++i) {
        float4 kv = *reinterpret_cast<const float4*>(skg + i * Kp + kb);
        float4 vv = *reinterpret_cast<const float4*>(svt + i * VS + 4 * tx);
        const float kr[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          acc[r][0] = fmaf(kr[r], vv.x, acc[r][0]); acc[r][1] = fmaf(kr[r], vv.y, acc[r][1]);
          acc[r][2] = fmaf(kr[r], vv.z, acc[r][2]); acc[r][3] = fmaf(kr[r], vv.w, acc[r][3]);
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float d = sdl[kb + r];
        float4* sp = reinterpret_cast<float4*>(sS + (kb + r) * VS + 4 * tx);
        float4 sv = *sp;
        sv.x = fmaf(sv.x, d, acc[r][0]); sv.y = fmaf(sv.y, d, acc[r][1]);
        sv.z = fmaf(sv.z, d, acc[r][2]); sv.w = fmaf(sv.w, d, acc[r][3]);
        *sp = sv;
      }
    }
    __syncthreads();
  }
  if (S_out)
    for (int idx = tid; idx < K * VS; idx += 256) {
      int kk = idx / VS, vv = idx % VS;
      if (v0 + vv < V) S_out[sbase + (int64_t)kk * V + v0 + vv] = sS[kk * VS + vv];
    }
}

static size_t kda_ws_layout(KdaChunkWs* ws, char* base, int B, int HV, int K, int V, int C, int NT) {
  size_t bh = (size_t)B * HV, Tp = (size_t)NT * C, off = 0;
  auto take = [&](size_t n) { float* p = (float*)(base + off); off += ((n * 4 + 255) / 256) * 256; return p; };
  float* w = take(bh * Tp * K);
  float* qg = take(bh * Tp * K);
  float* kg = take(bh * Tp * K);
  float* u = take(bh * Tp * V);
  float* aqk = take(bh * NT * C * C);
  float* dl = take(bh * NT * K);
  if (ws) { ws->w = w; ws->qg = qg; ws->kg = kg; ws->u = u; ws->aqk = aqk; ws->dl = dl; }
  return off;
}

static int kda_chunk_effective(int K, int chunk) {
  // the prepare kernel reuses a [C][K+1] tile for the [C][C+1] inverse, so C <= K; larger
  // requests run as smaller chunks (same mathematics, different fp32 summation order)
  int C = chunk < KDA_CMAX ? chunk : KDA_CMAX;
  if (C > K) C = K;
  return C < 1 ? 1 : C;
}

// tensor-core path (kda_mma.cu)
bool kch_kda_mma_supported(int K, int V, int chunk_size, float g_clamp_min, int dtype);
int64_t kch_kda_mma_workspace_bytes(int B, int T, int HV);
int kch_kda_chunk_mma(const void* q, const void* k, const void* v, const void* g, const void* beta,
                      const float* initial_state, void* o, float* final_state, int B, int T, int H, int HV,
                      float scale, float g_clamp_min, int64_t ld_qk, int64_t ld_v, int64_t ld_g, int64_t ld_beta,
                      void* workspace, int64_t workspace_bytes, void* stream, float gate_scale);

extern "C" int64_t kch_kda_chunk_workspace_bytes(int B, int T, int HV, int K, int V, int chunk_size) {
  if (B <= 0 || T <= 0 || HV <= 0 || K <= 0 || V <= 0 || chunk_size < 1) return 0;
  int C = kda_chunk_effective(K, chunk_size);
  int NT = (T + C - 1) / C;
  int64_t need = (int64_t)kda_ws_layout(nullptr, nullptr, B, HV, K, V, C, NT);
  // the dtype is not known here: size for whichever path may run
  if (kch_kda_mma_supported(K, V, chunk_size, 0.f, KCH_BF16)) {
    int64_t m = kch_kda_mma_workspace_bytes(B, T, HV);
    if (m > need) need = m;
  }
  return need;
}

static int kda_chunk_impl(const void* q, const void* k, const void* v, const void* g,
                          const void* beta, const float* initial_state, void* o,
                          float* final_state, int B, int T, int H, int HV, int K, int V,
                          int chunk_size, float scale, float g_clamp_min, int dtype, int64_t ld_qk,
                          int64_t ld_v, int64_t ld_g, int64_t ld_beta, void* workspace,
                          int64_t workspace_bytes, void* stream, float gate_scale) {
  if (ld_qk <= 0) ld_qk = (int64_t)H * K;
  if (ld_v <= 0) ld_v = (int64_t)HV * V;
  if (ld_g <= 0) ld_g = (int64_t)HV * K;
  if (ld_beta <= 0) ld_beta = HV;
  KCH_REQUIRE(H >= 1, "H=%d must be >= 1", H);
  KCH_REQUIRE(K >= 1, "K=%d must be >= 1", K);
  KCH_REQUIRE(V >= 1, "V=%d must be >= 1", V);
  KCH_REQUIRE(chunk_size >= 1, "chunk_size=%d must be >= 1", chunk_size);
  KCH_REQUIRE(HV >= 1 && HV % H == 0, "HV=%d must be divisible by H=%d (GVA factor)", HV, H);
  KCH_REQUIRE(B >= 0 && T >= 0, "B=%d T=%d", B, T);
  if (gate_scale != 0.f)
    KCH_REQUIRE(T > 0 && K <= 128 && kch_kda_mma_supported(K, V, chunk_size, g_clamp_min, dtype),
                "kch_kda_chunk_gate: the fused gate activation needs bf16, K = V = 128, chunk_size = 64 (K=%d V=%d chunk=%d)",
                K, V, chunk_size);
  if (K > 128)  // state slice + staging tiles exceed shared memory: same maths, token form
    return kch_kda_recurrent(q, k, v, g, beta, initial_state, o, final_state, B, T, H, HV, K, V, scale,
                             g_clamp_min, dtype, ld_qk, ld_v, ld_g, ld_beta, stream);
  if (B == 0) return KCH_OK;
  if (T > 0 && kch_kda_mma_supported(K, V, chunk_size, g_clamp_min, dtype))
    return kch_kda_chunk_mma(q, k, v, g, beta, initial_state, o, final_state, B, T, H, HV, scale, g_clamp_min,
                             ld_qk, ld_v, ld_g, ld_beta, workspace, workspace_bytes, stream, gate_scale);
  if (T == 0) {
    if (final_state) {
      size_t nb = (size_t)B * HV * K * V * sizeof(float);
      if (initial_state) KCH_CUDA_OK(cudaMemcpyAsync(final_state, initial_state, nb, cudaMemcpyDeviceToDevice, kch_stream(stream)));
      else KCH_CUDA_OK(cudaMemsetAsync(final_state, 0, nb, kch_stream(stream)));
    }
    return KCH_OK;
  }
  int C = kda_chunk_effective(K, chunk_size);
  int NT = (T + C - 1) / C;
  KdaChunkWs ws;
  size_t need = kda_ws_layout(&ws, (char*)workspace, B, HV, K, V, C, NT);
  KCH_REQUIRE(workspace && (size_t)workspace_bytes >= need, "kch_kda_chunk: workspace %lld < %lld bytes",
              (long long)workspace_bytes, (long long)need);
  cudaStream_t s = kch_stream(stream);
  size_t smem1 = ((size_t)3 * C * (K + 1) + (size_t)C * (C + 1) + C) * sizeof(float);
  int Kp = (K + 3) & ~3;
  size_t smem2 = ((size_t)3 * KDA_CMAX * Kp + KDA_CMAX * KDA_CMAX + KDA_CMAX * 32 + (size_t)Kp * 32 + Kp) * sizeof(float);
  dim3 g1(NT, HV, B), g2((V + 31) / 32, HV, B);
#define GO(T_)                                                                                       \
  do {                                                                                               \
    KCH_CUDA_OK(cudaFuncSetAttribute(kda_chunk_prepare_kernel<T_>,                                   \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));      \
    KCH_CUDA_OK(cudaFuncSetAttribute(kda_chunk_scan_kernel<T_>,                                      \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));      \
    kda_chunk_prepare_kernel<T_><<<g1, 256, smem1, s>>>((const T_*)q, (const T_*)k, (const T_*)v,    \
        (const T_*)g, (const T_*)beta, ws, T, H, HV, K, V, C, NT, scale, g_clamp_min, ld_qk, ld_v,    \
        ld_g, ld_beta);                                                                              \
    kda_chunk_scan_kernel<T_><<<g2, 256, smem2, s>>>(ws, initial_state, (T_*)o, final_state, T, HV,  \
        K, V, C, NT);                                                                                \
  } while (0)
  KCH_DISPATCH_FLOAT(dtype, T_, GO(T_));
#undef GO
  kch_note_launch(1);  // two kernels per call
  KCH_LAUNCH_OK();
  return KCH_OK;
}

extern "C" int kch_kda_chunk(const void* q, const void* k, const void* v, const void* g,
                             const void* beta, const float* initial_state, void* o,
                             float* final_state, int B, int T, int H, int HV, int K, int V,
                             int chunk_size, float scale, float g_clamp_min, int dtype, int64_t ld_qk,
                             int64_t ld_v, int64_t ld_g, int64_t ld_beta, void* workspace,
                             int64_t workspace_bytes, void* stream) {
  return kda_chunk_impl(q, k, v, g, beta, initial_state, o, final_state, B, T, H, HV, K, V, chunk_size, scale,
                        g_clamp_min, dtype, ld_qk, ld_v, ld_g, ld_beta, workspace, workspace_bytes, stream, 0.f);
}

extern "C" int kch_kda_chunk_gate_supported(int K, int V, int chunk_size, float g_clamp_min, int dtype) {
  return K <= 128 && kch_kda_mma_supported(K, V, chunk_size, g_clamp_min, dtype) ? 1 : 0;
}

extern "C" int kch_kda_chunk_gate(const void* q, const void* k, const void* v, const void* g_pre,
                                  const void* beta, const float* initial_state, void* o,
                                  float* final_state, int B, int T, int H, int HV, int K, int V,
                                  int chunk_size, float scale, float g_clamp_min, float gate_scale, int dtype,
                                  int64_t ld_qk, int64_t ld_v, int64_t ld_g, int64_t ld_beta, void* workspace,
                                  int64_t workspace_bytes, void* stream) {
  KCH_REQUIRE(gate_scale > 0.f, "kch_kda_chunk_gate: gate_scale=%g must be > 0", (double)gate_scale);
  return kda_chunk_impl(q, k, v, g_pre, beta, initial_state, o, final_state, B, T, H, HV, K, V, chunk_size, scale,
                        g_clamp_min, dtype, ld_qk, ld_v, ld_g, ld_beta, workspace, workspace_bytes, stream, gate_scale);
}
