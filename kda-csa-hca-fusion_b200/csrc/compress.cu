// KV compression: per block of m tokens and per channel, a softmax over the block's
// positions (logits Z + positional bias) weights the entries C.
//   single branch : csa_compress_kv            (ops_csa.py:198-234)
//   two branches  : csa_compress_kv_overlapped (ops_csa.py:237-305), block i also mixes the
//                   b-branch of block i-1 under the same softmax (absent for block 0).
// HBM-bound: every input element is read exactly once, every output written once.  Inputs may be
// column slices of a wider projection output (row stride ld).  Output fp32.
//   compress_vec_kernel : bf16 inputs, c a power of two times 8.  A thread owns 8 channels (one 16-byte
//                         load per row and operand) and a subset of the block's rows, carries a running
//                         (max, denominator, weighted sum) per channel -- one pass over the data -- and
//                         the subsets are merged by shuffles inside a warp and through shared memory
//                         between the warps of a block of tokens (m = 128 uses all 256 threads of a CTA
//                         on one block: 16 row subsets x 16 channel chunks).
//   compress_kernel     : any dtype / width: a thread owns one (batch, block, channel), two passes.
#include <math.h>

#include "kch_common.cuh"

template <typename T, typename TB, bool OVERLAP>
__global__ void compress_kernel(const T* __restrict__ Ca, const T* __restrict__ Za,
                                      const T* __restrict__ Cb, const T* __restrict__ Zb,
                                      const TB* __restrict__ Ba, const TB* __restrict__ Bb,
                                      const T* __restrict__ prevCb, const T* __restrict__ prevZb,
                                      float* __restrict__ out, int64_t ld, int64_t batch_stride_rows,
                                      int B, int nblk, int c, int m, int64_t out_batch_stride,
                                      int64_t prev_ld) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)B * nblk * c;
  if (i >= total) return;
  int ch = (int)(i % c);
  int64_t bn = i / c;
  int n = (int)(bn % nblk);
  int b = (int)(bn / nblk);
  int64_t row0 = (int64_t)b * batch_stride_rows + (int64_t)n * m;
  const T* pc = nullptr;
  const T* pz = nullptr;
  int64_t pld = ld, prow = 0;
  if (OVERLAP) {
    if (n > 0) { pc = Cb; pz = Zb; prow = row0 - m; }
    else if (prevCb) { pc = prevCb; pz = prevZb; pld = prev_ld; prow = (int64_t)b * m; }
  }
  // two passes (max, then sum) exactly as a dense softmax would do it
  float mx = -INFINITY;
  for (int j = 0; j < m; ++j)
    mx = fmaxf(mx, ldf(Za + (row0 + j) * ld + ch) + ldf(Ba + (int64_t)j * c + ch));
  if (pc)
    for (int j = 0; j < m; ++j)
      mx = fmaxf(mx, ldf(pz + (prow + j) * pld + ch) + ldf(Bb + (int64_t)j * c + ch));
  float den = 0.f, acc = 0.f;
  for (int j = 0; j < m; ++j) {
    int64_t off = (row0 + j) * ld + ch;
    float e = expf(ldf(Za + off) + ldf(Ba + (int64_t)j * c + ch) - mx);
    den += e;
    acc = fmaf(e, ldf(Ca + off), acc);
  }
  float accb = 0.f;
  if (pc)
    for (int j = 0; j < m; ++j) {
      int64_t off = (prow + j) * pld + ch;
      float e = expf(ldf(pz + off) + ldf(Bb + (int64_t)j * c + ch) - mx);
      den += e;
      accb = fmaf(e, ldf(pc + off), accb);
    }
  out[(int64_t)b * out_batch_stride + (int64_t)n * c + ch] = acc / den + accb / den;
}

// running softmax-weighted sum over rows, 8 channels per thread
struct CvState { float mx[8], den[8], acc[8]; };
__device__ __forceinline__ void cv_init(CvState& st) {
#pragma unroll
  for (int k = 0; k < 8; ++k) { st.mx[k] = -INFINITY; st.den[k] = 0.f; st.acc[k] = 0.f; }
}
__device__ __forceinline__ void cv_row(CvState& st, const uint4& zr, const uint4& cr, const float (&bias)[8]) {
  const bf16* z = reinterpret_cast<const bf16*>(&zr);
  const bf16* cv = reinterpret_cast<const bf16*>(&cr);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float lg = __bfloat162float(z[k]) + bias[k];
    const float nm = fmaxf(st.mx[k], lg);
    const float so = __expf(st.mx[k] - nm), e = __expf(lg - nm);       // so = 0 for the first row (mx = -inf)
    st.den[k] = fmaf(st.den[k], so, e);
    st.acc[k] = fmaf(st.acc[k], so, e * __bfloat162float(cv[k]));
    st.mx[k] = nm;
  }
}
__device__ __forceinline__ void cv_merge(float& mx, float& den, float& acc, float omx, float oden, float oacc) {
  const float nm = fmaxf(mx, omx);
  const float s1 = mx == -INFINITY ? 0.f : __expf(mx - nm), s2 = omx == -INFINITY ? 0.f : __expf(omx - nm);
  den = den * s1 + oden * s2;
  acc = acc * s1 + oacc * s2;
  mx = nm;
}

template <typename TB, bool OVERLAP>
__global__ void __launch_bounds__(256)
compress_vec_kernel(const bf16* __restrict__ Ca, const bf16* __restrict__ Za, const bf16* __restrict__ Cb,
                    const bf16* __restrict__ Zb, const TB* __restrict__ Ba, const TB* __restrict__ Bb,
                    const bf16* __restrict__ prevCb, const bf16* __restrict__ prevZb, float* __restrict__ out,
                    int64_t ld, int64_t batch_stride_rows, int B, int nblk, int c, int m, int64_t out_batch_stride,
                    int64_t prev_ld, int cpr, int wpu) {
  // cpr = c / 8 chunks per row (power of two <= 32); wpu warps work on one block of m tokens (1, 2, 4 or 8)
  extern __shared__ float cv_smem[];                      // [8 warps][c][3] when wpu > 1
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c8 = lane & (cpr - 1), sub = lane / cpr, subs = 32 / cpr;
  const int unit_in_cta = warp / wpu, wsub = warp % wpu;
  const int64_t unit = (int64_t)blockIdx.x * (8 / wpu) + unit_in_cta;
  const bool live = unit < (int64_t)B * nblk;
  const int n = live ? (int)(unit % nblk) : 0, b = live ? (int)(unit / nblk) : 0;
  const int splits = wpu * subs, split = wsub * subs + sub;
  const int64_t row0 = (int64_t)b * batch_stride_rows + (int64_t)n * m;
  CvState st;
  cv_init(st);
  if (live) {
    for (int j = split; j < m; j += splits) {
      const int64_t off = (row0 + j) * ld + 8 * c8;
      const uint4 zr = *reinterpret_cast<const uint4*>(Za + off);
      const uint4 cr = *reinterpret_cast<const uint4*>(Ca + off);
      float bias[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) bias[k] = ldf(Ba + (int64_t)j * c + 8 * c8 + k);
      cv_row(st, zr, cr, bias);
    }
    if (OVERLAP) {
      const bf16* pc = nullptr;
      const bf16* pz = nullptr;
      int64_t pld = ld, prow = 0;
      if (n > 0) { pc = Cb; pz = Zb; prow = row0 - m; }
      else if (prevCb) { pc = prevCb; pz = prevZb; pld = prev_ld; prow = (int64_t)b * m; }
      if (pc)
        for (int j = split; j < m; j += splits) {
          const int64_t off = (prow + j) * pld + 8 * c8;
          const uint4 zr = *reinterpret_cast<const uint4*>(pz + off);
          const uint4 cr = *reinterpret_cast<const uint4*>(pc + off);
          float bias[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) bias[k] = ldf(Bb + (int64_t)j * c + 8 * c8 + k);
          cv_row(st, zr, cr, bias);
        }
    }
  }
  // row subsets held by the lanes of this warp
  for (int o = cpr; o < 32; o <<= 1) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float omx = __shfl_xor_sync(0xffffffffu, st.mx[k], o), oden = __shfl_xor_sync(0xffffffffu, st.den[k], o),
                  oacc = __shfl_xor_sync(0xffffffffu, st.acc[k], o);
      cv_merge(st.mx[k], st.den[k], st.acc[k], omx, oden, oacc);
    }
  }
  if (wpu > 1) {                                          // ... and by the other warps of the block
    float* mine = cv_smem + ((size_t)warp * c + 8 * c8) * 3;
    if (sub == 0)
#pragma unroll
      for (int k = 0; k < 8; ++k) { mine[3 * k] = st.mx[k]; mine[3 * k + 1] = st.den[k]; mine[3 * k + 2] = st.acc[k]; }
    __syncthreads();
    if (wsub == 0 && sub == 0)
      for (int w2 = 1; w2 < wpu; ++w2) {
        const float* oth = cv_smem + ((size_t)(warp + w2) * c + 8 * c8) * 3;
#pragma unroll
        for (int k = 0; k < 8; ++k) cv_merge(st.mx[k], st.den[k], st.acc[k], oth[3 * k], oth[3 * k + 1], oth[3 * k + 2]);
      }
  }
  if (live && wsub == 0 && sub == 0) {
    float4* dst = reinterpret_cast<float4*>(out + (int64_t)b * out_batch_stride + (int64_t)n * c + 8 * c8);
    dst[0] = make_float4(st.acc[0] / st.den[0], st.acc[1] / st.den[1], st.acc[2] / st.den[2], st.acc[3] / st.den[3]);
    dst[1] = make_float4(st.acc[4] / st.den[4], st.acc[5] / st.den[5], st.acc[6] / st.den[6], st.acc[7] / st.den[7]);
  }
}

static int launch_compress(const void* Ca, const void* Za, const void* Cb, const void* Zb,
                           const void* Ba, const void* Bb, const void* prevCb, const void* prevZb,
                           float* out, int64_t ld, int64_t batch_stride_rows, int B, int nblk, int c,
                           int m, int64_t out_batch_stride, int64_t prev_ld, int dtype, int bdtype,
                           bool overlap, void* stream) {
  int64_t total = (int64_t)B * nblk * c;
  if (total == 0) return KCH_OK;
  cudaStream_t s = kch_stream(stream);
  {
    // vectorised kernel: bf16 rows of a power-of-two number (<= 32) of 16-byte chunks, everything 16-byte aligned
    static const bool scalar_only = [] { const char* e = getenv("KCH_COMPRESS"); return e && e[0] == 's'; }();
    const int cpr = c / 8;
    const uintptr_t al = (uintptr_t)Ca | (uintptr_t)Za | (uintptr_t)Cb | (uintptr_t)Zb | (uintptr_t)prevCb | (uintptr_t)prevZb |
                         (uintptr_t)out;
    if (!scalar_only && dtype == KCH_BF16 && c % 8 == 0 && cpr >= 1 && cpr <= 32 && (cpr & (cpr - 1)) == 0 && (ld % 8) == 0 &&
        (prev_ld % 8) == 0 && (al & 15) == 0 && (out_batch_stride % 4) == 0) {
      // enough row subsets that a thread sees about four rows: warps per block of tokens
      const int subs = 32 / cpr;
      int wpu = 1;
      while (wpu < 8 && m > 4 * subs * wpu) wpu *= 2;
      const int64_t units = (int64_t)B * nblk;
      const unsigned g = (unsigned)ceil_div64(units, 8 / wpu);
      const size_t smem = wpu > 1 ? (size_t)8 * c * 3 * sizeof(float) : 0;
#define GOV(TB, OV)                                                                                              \
      compress_vec_kernel<TB, OV><<<g, 256, smem, s>>>((const bf16*)Ca, (const bf16*)Za, (const bf16*)Cb, (const bf16*)Zb, \
          (const TB*)Ba, (const TB*)Bb, (const bf16*)prevCb, (const bf16*)prevZb, out, ld, batch_stride_rows, B, nblk, c, m, \
          out_batch_stride, prev_ld, cpr, wpu)
      if (overlap) { KCH_DISPATCH_FLOAT(bdtype, TB, (GOV(TB, true))); }
      else { KCH_DISPATCH_FLOAT(bdtype, TB, (GOV(TB, false))); }
#undef GOV
      KCH_LAUNCH_OK();
      return KCH_OK;
    }
  }
  dim3 grid((unsigned)ceil_div64(total, 128)), block(128);
#define GO(T, TB, OV)                                                                           \
  compress_kernel<T, TB, OV><<<grid, block, 0, s>>>(                                      \
      (const T*)Ca, (const T*)Za, (const T*)Cb, (const T*)Zb, (const TB*)Ba, (const TB*)Bb,     \
      (const T*)prevCb, (const T*)prevZb, out, ld, batch_stride_rows, B, nblk, c, m,            \
      out_batch_stride, prev_ld)
  if (overlap) {
    KCH_DISPATCH_FLOAT(dtype, T, KCH_DISPATCH_FLOAT(bdtype, TB, (GO(T, TB, true))));
  } else {
    KCH_DISPATCH_FLOAT(dtype, T, KCH_DISPATCH_FLOAT(bdtype, TB, (GO(T, TB, false))));
  }
#undef GO
  KCH_LAUNCH_OK();
  return KCH_OK;
}

extern "C" int kch_compress_kv(const void* C, const void* Z, const void* B_pos, float* out, int B,
                               int64_t T, int c, int m, int64_t ld, int64_t batch_stride_rows,
                               int64_t out_batch_stride_elems, int dtype, int bias_dtype, void* stream) {
  KCH_REQUIRE(m >= 1, "compression factor m=%d must be >= 1", m);
  KCH_REQUIRE(T % m == 0, "T=%lld must be divisible by m=%d", (long long)T, m);
  KCH_REQUIRE(B >= 0 && c >= 1 && ld >= c, "kch_compress_kv: B=%d c=%d ld=%lld", B, c, (long long)ld);
  return launch_compress(C, Z, nullptr, nullptr, B_pos, nullptr, nullptr, nullptr, out, ld,
                         batch_stride_rows, B, (int)(T / m), c, m, out_batch_stride_elems, 0, dtype,
                         bias_dtype, false, stream);
}

extern "C" int kch_compress_kv_overlapped(const void* Ca, const void* Cb, const void* Za,
                                          const void* Zb, const void* Ba, const void* Bb,
                                          const void* prev_Cb, const void* prev_Zb, int64_t prev_ld,
                                          float* out, int B, int64_t T, int c, int m, int64_t ld,
                                          int64_t batch_stride_rows, int64_t out_batch_stride_elems,
                                          int dtype, int bias_dtype, void* stream) {
  KCH_REQUIRE(m >= 1, "compression factor m=%d must be >= 1", m);
  KCH_REQUIRE(T % m == 0, "T=%lld must be divisible by m=%d", (long long)T, m);
  KCH_REQUIRE(B >= 0 && c >= 1 && ld >= c, "kch_compress_kv_overlapped: B=%d c=%d ld=%lld", B, c,
              (long long)ld);
  KCH_REQUIRE((prev_Cb == nullptr) == (prev_Zb == nullptr), "prev_Cb and prev_Zb must be given together");
  return launch_compress(Ca, Za, Cb, Zb, Ba, Bb, prev_Cb, prev_Zb, out, ld, batch_stride_rows, B,
                         (int)(T / m), c, m, out_batch_stride_elems, prev_ld, dtype, bias_dtype, true,
                         stream);
}
