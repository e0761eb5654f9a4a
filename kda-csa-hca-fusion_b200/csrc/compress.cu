// KV compression: per block of m tokens and per channel, a softmax over the block's
// positions (logits Z + positional bias) weights the entries C.
//   single branch : csa_compress_kv            (ops_csa.py:198-234)
//   two branches  : csa_compress_kv_overlapped (ops_csa.py:237-305), block i also mixes the
//                   b-branch of block i-1 under the same softmax (absent for block 0).
// HBM-bound: every input element is read exactly once, every output written once.  A thread
// owns one (batch, block, channel); consecutive threads own consecutive channels, so each
// token row is read with fully coalesced accesses.  Inputs may be column slices of a wider
// projection output (row stride ld).  Output fp32 (optionally also rounded to bf16 rows for
// the decode caches).
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

static int launch_compress(const void* Ca, const void* Za, const void* Cb, const void* Zb,
                           const void* Ba, const void* Bb, const void* prevCb, const void* prevZb,
                           float* out, int64_t ld, int64_t batch_stride_rows, int B, int nblk, int c,
                           int m, int64_t out_batch_stride, int64_t prev_ld, int dtype, int bdtype,
                           bool overlap, void* stream) {
  int64_t total = (int64_t)B * nblk * c;
  if (total == 0) return KCH_OK;
  dim3 grid((unsigned)ceil_div64(total, 128)), block(128);
  cudaStream_t s = kch_stream(stream);
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
