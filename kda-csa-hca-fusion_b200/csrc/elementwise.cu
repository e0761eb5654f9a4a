// Row-wise glue kernels of the hybrid layer: fp32 LayerNorm, the causal depthwise
// short convolution, activation epilogues, L2 row normalisation.
// All are single-pass HBM-bound kernels: one read of the input, one write of the output.
#include <math.h>

#include "kch_common.cuh"

// ---------------------------------------------------------------------------------------
// LayerNorm evaluated in fp32, stored in the input dtype.  One warp per row.
// Follows _Fp32LayerNorm.forward (ops_fused.py:52-60).
// ---------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void layernorm_kernel(const T* __restrict__ x, const TW* __restrict__ w,
                                 const TW* __restrict__ b, T* __restrict__ y, int64_t rows, int d,
                                 float eps) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * d;
  float s = 0.f;
  for (int i = lane; i < d; i += 32) s += ldf(xr + i);
  float mean = warp_sum(s) / (float)d;
  float v = 0.f;
  for (int i = lane; i < d; i += 32) {
    float t = ldf(xr + i) - mean;
    v += t * t;
  }
  float rstd = 1.0f / sqrtf(warp_sum(v) / (float)d + eps);
  T* yr = y + row * d;
  for (int i = lane; i < d; i += 32)
    stf(yr + i, (ldf(xr + i) - mean) * rstd * ldf(w + i) + ldf(b + i));
}

// bf16 fast path for d % 256 == 0 and d <= 4096: 8 values per lane per 256 columns, row kept in registers
template <typename TW, int NV>
__global__ void layernorm_kernel_bf16_vec(const bf16* __restrict__ x, const TW* __restrict__ w,
                                          const TW* __restrict__ b, bf16* __restrict__ y, int64_t rows, int d,
                                          float eps) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + row * d;
  float v[NV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    uint4 raw = *reinterpret_cast<const uint4*>(xr + i * 256 + lane * 8);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) { v[i][k] = __bfloat162float(e[k]); s += v[i][k]; }
  }
  const float mean = warp_sum(s) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 8; ++k) { float t = v[i][k] - mean; q += t * t; }
  const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)d + eps);
  bf16* yr = y + row * d;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    uint4 outv;
    bf16* out = reinterpret_cast<bf16*>(&outv);
    const int c0 = i * 256 + lane * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = __float2bfloat16_rn((v[i][k] - mean) * rstd * ldf(w + c0 + k) + ldf(b + c0 + k));
    *reinterpret_cast<uint4*>(yr + c0) = outv;
  }
}

// A few rows only (a decode batch): one CTA per row, 8 channels per thread, so every load of the row and of the
// parameters is issued at once and the launch is one memory round trip plus two block reductions.
template <typename TW>
__device__ __forceinline__ void ld8p(const TW* p, float (&o)[8]) {
  if constexpr (sizeof(TW) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = __bfloat162float(e[k]);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  }
}
// sum over the 256 threads of a CTA; `red` is 8 floats of shared memory (reusable after the call returns)
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
}

template <typename TW>
__global__ void __launch_bounds__(256)
layernorm_row_kernel_bf16(const bf16* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                          bf16* __restrict__ y, int d, float eps) {
  __shared__ float red[8];
  const int c0 = threadIdx.x * 8;
  const bool on = c0 < d;
  const int64_t row = blockIdx.x;
  float v[8], wv[8], bv[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = wv[k] = bv[k] = 0.f;
  if (on) { ld8p(x + row * d + c0, v); ld8p(w + c0, wv); ld8p(b + c0, bv); }
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += v[k];
  const float mean = block_sum_256(s, red) / (float)d;
  float q = 0.f;
  if (on) {
#pragma unroll
    for (int k = 0; k < 8; ++k) { const float t = v[k] - mean; q += t * t; }
  }
  const float rstd = 1.0f / sqrtf(block_sum_256(q, red) / (float)d + eps);
  if (on) {
    uint4 outv;
    bf16* out = reinterpret_cast<bf16*>(&outv);
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = __float2bfloat16_rn((v[k] - mean) * rstd * wv[k] + bv[k]);
    *reinterpret_cast<uint4*>(y + row * d + c0) = outv;
  }
}

extern "C" int kch_layernorm(const void* x, const void* weight, const void* bias, void* y,
                             int64_t rows, int d, float eps, int dtype, int wdtype, void* stream) {
  KCH_REQUIRE(rows >= 0 && d >= 1, "kch_layernorm: rows=%lld d=%d", (long long)rows, d);
  if (rows == 0) return KCH_OK;
  const int wpb = 8;
  dim3 grid((unsigned)ceil_div64(rows, wpb)), block(wpb * 32);
  if (dtype == KCH_BF16 && rows <= 512 && (d % 8) == 0 && d <= 2048 &&
      (((uintptr_t)x | (uintptr_t)y | (uintptr_t)weight | (uintptr_t)bias) & 15) == 0) {
    cudaStream_t s = kch_stream(stream);
    KCH_DISPATCH_FLOAT(wdtype, TW, (layernorm_row_kernel_bf16<TW><<<(unsigned)rows, 256, 0, s>>>(
        (const bf16*)x, (const TW*)weight, (const TW*)bias, (bf16*)y, d, eps)));
    KCH_LAUNCH_OK();
    return KCH_OK;
  }
  if (dtype == KCH_BF16 && (d % 256) == 0 && d <= 2048 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
    cudaStream_t s = kch_stream(stream);
#define LNV(NV)                                                                                              \
    KCH_DISPATCH_FLOAT(wdtype, TW, (layernorm_kernel_bf16_vec<TW, NV><<<grid, block, 0, s>>>(                 \
        (const bf16*)x, (const TW*)weight, (const TW*)bias, (bf16*)y, rows, d, eps)))
    switch (d / 256) {
      case 1: LNV(1); break; case 2: LNV(2); break; case 3: LNV(3); break; case 4: LNV(4); break;
      case 5: LNV(5); break; case 6: LNV(6); break; case 7: LNV(7); break; default: LNV(8); break;
    }
#undef LNV
    KCH_LAUNCH_OK();
    return KCH_OK;
  }
  KCH_DISPATCH_FLOAT(dtype, T, KCH_DISPATCH_FLOAT(wdtype, TW,
      (layernorm_kernel<T, TW><<<grid, block, 0, kch_stream(stream)>>>(
          (const T*)x, (const TW*)weight, (const TW*)bias, (T*)y, rows, d, eps))));
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// ---------------------------------------------------------------------------------------
// Causal depthwise convolution over time, kernel size 3, with bias:
//   y[b,t,ch] = bias[ch] + w[ch,0] x[t-2] + w[ch,1] x[t-1] + w[ch,2] x[t]
// where x[-1], x[-2] come from the [B,2,d] lookback (zeros when absent).
// Follows KDAHybridLayer.forward_functional (ops_fused.py:505-527).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ x, const T* lb,
                                  const T* __restrict__ w, const T* __restrict__ bias,
                                  T* __restrict__ y, int B, int T_, int d, T* lb_out = nullptr) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)B * T_ * d;
  if (i >= total) return;
  int ch = (int)(i % d);
  int64_t bt = i / d;
  int t = (int)(bt % T_);
  int b = (int)(bt / T_);
  const T* xb = x + (int64_t)b * T_ * d;
  float x0 = ldf(xb + (int64_t)t * d + ch);
  float x1, x2;
  if (t >= 1) x1 = ldf(xb + (int64_t)(t - 1) * d + ch);
  else x1 = lb ? ldf(lb + ((int64_t)b * 2 + 1) * d + ch) : 0.f;
  if (t >= 2) x2 = ldf(xb + (int64_t)(t - 2) * d + ch);
  else x2 = lb ? ldf(lb + ((int64_t)b * 2 + t) * d + ch) : 0.f;
  float acc = ldf(w + ch * 3 + 0) * x2;
  acc = fmaf(ldf(w + ch * 3 + 1), x1, acc);
  acc = fmaf(ldf(w + ch * 3 + 2), x0, acc);
  stf(y + i, acc + ldf(bias + ch));
  if (lb_out) {   // one-token step: the lookback slides by one token, in place (this thread owns channel ch)
    stf(lb_out + ((int64_t)b * 2 + 0) * d + ch, x1);
    stf(lb_out + ((int64_t)b * 2 + 1) * d + ch, x0);
  }
}

// bf16 fast path: 8 channels (16 bytes) per thread
__global__ void short_conv_kernel_bf16x8(const bf16* __restrict__ x, const bf16* lb,
                                         const bf16* __restrict__ w, const bf16* __restrict__ bias,
                                         bf16* __restrict__ y, int B, int T_, int d, bf16* lb_out = nullptr) {
  const int d8 = d >> 3;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)B * T_ * d8) return;
  const int c0 = (int)(i % d8) * 8;
  const int64_t bt = i / d8;
  const int t = (int)(bt % T_), b = (int)(bt / T_);
  const bf16* xb = x + (int64_t)b * T_ * d;
  auto ld8 = [&](const bf16* p, float (&o)[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = __bfloat162float(e[k]);
  };
  float x0[8], x1[8], x2[8], bb[8];
  ld8(xb + (int64_t)t * d + c0, x0);
  if (t >= 1) ld8(xb + (int64_t)(t - 1) * d + c0, x1);
  else if (lb) ld8(lb + ((int64_t)b * 2 + 1) * d + c0, x1);
  else {
#pragma unroll
    for (int k = 0; k < 8; ++k) x1[k] = 0.f;
  }
  if (t >= 2) ld8(xb + (int64_t)(t - 2) * d + c0, x2);
  else if (lb) ld8(lb + ((int64_t)b * 2 + t) * d + c0, x2);
  else {
#pragma unroll
    for (int k = 0; k < 8; ++k) x2[k] = 0.f;
  }
  ld8(bias + c0, bb);
  // taps of 8 channels: 24 consecutive bf16 (48 bytes, 16-byte aligned because c0 % 8 == 0)
  float wt[24];
  {
    const uint4* wp = reinterpret_cast<const uint4*>(w + c0 * 3);
#pragma unroll
    for (int v = 0; v < 3; ++v) {
      uint4 raw = wp[v];
      const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) wt[8 * v + k] = __bfloat162float(e[k]);
    }
  }
  uint4 outv;
  bf16* out = reinterpret_cast<bf16*>(&outv);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float acc = wt[3 * k] * x2[k];
    acc = fmaf(wt[3 * k + 1], x1[k], acc);
    acc = fmaf(wt[3 * k + 2], x0[k], acc);
    out[k] = __float2bfloat16_rn(acc + bb[k]);
  }
  *reinterpret_cast<uint4*>(y + bt * d + c0) = outv;
  if (lb_out) {   // one-token step (T_ == 1): slide the lookback in place; the values are exact bf16 already
    uint4 v1, v0;
    bf16* e1 = reinterpret_cast<bf16*>(&v1);
    bf16* e0 = reinterpret_cast<bf16*>(&v0);
#pragma unroll
    for (int k = 0; k < 8; ++k) { e1[k] = __float2bfloat16_rn(x1[k]); e0[k] = __float2bfloat16_rn(x0[k]); }
    *reinterpret_cast<uint4*>(lb_out + ((int64_t)b * 2 + 0) * d + c0) = v1;
    *reinterpret_cast<uint4*>(lb_out + ((int64_t)b * 2 + 1) * d + c0) = v0;
  }
}

extern "C" int kch_short_conv(const void* x, const void* lookback, const void* weight,
                              const void* bias, void* y, int B, int T, int d, int dtype,
                              void* stream) {
  KCH_REQUIRE(B >= 0 && T >= 0 && d >= 1, "kch_short_conv: B=%d T=%d d=%d", B, T, d);
  int64_t total = (int64_t)B * T * d;
  if (total == 0) return KCH_OK;
  const uintptr_t al = (uintptr_t)x | (uintptr_t)y | (uintptr_t)weight | (uintptr_t)bias | (uintptr_t)lookback;
  if (dtype == KCH_BF16 && (d % 8) == 0 && (al & 15) == 0) {
    dim3 grid((unsigned)ceil_div64(total / 8, 256)), block(256);
    short_conv_kernel_bf16x8<<<grid, block, 0, kch_stream(stream)>>>((const bf16*)x, (const bf16*)lookback,
                                                                    (const bf16*)weight, (const bf16*)bias, (bf16*)y, B, T, d);
  } else {
    dim3 grid((unsigned)ceil_div64(total, 256)), block(256);
    KCH_DISPATCH_FLOAT(dtype, T_, (short_conv_kernel<T_><<<grid, block, 0, kch_stream(stream)>>>(
        (const T_*)x, (const T_*)lookback, (const T_*)weight, (const T_*)bias, (T_*)y, B, T, d)));
  }
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// ---------------------------------------------------------------------------------------
// LayerNorm + short convolution in one pass (the KDA sub-layer reads LayerNorm(x) only through the
// convolution, ops_fused.py:505-527 after :52-60): a CTA normalises a tile of LC_TT tokens plus the two
// tokens before it into shared memory (bf16, exactly what the separate LayerNorm kernel would have stored)
// and convolves from there, so the normalised activations never travel to HBM and back.  The two
// normalised rows that end the sequence are written out as the next call's lookback.
// HBM traffic per token: d*2 bytes in, d*2 bytes out (+ 2/LC_TT re-read of the halo rows, L2 hits).
// ---------------------------------------------------------------------------------------
#define LC_TT 14
#define LC_ROWS (LC_TT + 2)

template <typename TW, int NV>
__global__ void __launch_bounds__(256)
ln_conv_kernel_bf16(const bf16* __restrict__ x, const TW* __restrict__ lw, const TW* __restrict__ lb2, float eps,
                    const bf16* __restrict__ lookback, const bf16* __restrict__ cw, const bf16* __restrict__ cb,
                    bf16* __restrict__ y, bf16* __restrict__ lb_out, int T_, int d) {
  extern __shared__ __align__(16) uint8_t lc_smem[];
  bf16* sh = reinterpret_cast<bf16*>(lc_smem);               // [LC_ROWS][d] normalised rows t0-2 .. t0+LC_TT-1
  const int b = blockIdx.y, t0 = blockIdx.x * LC_TT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < LC_ROWS; r += 8) {
    const int t = t0 - 2 + r;
    bf16* dst = sh + (size_t)r * d;
    if (t >= T_) continue;
    if (t < 0) {                                             // before the sequence: lookback row t+2, or zeros
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (lookback) v = *reinterpret_cast<const uint4*>(lookback + ((int64_t)b * 2 + (t + 2)) * d + i * 256 + lane * 8);
        *reinterpret_cast<uint4*>(dst + i * 256 + lane * 8) = v;
      }
      continue;
    }
    const bf16* xr = x + ((int64_t)b * T_ + t) * d;
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      uint4 raw = *reinterpret_cast<const uint4*>(xr + i * 256 + lane * 8);
      const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) { v[i][k] = __bfloat162float(e[k]); s += v[i][k]; }
    }
    const float mean = warp_sum(s) / (float)d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) { float tt = v[i][k] - mean; q += tt * tt; }
    const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)d + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      uint4 outv;
      bf16* out = reinterpret_cast<bf16*>(&outv);
      const int c0 = i * 256 + lane * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k) out[k] = __float2bfloat16_rn((v[i][k] - mean) * rstd * ldf(lw + c0 + k) + ldf(lb2 + c0 + k));
      *reinterpret_cast<uint4*>(dst + c0) = outv;
      if (lb_out && t >= T_ - 2) *reinterpret_cast<uint4*>(lb_out + ((int64_t)b * 2 + (t - (T_ - 2))) * d + c0) = outv;
    }
  }
  __syncthreads();
  auto ld8 = [&](const bf16* p, float (&o)[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = __bfloat162float(e[k]);
  };
  for (int ch = threadIdx.x; ch < d / 8; ch += 256) {
    const int c0 = ch * 8;
    float wt[24], bb[8], x2[8], x1[8], x0[8];
    {
      const uint4* wp = reinterpret_cast<const uint4*>(cw + c0 * 3);
#pragma unroll
      for (int v3 = 0; v3 < 3; ++v3) {
        uint4 raw = wp[v3];
        const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
        for (int k = 0; k < 8; ++k) wt[8 * v3 + k] = __bfloat162float(e[k]);
      }
    }
    ld8(cb + c0, bb);
    ld8(sh + c0, x2);
    ld8(sh + (size_t)d + c0, x1);
    const int tmax = min(LC_TT, T_ - t0);
    for (int tt = 0; tt < tmax; ++tt) {
      ld8(sh + (size_t)(tt + 2) * d + c0, x0);
      uint4 outv;
      bf16* out = reinterpret_cast<bf16*>(&outv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float acc = wt[3 * k] * x2[k];
        acc = fmaf(wt[3 * k + 1], x1[k], acc);
        acc = fmaf(wt[3 * k + 2], x0[k], acc);
        out[k] = __float2bfloat16_rn(acc + bb[k]);
        x2[k] = x1[k];
        x1[k] = x0[k];
      }
      *reinterpret_cast<uint4*>(y + ((int64_t)b * T_ + t0 + tt) * d + c0) = outv;
    }
  }
}

extern "C" int kch_layernorm_short_conv(const void* x, const void* ln_weight, const void* ln_bias, float eps,
                                        const void* lookback, const void* conv_weight, const void* conv_bias, void* y,
                                        void* lookback_out, int B, int T, int d, int dtype, int wdtype, void* stream) {
  KCH_REQUIRE(dtype == KCH_BF16 && (d % 256) == 0 && d >= 256 && d <= 2048,
              "kch_layernorm_short_conv: bf16 with d %% 256 == 0 and d <= 2048 only (dtype tag %d, d=%d)", dtype, d);
  KCH_REQUIRE(B >= 1 && T >= 2, "kch_layernorm_short_conv: B=%d T=%d (needs T >= 2)", B, T);
  const uintptr_t al = (uintptr_t)x | (uintptr_t)y | (uintptr_t)conv_weight | (uintptr_t)conv_bias | (uintptr_t)lookback |
                       (uintptr_t)lookback_out;
  KCH_REQUIRE((al & 15) == 0, "kch_layernorm_short_conv: operands must be 16-byte aligned");
  const size_t smem = (size_t)LC_ROWS * d * 2;
  dim3 grid((unsigned)((T + LC_TT - 1) / LC_TT), B);
  cudaStream_t s = kch_stream(stream);
#define LCV(NV)                                                                                                   \
  KCH_DISPATCH_FLOAT(wdtype, TW, {                                                                                 \
    KCH_CUDA_OK(cudaFuncSetAttribute(ln_conv_kernel_bf16<TW, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    ln_conv_kernel_bf16<TW, NV><<<grid, 256, smem, s>>>((const bf16*)x, (const TW*)ln_weight, (const TW*)ln_bias, eps, \
        (const bf16*)lookback, (const bf16*)conv_weight, (const bf16*)conv_bias, (bf16*)y, (bf16*)lookback_out, T, d); \
  })
  switch (d / 256) {
    case 1: LCV(1); break; case 2: LCV(2); break; case 3: LCV(3); break; case 4: LCV(4); break;
    case 5: LCV(5); break; case 6: LCV(6); break; case 7: LCV(7); break; default: LCV(8); break;
  }
#undef LCV
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// One-token step of the conv with the lookback [B,2,d] updated where it lies (ops_fused.py:560-569 builds
// the new lookback by concatenation; here the same two rows are written back by the thread that read them).
extern "C" int kch_short_conv_step(const void* x, void* lookback, const void* weight, const void* bias, void* y,
                                   int B, int d, int dtype, void* stream) {
  KCH_REQUIRE(B >= 1 && d >= 1 && x && lookback && y, "kch_short_conv_step: B=%d d=%d", B, d);
  int64_t total = (int64_t)B * d;
  const uintptr_t al = (uintptr_t)x | (uintptr_t)y | (uintptr_t)weight | (uintptr_t)bias | (uintptr_t)lookback;
  if (dtype == KCH_BF16 && (d % 8) == 0 && (al & 15) == 0) {
    dim3 grid((unsigned)ceil_div64(total / 8, 256)), block(256);
    short_conv_kernel_bf16x8<<<grid, block, 0, kch_stream(stream)>>>((const bf16*)x, (const bf16*)lookback,
                                                                    (const bf16*)weight, (const bf16*)bias, (bf16*)y, B, 1, d,
                                                                    (bf16*)lookback);
  } else {
    dim3 grid((unsigned)ceil_div64(total, 256)), block(256);
    KCH_DISPATCH_FLOAT(dtype, T_, (short_conv_kernel<T_><<<grid, block, 0, kch_stream(stream)>>>(
        (const T_*)x, (const T_*)lookback, (const T_*)weight, (const T_*)bias, (T_*)y, B, 1, d, (T_*)lookback)));
  }
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// LayerNorm + one-token conv step in one launch (the decode step of a KDA sub-layer: ops_fused.py:52-60 then
// :560-569): one CTA per batch row normalises it in registers (8 channels per thread), convolves with the two lookback rows of its own
// channels and slides the lookback where it lies.  Same arithmetic and rounding points as kch_layernorm followed by
// kch_short_conv_step (the normalised row is rounded to bf16 before the taps see it).
template <typename TW>
__global__ void __launch_bounds__(256)
ln_conv_step_kernel_bf16(const bf16* __restrict__ x, const TW* __restrict__ lw, const TW* __restrict__ lb2, float eps,
                         bf16* lookback, const bf16* __restrict__ cw, const bf16* __restrict__ cb,
                         bf16* __restrict__ y, int d) {
  __shared__ float red[8];
  const int c0 = threadIdx.x * 8;
  const bool on = c0 < d;
  const int64_t row = blockIdx.x;
  bf16* l0 = lookback + row * 2 * d;
  bf16* l1 = l0 + d;
  float v[8], wv[8], bv[8];
  uint4 r2 = make_uint4(0u, 0u, 0u, 0u), r1 = r2, cbv = r2, cwv[3] = {r2, r2, r2};
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = wv[k] = bv[k] = 0.f;
  if (on) {
    ld8p(x + row * d + c0, v); ld8p(lw + c0, wv); ld8p(lb2 + c0, bv);
    r2 = *reinterpret_cast<const uint4*>(l0 + c0);
    r1 = *reinterpret_cast<const uint4*>(l1 + c0);
    cbv = *reinterpret_cast<const uint4*>(cb + c0);
    const uint4* wp = reinterpret_cast<const uint4*>(cw + c0 * 3);   // taps of 8 channels: 24 consecutive bf16
    cwv[0] = wp[0]; cwv[1] = wp[1]; cwv[2] = wp[2];
  }
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += v[k];
  const float mean = block_sum_256(s, red) / (float)d;
  float q = 0.f;
  if (on) {
#pragma unroll
    for (int k = 0; k < 8; ++k) { const float t = v[k] - mean; q += t * t; }
  }
  const float rstd = 1.0f / sqrtf(block_sum_256(q, red) / (float)d + eps);
  if (!on) return;
  uint4 nv, outv;
  bf16* xn = reinterpret_cast<bf16*>(&nv);
  bf16* out = reinterpret_cast<bf16*>(&outv);
  const bf16* wt = reinterpret_cast<const bf16*>(cwv);
  const bf16* e2 = reinterpret_cast<const bf16*>(&r2);
  const bf16* e1 = reinterpret_cast<const bf16*>(&r1);
  const bf16* eb = reinterpret_cast<const bf16*>(&cbv);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    xn[k] = __float2bfloat16_rn((v[k] - mean) * rstd * wv[k] + bv[k]);
    float acc = __bfloat162float(wt[3 * k]) * __bfloat162float(e2[k]);
    acc = fmaf(__bfloat162float(wt[3 * k + 1]), __bfloat162float(e1[k]), acc);
    acc = fmaf(__bfloat162float(wt[3 * k + 2]), __bfloat162float(xn[k]), acc);
    out[k] = __float2bfloat16_rn(acc + __bfloat162float(eb[k]));
  }
  *reinterpret_cast<uint4*>(y + row * d + c0) = outv;
  *reinterpret_cast<uint4*>(l0 + c0) = r1;
  *reinterpret_cast<uint4*>(l1 + c0) = nv;
}

extern "C" int kch_layernorm_short_conv_step(const void* x, const void* ln_weight, const void* ln_bias, float eps,
                                             void* lookback, const void* conv_weight, const void* conv_bias, void* y,
                                             int B, int d, int dtype, int wdtype, void* stream) {
  KCH_REQUIRE(dtype == KCH_BF16 && (d % 256) == 0 && d >= 256 && d <= 2048,
              "kch_layernorm_short_conv_step: bf16 with d %% 256 == 0 and d <= 2048 only (dtype tag %d, d=%d)", dtype, d);
  KCH_REQUIRE(B >= 1 && x && lookback && y, "kch_layernorm_short_conv_step: B=%d", B);
  const uintptr_t al = (uintptr_t)x | (uintptr_t)y | (uintptr_t)conv_weight | (uintptr_t)conv_bias | (uintptr_t)lookback;
  KCH_REQUIRE((al & 15) == 0, "kch_layernorm_short_conv_step: operands must be 16-byte aligned");
  KCH_REQUIRE(((((uintptr_t)ln_weight) | ((uintptr_t)ln_bias)) & 15) == 0,
              "kch_layernorm_short_conv_step: LayerNorm parameters must be 16-byte aligned");
  cudaStream_t s = kch_stream(stream);
  KCH_DISPATCH_FLOAT(wdtype, TW, (ln_conv_step_kernel_bf16<TW><<<(unsigned)B, 256, 0, s>>>(
      (const bf16*)x, (const TW*)ln_weight, (const TW*)ln_bias, eps, (bf16*)lookback, (const bf16*)conv_weight,
      (const bf16*)conv_bias, (bf16*)y, d)));
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// ---------------------------------------------------------------------------------------
// Activations applied to a projection output that is already stored in dtype T, reproducing
// the reference's rounding points: each op reads T, computes in fp32, rounds to T.
//   KCH_ACT_SILU            y = x*sigmoid(x)
//   KCH_ACT_SIGMOID         y = sigmoid(x)
//   KCH_ACT_NEG_SOFTPLUS    y = round(-round(softplus(x)) * param)       (KDA gate)
//   KCH_ACT_SILU_L2NORM     y = round(s / max(round(||s||), eps)), s = round(silu(x)), per
//                           group of `group` consecutive columns         (KDA q,k)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void act_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols, int64_t ldx,
                           int64_t ldy, int act, float param) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  int64_t r = i / cols;
  int cidx = (int)(i % cols);
  float v = ldf(x + r * ldx + cidx);
  float o;
  if (act == KCH_ACT_SILU) o = silu_f(v);
  else if (act == KCH_ACT_SIGMOID) o = sigmoid_f(v);
  else o = -round_to<T>(softplus_f(v)) * param;
  stf(y + r * ldy + cidx, o);
}

// bf16 fast path: 8 consecutive columns (16 bytes) per thread
__global__ void act_kernel_bf16x8(const bf16* __restrict__ x, bf16* __restrict__ y, int64_t rows, int cols8,
                                  int64_t ldx, int64_t ldy, int act, float param) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols8) return;
  int64_t r = i / cols8;
  int c8 = (int)(i % cols8) * 8;
  uint4 raw = *reinterpret_cast<const uint4*>(x + r * ldx + c8);
  const bf16* in = reinterpret_cast<const bf16*>(&raw);
  uint4 outv;
  bf16* out = reinterpret_cast<bf16*>(&outv);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float v = __bfloat162float(in[e]), o;
    if (act == KCH_ACT_SILU) o = silu_f(v);
    else if (act == KCH_ACT_SIGMOID) o = sigmoid_f(v);
    else o = -round_to<bf16>(softplus_f(v)) * param;
    out[e] = __float2bfloat16_rn(o);
  }
  *reinterpret_cast<uint4*>(y + r * ldy + c8) = outv;
}

// bf16 fast path of silu + L2 norm for groups of 128 columns: one warp per (row, group), 4 columns per lane
__global__ void silu_l2norm_kernel_bf16_g128(const bf16* __restrict__ x, bf16* __restrict__ y, int64_t rows,
                                             int gpr, int64_t ldx, int64_t ldy) {
  int64_t gidx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (gidx >= rows * gpr) return;
  int64_t r = gidx / gpr;
  int g0 = (int)(gidx % gpr) * 128 + lane * 4;
  uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + g0);
  const bf16* in = reinterpret_cast<const bf16*>(&raw);
  float s[4], ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) { s[e] = round_to<bf16>(silu_f(__bfloat162float(in[e]))); ss += s[e] * s[e]; }
  float nrm = fmaxf(round_to<bf16>(sqrtf(warp_sum(ss))), 1e-12f);
  uint2 outv;
  bf16* out = reinterpret_cast<bf16*>(&outv);
#pragma unroll
  for (int e = 0; e < 4; ++e) out[e] = __float2bfloat16_rn(s[e] / nrm);
  *reinterpret_cast<uint2*>(y + r * ldy + g0) = outv;
}

// one warp per (row, group)
template <typename T>
__global__ void silu_l2norm_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols,
                                   int64_t ldx, int64_t ldy, int group) {
  int64_t gidx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  int gpr = cols / group;
  if (gidx >= rows * gpr) return;
  int64_t r = gidx / gpr;
  int g0 = (int)(gidx % gpr) * group;
  const T* xr = x + r * ldx + g0;
  T* yr = y + r * ldy + g0;
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) {
    float s = round_to<T>(silu_f(ldf(xr + i)));
    ss += s * s;
  }
  float nrm = fmaxf(round_to<T>(sqrtf(warp_sum(ss))), 1e-12f);
  for (int i = lane; i < group; i += 32) {
    float s = round_to<T>(silu_f(ldf(xr + i)));
    stf(yr + i, s / nrm);
  }
}

extern "C" int kch_activation(const void* x, void* y, int64_t rows, int cols, int act, float param,
                              int group, int dtype, int64_t ldx, int64_t ldy, void* stream) {
  KCH_REQUIRE(rows >= 0 && cols >= 1, "kch_activation: rows=%lld cols=%d", (long long)rows, cols);
  KCH_REQUIRE(ldx >= cols && ldy >= cols, "kch_activation: ldx=%lld ldy=%lld < cols=%d", (long long)ldx,
              (long long)ldy, cols);
  int64_t n = rows * cols;
  if (n == 0) return KCH_OK;
  if (act == KCH_ACT_SILU_L2NORM) {
    KCH_REQUIRE(group >= 1 && cols % group == 0, "kch_activation: group=%d must divide cols=%d", group, cols);
    int64_t ng = n / group;
    dim3 grid((unsigned)ceil_div64(ng, 8)), block(256);
    if (dtype == KCH_BF16 && group == 128 && (ldx % 4) == 0 && (ldy % 4) == 0 && (((uintptr_t)x | (uintptr_t)y) & 7) == 0) {
      silu_l2norm_kernel_bf16_g128<<<grid, block, 0, kch_stream(stream)>>>((const bf16*)x, (bf16*)y, rows, cols / 128,
                                                                          ldx, ldy);
    } else {
      KCH_DISPATCH_FLOAT(dtype, T, (silu_l2norm_kernel<T><<<grid, block, 0, kch_stream(stream)>>>(
          (const T*)x, (T*)y, rows, cols, ldx, ldy, group)));
    }
  } else {
    KCH_REQUIRE(act == KCH_ACT_SILU || act == KCH_ACT_SIGMOID || act == KCH_ACT_NEG_SOFTPLUS,
                "kch_activation: unknown act %d", act);
    if (dtype == KCH_BF16 && (cols % 8) == 0 && (ldx % 8) == 0 && (ldy % 8) == 0 &&
        (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
      dim3 grid((unsigned)ceil_div64(n / 8, 256)), block(256);
      act_kernel_bf16x8<<<grid, block, 0, kch_stream(stream)>>>((const bf16*)x, (bf16*)y, rows, cols / 8, ldx, ldy,
                                                               act, param);
    } else {
      dim3 grid((unsigned)ceil_div64(n, 256)), block(256);
      KCH_DISPATCH_FLOAT(dtype, T, (act_kernel<T><<<grid, block, 0, kch_stream(stream)>>>(
          (const T*)x, (T*)y, rows, cols, ldx, ldy, act, param)));
    }
  }
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// ---------------------------------------------------------------------------------------
// L2 row normalisation into fp32:  y = fp32(x) / max(||fp32(x)||, 1e-12)   (F.normalize).
// Input rows may be strided (ld elements between rows); one warp per row.
// `norms` (optional) receives max(||x||,eps) per row; `y` may be null when only norms are wanted.
// ---------------------------------------------------------------------------------------
template <typename T, typename TO>
__global__ void rownorm_kernel(const T* __restrict__ x, int64_t ld, TO* __restrict__ y,
                               float* __restrict__ norms, int64_t rows, int c) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * ld;
  float ss = 0.f;
  for (int i = lane; i < c; i += 32) {
    float v = ldf(xr + i);
    ss += v * v;
  }
  float nrm = fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
  if (norms && lane == 0) norms[row] = nrm;
  if (y)
    for (int i = lane; i < c; i += 32) stf(y + row * c + i, ldf(xr + i) / nrm);
}

extern "C" int kch_rownorm(const void* x, int64_t ld, void* y, float* norms, int64_t rows, int c,
                           int dtype, int out_dtype, void* stream) {
  KCH_REQUIRE(rows >= 0 && c >= 1 && ld >= c, "kch_rownorm: rows=%lld c=%d ld=%lld", (long long)rows, c,
              (long long)ld);
  if (rows == 0) return KCH_OK;
  dim3 grid((unsigned)ceil_div64(rows, 8)), block(256);
  KCH_DISPATCH_FLOAT(dtype, T, KCH_DISPATCH_FLOAT(out_dtype, TO,
      (rownorm_kernel<T, TO><<<grid, block, 0, kch_stream(stream)>>>((const T*)x, ld, (TO*)y, norms, rows, c))));
  KCH_LAUNCH_OK();
  return KCH_OK;
}
