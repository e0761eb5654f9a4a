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

extern "C" int kch_layernorm(const void* x, const void* weight, const void* bias, void* y,
                             int64_t rows, int d, float eps, int dtype, int wdtype, void* stream) {
  KCH_REQUIRE(rows >= 0 && d >= 1, "kch_layernorm: rows=%lld d=%d", (long long)rows, d);
  if (rows == 0) return KCH_OK;
  const int wpb = 8;
  dim3 grid((unsigned)ceil_div64(rows, wpb)), block(wpb * 32);
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
__global__ void short_conv_kernel(const T* __restrict__ x, const T* __restrict__ lb,
                                  const T* __restrict__ w, const T* __restrict__ bias,
                                  T* __restrict__ y, int B, int T_, int d) {
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
}

extern "C" int kch_short_conv(const void* x, const void* lookback, const void* weight,
                              const void* bias, void* y, int B, int T, int d, int dtype,
                              void* stream) {
  KCH_REQUIRE(B >= 0 && T >= 0 && d >= 1, "kch_short_conv: B=%d T=%d d=%d", B, T, d);
  int64_t total = (int64_t)B * T * d;
  if (total == 0) return KCH_OK;
  dim3 grid((unsigned)ceil_div64(total, 256)), block(256);
  KCH_DISPATCH_FLOAT(dtype, T_, (short_conv_kernel<T_><<<grid, block, 0, kch_stream(stream)>>>(
      (const T_*)x, (const T_*)lookback, (const T_*)weight, (const T_*)bias, (T_*)y, B, T, d)));
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
    KCH_DISPATCH_FLOAT(dtype, T, (silu_l2norm_kernel<T><<<grid, block, 0, kch_stream(stream)>>>(
        (const T*)x, (T*)y, rows, cols, ldx, ldy, group)));
  } else {
    KCH_REQUIRE(act == KCH_ACT_SILU || act == KCH_ACT_SIGMOID || act == KCH_ACT_NEG_SOFTPLUS,
                "kch_activation: unknown act %d", act);
    dim3 grid((unsigned)ceil_div64(n, 256)), block(256);
    KCH_DISPATCH_FLOAT(dtype, T, (act_kernel<T><<<grid, block, 0, kch_stream(stream)>>>(
        (const T*)x, (T*)y, rows, cols, ldx, ldy, act, param)));
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
