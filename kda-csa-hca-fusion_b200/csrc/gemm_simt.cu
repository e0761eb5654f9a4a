// Linear layer  C[M,N] = A[M,K] . W[N,K]^T  (nn.Linear weight layout), fp32 accumulation,
// result rounded once to the storage type, optional residual add (in fp32, rounded once more, which
// is what `residual + o_proj(o)` does on stored tensors).
//
// This file holds the CUDA-core version: any shape, any leading dimensions, fp32 or bf16.  It
// serves fp32 inputs and shapes the tensor-core kernel does not take (see gemm_tcgen05.cu).
#include "kch_common.cuh"

#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, T* __restrict__ C,
                 const T* __restrict__ R, int64_t M, int N, int K, int64_t lda, int64_t ldw,
                 int64_t ldc, int64_t ldr) {
  __shared__ float sa[SG_BK][SG_BM + 1];
  __shared__ float sw[SG_BK][SG_BN + 1];
  const int64_t m0 = (int64_t)blockIdx.x * SG_BM;
  const int n0 = blockIdx.y * SG_BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += SG_BK) {
    for (int idx = threadIdx.x; idx < SG_BM * SG_BK; idx += 256) {
      int r = idx / SG_BK, kk = idx % SG_BK;
      int64_t mm = m0 + r;
      sa[kk][r] = (mm < M && k0 + kk < K) ? ldf(A + mm * lda + k0 + kk) : 0.f;
    }
    for (int idx = threadIdx.x; idx < SG_BN * SG_BK; idx += 256) {
      int r = idx / SG_BK, kk = idx % SG_BK;
      int nn = n0 + r;
      sw[kk][r] = (nn < N && k0 + kk < K) ? ldf(W + (int64_t)nn * ldw + k0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SG_BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sa[kk][ty * 4 + i]; w[i] = sw[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t mm = m0 + ty * 4 + i;
    if (mm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int nn = n0 + tx * 4 + j;
      if (nn >= N) continue;
      float v = round_to<T>(acc[i][j]);
      if (R) v += ldf(R + mm * ldr + nn);
      stf(C + mm * ldc + nn, v);
    }
  }
}

int kch_linear_simt(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K,
                    int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype, void* stream) {
  if (M == 0 || N == 0) return KCH_OK;
  dim3 grid((unsigned)ceil_div64(M, SG_BM), (N + SG_BN - 1) / SG_BN), block(256);
  KCH_DISPATCH_FLOAT(dtype, T, (gemm_simt_kernel<T><<<grid, block, 0, kch_stream(stream)>>>(
      (const T*)A, (const T*)W, (T*)C, (const T*)residual, M, N, K, lda, ldw, ldc, ldr)));
  KCH_LAUNCH_OK();
  return KCH_OK;
}
