// Shared device/host helpers for the kch_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kch_b200.h"

// ---- error reporting -----------------------------------------------------------------
void kch_set_error(const char* fmt, ...);
void kch_note_launch(int n);   // host-side count of kernels launched by this library

#define KCH_REQUIRE(cond, ...)            \
  do {                                    \
    if (!(cond)) {                        \
      kch_set_error(__VA_ARGS__);         \
      return KCH_ERR_INVALID;             \
    }                                     \
  } while (0)

#define KCH_CUDA_OK(expr)                                                        \
  do {                                                                           \
    cudaError_t _e = (expr);                                                     \
    if (_e != cudaSuccess) {                                                     \
      kch_set_error("%s failed: %s", #expr, cudaGetErrorString(_e));             \
      return KCH_ERR_CUDA;                                                       \
    }                                                                            \
  } while (0)

#define KCH_LAUNCH_OK()                                                          \
  do {                                                                           \
    kch_note_launch(1);                                                          \
    cudaError_t _e = cudaGetLastError();                                         \
    if (_e != cudaSuccess) {                                                     \
      kch_set_error("kernel launch failed at %s:%d: %s", __FILE__, __LINE__,     \
                    cudaGetErrorString(_e));                                     \
      return KCH_ERR_CUDA;                                                       \
    }                                                                            \
  } while (0)

static inline cudaStream_t kch_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- typed loads / stores ---------------------------------------------------------------
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// round a float through the storage type T (identity for float)
template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ float round_to<bf16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// generic load by runtime dtype tag (slow path helpers)
__device__ __forceinline__ float ld_any(const void* p, int64_t i, int dtype) {
  return dtype == KCH_BF16 ? __bfloat162float(((const bf16*)p)[i]) : ((const float*)p)[i];
}

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

#define KCH_DISPATCH_FLOAT(dtype, T, ...)                       \
  do {                                                          \
    if ((dtype) == KCH_F32) {                                   \
      typedef float T;                                          \
      __VA_ARGS__;                                              \
    } else if ((dtype) == KCH_BF16) {                           \
      typedef bf16 T;                                           \
      __VA_ARGS__;                                              \
    } else {                                                    \
      kch_set_error("unsupported dtype tag %d", (int)(dtype));  \
      return KCH_ERR_INVALID;                                   \
    }                                                           \
  } while (0)
