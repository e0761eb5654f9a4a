// Decode-time cache maintenance for the CSA / HCA layers
// (CSADecodingCache.append_step, ops_decoding_cache.py:631-779; HCADecodingCache.append_step, 1200-1264).
//
// One fused kernel per appended token: stash the token's projections in the partial-block
// accumulator, push the L2-normalised key into the sliding-window ring, and, when the token closes a
// block of m tokens, compress the block (with the previous block's b-branch for CSA), round the new
// row to the cache dtype exactly as the reference does (ops_decoding_cache.py:754-762), optionally
// re-encode it as block-scaled e4m3 / int8 (one fp32 scale per 64 elements), and record the fp32 norm
// of the stored row so that attention can use  row / max(||row||, eps)  without a second pass.
// HBM traffic per token and sequence: the token's projections once, the accumulator once when a block
// closes, one output row.
#include <math.h>

#include "kch_common.cuh"

unsigned int* kch_status_device_ptr();   // device address of the library's status word

struct AppendArgs {
  const void *Ca, *Cb, *Za, *Zb, *Ki, *Zi;   // new token rows, row b at element offset b*ld
  int64_t ld_c, ld_i;
  void *accCa, *accCb, *accZa, *accZb, *accKi, *accZi;   // [B,m,c] / [B,m,cI]
  void *prevCb, *prevZb;                                 // [B,m,c]
  int has_prev;
  const void *Ba, *Bb, *Bi;                              // [m,c], [m,c], [m,cI]
  void* comp; float* comp_scales; float* comp_norms;     // [B,cap,c] (+ [B,cap,c/64], [B,cap])
  int comp_kind;                                         // KCH_F32 / KCH_BF16 / KCH_FP8_E4M3 / KCH_INT8
  void* kcomp; float* kcomp_norms;                       // [B,cap,cI] stored indexer keys, [B,cap] their fp32 norms
  int64_t cap; int n_blocks;
  void* ring; int ring_pos; int win;
  int acc_len, m, c, cI, normalize, overlap;
  const int32_t* counters;                               // device-resident {acc_len, n_blocks, ring_n, has_prev, ...} or null
  unsigned int* status;
  int advance;                                           // 1: the last CTA to finish advances the device counters
  int n_ctas;
};

template <typename T>
__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

// With `advance` set the CTA that finishes last advances the device counters (every CTA read them when it started,
// so nobody can see the new values too early) -- the separate one-thread kernel of kch_cache_advance folded in.
__device__ __forceinline__ void cache_append_finish(const AppendArgs& a) {
  if (!a.advance || !a.counters) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t* ctr = const_cast<int32_t*>(a.counters);
    __threadfence();
    if (atomicAdd(&ctr[KCH_CTR_ARRIVALS], 1) == a.n_ctas - 1) {
      ctr[KCH_CTR_ARRIVALS] = 0;
      int acc = ctr[KCH_CTR_ACC_LEN] + 1;
      ctr[KCH_CTR_RING_N] += 1;
      ctr[KCH_CTR_TOKENS] += 1;
      if (acc >= a.m) {
        acc = 0;
        ctr[KCH_CTR_N_BLOCKS] += 1;
        ctr[KCH_CTR_HAS_PREV] = 1;
      }
      ctr[KCH_CTR_ACC_LEN] = acc;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) cache_append_kernel(AppendArgs a) {
  extern __shared__ float srow[];   // [c] compressed row, then [cI]
  __shared__ float red[4];
  const int b = blockIdx.x, tid = threadIdx.x;
  if (a.counters) {   // the step is replayed from a CUDA graph: the counters live on the device
    a.acc_len = a.counters[KCH_CTR_ACC_LEN];
    a.n_blocks = a.counters[KCH_CTR_N_BLOCKS];
    a.ring_pos = a.win > 0 ? a.counters[KCH_CTR_RING_N] % a.win : 0;
    a.has_prev = a.counters[KCH_CTR_HAS_PREV];
    if (a.acc_len < 0 || a.acc_len >= a.m || (a.acc_len + 1 == a.m && (a.n_blocks >= a.cap || !a.comp))) {
      if (tid == 0) atomicCAS(a.status, 0u, (unsigned)KCH_STATUS_CACHE_CAPACITY);
      cache_append_finish(a);
      return;
    }
  }
  const int c = a.c, cI = a.cI, m = a.m, slot = a.acc_len;
  const int64_t accoff = ((int64_t)b * m + slot) * c;
  // 1. stash the token
  float ss = 0.f;
  for (int d = tid; d < c; d += 128) {
    T ca = ((const T*)a.Ca)[b * a.ld_c + d];
    ((T*)a.accCa)[accoff + d] = ca;
    ((T*)a.accZa)[accoff + d] = ((const T*)a.Za)[b * a.ld_c + d];
    if (a.overlap) {
      ((T*)a.accCb)[accoff + d] = ((const T*)a.Cb)[b * a.ld_c + d];
      ((T*)a.accZb)[accoff + d] = ((const T*)a.Zb)[b * a.ld_c + d];
    }
    float f = ldf(&ca);
    ss += f * f;
  }
  if (a.Ki)
    for (int d = tid; d < cI; d += 128) {
      ((T*)a.accKi)[((int64_t)b * m + slot) * cI + d] = ((const T*)a.Ki)[b * a.ld_i + d];
      ((T*)a.accZi)[((int64_t)b * m + slot) * cI + d] = ((const T*)a.Zi)[b * a.ld_i + d];
    }
  // 2. window ring
  if (a.ring) {
    float nrm = 1.f;
    if (a.normalize) nrm = fmaxf(sqrtf(block_sum_128<T>(ss, red)), 1e-12f);
    for (int d = tid; d < c; d += 128)
      stf((T*)a.ring + ((int64_t)b * a.win + a.ring_pos) * c + d, ldf((const T*)a.Ca + b * a.ld_c + d) / nrm);
  }
  if (slot + 1 < m) { cache_append_finish(a); return; }
  __syncthreads();  // the accumulator rows written above are read below by other threads? no: same channel
  // 3. the block is complete: compress channel-wise
  const int64_t blk = (int64_t)b * m * c;
  float nsq = 0.f;
  for (int d = tid; d < c; d += 128) {
    float mx = -INFINITY;
    for (int j = 0; j < m; ++j)
      mx = fmaxf(mx, ldf((const T*)a.accZa + blk + (int64_t)j * c + d) + ldf((const T*)a.Ba + j * c + d));
    const bool ov = a.overlap && a.has_prev;
    if (ov)
      for (int j = 0; j < m; ++j)
        mx = fmaxf(mx, ldf((const T*)a.prevZb + blk + (int64_t)j * c + d) + ldf((const T*)a.Bb + j * c + d));
    float den = 0.f, acc = 0.f, accb = 0.f;
    for (int j = 0; j < m; ++j) {
      float e = expf(ldf((const T*)a.accZa + blk + (int64_t)j * c + d) + ldf((const T*)a.Ba + j * c + d) - mx);
      den += e;
      acc = fmaf(e, ldf((const T*)a.accCa + blk + (int64_t)j * c + d), acc);
    }
    if (ov)
      for (int j = 0; j < m; ++j) {
        float e = expf(ldf((const T*)a.prevZb + blk + (int64_t)j * c + d) + ldf((const T*)a.Bb + j * c + d) - mx);
        den += e;
        accb = fmaf(e, ldf((const T*)a.prevCb + blk + (int64_t)j * c + d), accb);
      }
    float r = round_to<T>(acc / den + accb / den);   // the cache stores rows in its own dtype
    srow[d] = r;
  }
  __syncthreads();
  const int64_t orow = (int64_t)b * a.cap + a.n_blocks;
  if (a.comp_kind == KCH_FP8_E4M3 || a.comp_kind == KCH_INT8) {
    // per 64-element block: scale = max|x| / qmax (1 for an all-zero block)
    const float qmax = a.comp_kind == KCH_FP8_E4M3 ? 448.f : 127.f;
    for (int blk64 = tid >> 5; blk64 < c / 64; blk64 += 4) {
      int lane = tid & 31;
      float v0 = srow[blk64 * 64 + lane], v1 = srow[blk64 * 64 + 32 + lane];
      float am = warp_max(fmaxf(fabsf(v0), fabsf(v1)));
      float sc = am > 0.f ? am / qmax : 1.f;
      if (lane == 0) a.comp_scales[orow * (c / 64) + blk64] = sc;
      float q0, q1;
      if (a.comp_kind == KCH_FP8_E4M3) {
        __nv_fp8_e4m3 p0(v0 / sc), p1(v1 / sc);
        ((__nv_fp8_e4m3*)a.comp)[orow * c + blk64 * 64 + lane] = p0;
        ((__nv_fp8_e4m3*)a.comp)[orow * c + blk64 * 64 + 32 + lane] = p1;
        q0 = float(p0) * sc; q1 = float(p1) * sc;
      } else {
        float r0 = fminf(fmaxf(rintf(v0 / sc), -127.f), 127.f), r1 = fminf(fmaxf(rintf(v1 / sc), -127.f), 127.f);
        ((int8_t*)a.comp)[orow * c + blk64 * 64 + lane] = (int8_t)r0;
        ((int8_t*)a.comp)[orow * c + blk64 * 64 + 32 + lane] = (int8_t)r1;
        q0 = r0 * sc; q1 = r1 * sc;
      }
      srow[blk64 * 64 + lane] = q0;
      srow[blk64 * 64 + 32 + lane] = q1;
    }
    __syncthreads();
    for (int d = tid; d < c; d += 128) nsq += srow[d] * srow[d];
  } else {
    for (int d = tid; d < c; d += 128) {
      float r = srow[d];
      if (a.comp_kind == KCH_BF16) ((bf16*)a.comp)[orow * c + d] = __float2bfloat16_rn(r);
      else ((float*)a.comp)[orow * c + d] = r;
      nsq += r * r;
    }
  }
  float nrm = fmaxf(sqrtf(block_sum_128<T>(nsq, red)), 1e-12f);
  if (tid == 0) a.comp_norms[orow] = nrm;
  // 4. indexer key of the block (single branch) and the fp32 norm of the stored key
  if (a.Ki) {
    __syncthreads();
    const int64_t blki = (int64_t)b * m * cI;
    float isq = 0.f;
    for (int d = tid; d < cI; d += 128) {
      float mx = -INFINITY;
      for (int j = 0; j < m; ++j)
        mx = fmaxf(mx, ldf((const T*)a.accZi + blki + (int64_t)j * cI + d) + ldf((const T*)a.Bi + j * cI + d));
      float den = 0.f, acc = 0.f;
      for (int j = 0; j < m; ++j) {
        float e = expf(ldf((const T*)a.accZi + blki + (int64_t)j * cI + d) + ldf((const T*)a.Bi + j * cI + d) - mx);
        den += e;
        acc = fmaf(e, ldf((const T*)a.accKi + blki + (int64_t)j * cI + d), acc);
      }
      float r = round_to<T>(acc / den);
      srow[d] = r;
      stf((T*)a.kcomp + orow * cI + d, r);
      isq += r * r;
    }
    float inrm = fmaxf(sqrtf(block_sum_128<T>(isq, red)), 1e-12f);
    if (tid == 0) a.kcomp_norms[orow] = inrm;
  }
  // 5. this block's b-branch becomes the overlap partner of the next block
  if (a.overlap) {
    for (int idx = tid; idx < m * c; idx += 128) {
      ((T*)a.prevCb)[blk + idx] = ((const T*)a.accCb)[blk + idx];
      ((T*)a.prevZb)[blk + idx] = ((const T*)a.accZb)[blk + idx];
    }
  }
  cache_append_finish(a);
}

static int cache_append_launch(const kch_cache_append_args* p, void* stream, int advance);

extern "C" int kch_cache_append_token(const kch_cache_append_args* p, void* stream) {
  return cache_append_launch(p, stream, 0);
}

extern "C" int kch_cache_append_token_advance(const kch_cache_append_args* p, void* stream) {
  KCH_REQUIRE(p != nullptr && p->counters != nullptr, "kch_cache_append_token_advance: needs device counters");
  return cache_append_launch(p, stream, 1);
}

static int cache_append_launch(const kch_cache_append_args* p, void* stream, int advance) {
  KCH_REQUIRE(p != nullptr, "kch_cache_append_token: null args");
  KCH_REQUIRE(p->B >= 1, "B=%d must be >= 1", p->B);
  KCH_REQUIRE(p->c >= 1, "c=%d must be >= 1", p->c);
  KCH_REQUIRE(p->m >= 1, "m=%d must be >= 1", p->m);
  KCH_REQUIRE(p->counters || (p->acc_len >= 0 && p->acc_len < p->m), "acc_len=%d out of range for m=%d", p->acc_len, p->m);
  KCH_REQUIRE(p->dtype == KCH_F32 || p->dtype == KCH_BF16, "cache dtype tag %d unsupported", p->dtype);
  // with device counters the host cannot know whether this token closes a block: require the storage up front
  const bool closes = p->counters ? true : p->acc_len + 1 == p->m;
  if (p->comp_kind == KCH_FP8_E4M3 || p->comp_kind == KCH_INT8)
    KCH_REQUIRE(p->c % 64 == 0 && (!closes || p->comp_scales),
                "block-scaled 8-bit rows need c %% 64 == 0 (c=%d) and a scale buffer", p->c);
  else
    KCH_REQUIRE(p->comp_kind == p->dtype, "comp_kind=%d must equal the cache dtype or be an 8-bit kind", p->comp_kind);
  if (closes)
    KCH_REQUIRE(p->comp && p->comp_norms && (p->counters || p->n_blocks < p->capacity),
                "compressed-row capacity %lld exhausted", (long long)p->capacity);
  if (closes && p->K_idx) KCH_REQUIRE(p->kcomp && p->kcomp_norms, "kch_cache_append_token: indexer key storage missing");
  AppendArgs a;
  a.Ca = p->Ca; a.Cb = p->Cb; a.Za = p->Za; a.Zb = p->Zb; a.Ki = p->K_idx; a.Zi = p->Z_idx;
  a.ld_c = p->ld_c; a.ld_i = p->ld_i;
  a.accCa = p->acc_Ca; a.accCb = p->acc_Cb; a.accZa = p->acc_Za; a.accZb = p->acc_Zb; a.accKi = p->acc_K_idx; a.accZi = p->acc_Z_idx;
  a.prevCb = p->prev_Cb; a.prevZb = p->prev_Zb; a.has_prev = p->has_prev;
  a.Ba = p->Ba; a.Bb = p->Bb; a.Bi = p->B_idx;
  a.comp = p->comp; a.comp_scales = p->comp_scales; a.comp_norms = p->comp_norms; a.comp_kind = p->comp_kind;
  a.kcomp = p->kcomp; a.kcomp_norms = p->kcomp_norms; a.cap = p->capacity; a.n_blocks = p->n_blocks;
  a.counters = p->counters; a.status = kch_status_device_ptr();
  a.ring = p->win > 0 ? p->ring : nullptr; a.ring_pos = p->ring_pos; a.win = p->win;
  a.acc_len = p->acc_len; a.m = p->m; a.c = p->c; a.cI = p->c_I; a.normalize = p->normalize; a.overlap = p->Cb != nullptr;
  if (!a.Ki) a.cI = 0;
  a.advance = advance; a.n_ctas = p->B;
  size_t smem = (size_t)(p->c > p->c_I ? p->c : p->c_I) * sizeof(float);
  cudaStream_t s = kch_stream(stream);
  if (p->dtype == KCH_BF16) cache_append_kernel<bf16><<<p->B, 128, smem, s>>>(a);
  else cache_append_kernel<float><<<p->B, 128, smem, s>>>(a);
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// One thread advances the device-resident counters after a token has been appended (a separate launch:
// every CTA of the append kernel reads the old values).
__global__ void cache_advance_kernel(int32_t* ctr, int m) {
  int acc = ctr[KCH_CTR_ACC_LEN] + 1;
  ctr[KCH_CTR_RING_N] += 1;
  ctr[KCH_CTR_TOKENS] += 1;
  if (acc >= m) {
    acc = 0;
    ctr[KCH_CTR_N_BLOCKS] += 1;
    ctr[KCH_CTR_HAS_PREV] = 1;
  }
  ctr[KCH_CTR_ACC_LEN] = acc;
}

extern "C" int kch_cache_advance(int32_t* counters, int m, void* stream) {
  KCH_REQUIRE(counters != nullptr && m >= 1, "kch_cache_advance: counters=%p m=%d", (void*)counters, m);
  cache_advance_kernel<<<1, 1, 0, kch_stream(stream)>>>(counters, m);
  KCH_LAUNCH_OK();
  return KCH_OK;
}

// ---------------------------------------------------------------------------------------
// Row-wise (de)quantisation helpers for bulk cache fills (prefill): rows [R,c] fp32/bf16 ->
// block-scaled 8-bit payload + scales + fp32 norm of the dequantised row.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void quantize_rows_kernel(const T* __restrict__ x, int64_t ld, void* __restrict__ payload,
                                     float* __restrict__ scales, float* __restrict__ norms, int64_t rows,
                                     int c, int kind) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float qmax = kind == KCH_FP8_E4M3 ? 448.f : 127.f;
  float nsq = 0.f;
  for (int b64 = 0; b64 < c / 64; ++b64) {
    float v0 = ldf(x + row * ld + b64 * 64 + lane), v1 = ldf(x + row * ld + b64 * 64 + 32 + lane);
    float am = warp_max(fmaxf(fabsf(v0), fabsf(v1)));
    float sc = am > 0.f ? am / qmax : 1.f;
    if (lane == 0) scales[row * (c / 64) + b64] = sc;
    float q0, q1;
    if (kind == KCH_FP8_E4M3) {
      __nv_fp8_e4m3 p0(v0 / sc), p1(v1 / sc);
      ((__nv_fp8_e4m3*)payload)[row * c + b64 * 64 + lane] = p0;
      ((__nv_fp8_e4m3*)payload)[row * c + b64 * 64 + 32 + lane] = p1;
      q0 = float(p0) * sc; q1 = float(p1) * sc;
    } else {
      float r0 = fminf(fmaxf(rintf(v0 / sc), -127.f), 127.f), r1 = fminf(fmaxf(rintf(v1 / sc), -127.f), 127.f);
      ((int8_t*)payload)[row * c + b64 * 64 + lane] = (int8_t)r0;
      ((int8_t*)payload)[row * c + b64 * 64 + 32 + lane] = (int8_t)r1;
      q0 = r0 * sc; q1 = r1 * sc;
    }
    nsq += q0 * q0 + q1 * q1;
  }
  nsq = warp_sum(nsq);
  if (norms && lane == 0) norms[row] = fmaxf(sqrtf(nsq), 1e-12f);
}

extern "C" int kch_quantize_rows(const void* x, int64_t ld, void* payload, float* scales, float* norms,
                                 int64_t rows, int c, int kind, int dtype, void* stream) {
  KCH_REQUIRE(kind == KCH_FP8_E4M3 || kind == KCH_INT8, "kch_quantize_rows: kind=%d", kind);
  KCH_REQUIRE(c >= 64 && c % 64 == 0, "kch_quantize_rows: c=%d must be a multiple of 64", c);
  if (rows <= 0) return KCH_OK;
  dim3 grid((unsigned)ceil_div64(rows, 8)), block(256);
  KCH_DISPATCH_FLOAT(dtype, T, (quantize_rows_kernel<T><<<grid, block, 0, kch_stream(stream)>>>(
      (const T*)x, ld, payload, scales, norms, rows, c, kind)));
  KCH_LAUNCH_OK();
  return KCH_OK;
}
