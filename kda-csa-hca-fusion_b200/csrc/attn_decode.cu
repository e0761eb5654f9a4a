// Attention of one decode step: one query per sequence over that sequence's cache storage
// (CSADecodingCache.forward_step ops_decoding_cache.py:1001-1070, HCADecodingCache.forward_step
// 1318-1395).  Same arithmetic as the full-sequence core: one joint softmax over the selected (or
// all visible) compressed rows and the window ring, a per-head sink logit in the denominator only,
// values == keys, rows used as row / max(||row||, eps) when the cache normalises.
//
// A decode batch has few queries, so the entries of each query are split over gridDim.x CTAs
// (split-softmax): every warp streams its rows once from HBM with an online softmax per head, the
// CTA merges its four warps and writes (max, sum, weighted rows) per head; a second small kernel
// merges the splits, adds the sink and normalises.  All per-step quantities (visible rows, window
// fill) are read from the cache's device counters, so the launch arguments never change from token
// to token.  HBM traffic: each attended row once (c bytes at 8 bits, 2c at bf16) plus its norm/scales.
//
// Geometry of this kernel: c == 128, nh <= 16.  Other shapes use the generic one-CTA-per-query kernel.
#include <math.h>
#include <stdlib.h>

#include "mma_utils.cuh"

#define AD_C 128
#define AD_NH 16
#define AD_THREADS 128
#define AD_MAX_SPLITS 32

struct AdArgs {
  const void* q; int q_dtype; int64_t q_ld; int q_normalize;
  int B, nh;
  const void* comp; int comp_dtype; int64_t cap;
  const float* comp_norms; const float* comp_scales;
  const int32_t* sel; int topk; int m;
  const void* win; int win_dtype; int W;
  const void* sink; int sink_dtype;
  float scale;
  void* out; int out_dtype;
  const int32_t* ctr;
  float* ws;
};

// four consecutive elements (lane*4 ..) of a stored row as fp32
__device__ __forceinline__ float4 load_row4(const void* base, int dtype, int64_t row, int lane, const float* scales) {
  float4 r;
  if (dtype == KCH_BF16) {
    uint2 u = *reinterpret_cast<const uint2*>((const bf16*)base + row * AD_C + lane * 4);
    r.x = __uint_as_float(u.x << 16); r.y = __uint_as_float(u.x & 0xFFFF0000u);
    r.z = __uint_as_float(u.y << 16); r.w = __uint_as_float(u.y & 0xFFFF0000u);
  } else if (dtype == KCH_F32) {
    r = *reinterpret_cast<const float4*>((const float*)base + row * AD_C + lane * 4);
  } else {
    const float sc = scales[row * (AD_C / 64) + (lane >> 4)];
    uint32_t u = *reinterpret_cast<const uint32_t*>((const uint8_t*)base + row * AD_C + lane * 4);
    if (dtype == KCH_FP8_E4M3) {
      __nv_fp8_e4m3 e0, e1, e2, e3;
      e0.__x = u & 0xFF; e1.__x = (u >> 8) & 0xFF; e2.__x = (u >> 16) & 0xFF; e3.__x = u >> 24;
      r.x = float(e0) * sc; r.y = float(e1) * sc; r.z = float(e2) * sc; r.w = float(e3) * sc;
    } else {
      r.x = (float)(int8_t)(u & 0xFF) * sc; r.y = (float)(int8_t)((u >> 8) & 0xFF) * sc;
      r.z = (float)(int8_t)((u >> 16) & 0xFF) * sc; r.w = (float)(int8_t)(u >> 24) * sc;
    }
  }
  return r;
}

__global__ void __launch_bounds__(AD_THREADS) attn_decode_split_kernel(AdArgs a) {
  const int sp = blockIdx.x, S = gridDim.x, b = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ float s_m[4][AD_NH], s_l[4][AD_NH];
  __shared__ float s_acc[4][AD_NH][AD_C];
  // ---- per-step geometry from the device counters -------------------------------------------------------
  const int nb = a.ctr[KCH_CTR_N_BLOCKS];
  int nvis = a.m > 0 ? a.ctr[KCH_CTR_TOKENS] / a.m : nb;
  nvis = a.comp ? min(nvis, nb) : 0;
  const int nw = (a.win && a.W > 0) ? min(a.ctr[KCH_CTR_RING_N], a.W) : 0;
  const int ns = a.sel ? a.topk : nvis;
  const int E = ns + nw;
  const int per = (E + S - 1) / S;
  const int e0 = sp * per, e1 = min(E, e0 + per);
  // ---- the query: lane holds elements lane*4..+3 of every head ---------------------------------------------
  float q[AD_NH][4];
#pragma unroll
  for (int h = 0; h < AD_NH; ++h) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q[h][i] = h < a.nh ? ld_any(a.q, (int64_t)b * a.q_ld + h * AD_C + lane * 4 + i, a.q_dtype) : 0.f;
      ss += q[h][i] * q[h][i];
    }
    if (a.q_normalize) {
      const float nrm = fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[h][i] /= nrm;
    }
  }
  // lane L keeps the running max / sum of head L>>1 (two lanes per head hold the same values)
  float m_run = -INFINITY, l_run = 0.f;
  float acc[AD_NH][4];
#pragma unroll
  for (int h = 0; h < AD_NH; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[h][i] = 0.f;
  const int32_t* selrow = a.sel ? a.sel + (int64_t)b * a.topk : nullptr;

  // Row e of this warp's share: entries e0+warp, e0+warp+4, ...  Block ids of up to 32 rows are fetched with
  // one load (lane i holds the id of the warp's i-th row), rows are then streamed four at a time so that
  // four independent HBM reads are in flight per warp.
  auto row_of = [&](int e, int id, bool& valid) -> int64_t {     // storage row (comp or ring) of entry e
    valid = false;
    if (e >= e1) return 0;
    if (e < ns) {
      if (id < 0 || id >= nvis) return 0;
      valid = true;
      return (int64_t)b * a.cap + id;
    }
    valid = true;
    return (int64_t)b * a.W + (e - ns);
  };
  auto fetch = [&](int e, int64_t row, bool valid) -> float4 {
    if (!valid) return make_float4(0.f, 0.f, 0.f, 0.f);
    if (e < ns) {
      float4 x = load_row4(a.comp, a.comp_dtype, row, lane, a.comp_scales);
      if (a.comp_norms) {
        const float dv = a.comp_norms[row];
        x.x /= dv; x.y /= dv; x.z /= dv; x.w /= dv;
      }
      return x;
    }
    return load_row4(a.win, a.win_dtype, row, lane, nullptr);
  };
  auto consume = [&](const float4& x) {
    // partial dot products of this lane, then a transposing butterfly: 16 shuffles leave the complete
    // dot product of head L>>1 in lane L
    float v[AD_NH];
#pragma unroll
    for (int h = 0; h < AD_NH; ++h) v[h] = q[h][0] * x.x + q[h][1] * x.y + q[h][2] * x.z + q[h][3] * x.w;
#pragma unroll
    for (int st = 0; st < 4; ++st) {
      const int off = 16 >> st, n = 8 >> st;
      const bool up = lane & off;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i < n) {
          const float send = up ? v[i] : v[i + n];
          const float keep = up ? v[i + n] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
      }
    }
    const float s = (v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1)) * a.scale;
    const float m_new = fmaxf(m_run, s);
    const float p = expf(s - m_new);
    const bool grew = m_new > m_run;
    const float corr = grew ? expf(m_run - m_new) : 1.f;     // exp(-inf) = 0 on the first row
    l_run = l_run * corr + p;
    m_run = m_new;
    if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
      for (int h = 0; h < AD_NH; ++h) {
        const float ch = __shfl_sync(0xffffffffu, corr, 2 * h);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] *= ch;
      }
    }
#pragma unroll
    for (int h = 0; h < AD_NH; ++h) {
      const float ph = __shfl_sync(0xffffffffu, p, 2 * h);
      acc[h][0] = fmaf(ph, x.x, acc[h][0]); acc[h][1] = fmaf(ph, x.y, acc[h][1]);
      acc[h][2] = fmaf(ph, x.z, acc[h][2]); acc[h][3] = fmaf(ph, x.w, acc[h][3]);
    }
  };
  for (int base = e0 + warp; base < e1; base += 128) {          // 32 rows of this warp per batch
    const int my_e = base + 4 * lane;
    int my_id = 0;
    if (my_e < e1 && my_e < ns) my_id = selrow ? selrow[my_e] : my_e;
#pragma unroll 1
    for (int i = 0; i < 32 && base + 4 * i < e1; i += 4) {
      float4 x[4]; bool ok[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = base + 4 * (i + j);
        const int id = __shfl_sync(0xffffffffu, my_id, (i + j) & 31);
        const int64_t row = row_of(e, id, ok[j]);
        x[j] = fetch(e, row, ok[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (ok[j]) consume(x[j]);
    }
  }
  // ---- merge the four warps ---------------------------------------------------------------------------
  if ((lane & 1) == 0) { s_m[warp][lane >> 1] = m_run; s_l[warp][lane >> 1] = l_run; }
#pragma unroll
  for (int h = 0; h < AD_NH; ++h)
    *reinterpret_cast<float4*>(&s_acc[warp][h][lane * 4]) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
  __syncthreads();
  float* wsb = a.ws + ((int64_t)b * S + sp) * a.nh * (AD_C + 2);
  for (int h = 0; h < a.nh; ++h) {
    const float M = fmaxf(fmaxf(s_m[0][h], s_m[1][h]), fmaxf(s_m[2][h], s_m[3][h]));
    float L = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = s_m[w][h] > -INFINITY ? expf(s_m[w][h] - M) : 0.f;
      L += s_l[w][h] * f;
      o += s_acc[w][h][tid] * f;
    }
    if (tid == 0) { wsb[h * (AD_C + 2)] = M; wsb[h * (AD_C + 2) + 1] = L; }
    wsb[h * (AD_C + 2) + 2 + tid] = o;
  }
}

__global__ void __launch_bounds__(AD_THREADS) attn_decode_combine_kernel(AdArgs a, int S) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float* wsb = a.ws + (int64_t)b * S * a.nh * (AD_C + 2) + h * (AD_C + 2);
  const int64_t stride = (int64_t)a.nh * (AD_C + 2);
  float M = -INFINITY;
  for (int s = 0; s < S; ++s) M = fmaxf(M, wsb[s * stride]);
  const bool any = M > -INFINITY;
  float sk = 0.f;
  if (a.sink) { sk = ld_any(a.sink, h, a.sink_dtype); if (any) M = fmaxf(M, sk); }
  float den = 0.f, o = 0.f;
  if (any) {
    for (int s = 0; s < S; ++s) {
      const float ms = wsb[s * stride];
      const float f = ms > -INFINITY ? expf(ms - M) : 0.f;
      den += wsb[s * stride + 1] * f;
      o += wsb[s * stride + 2 + d] * f;
    }
    if (a.sink) den += expf(sk - M);
    o /= den;
  }
  const int64_t off = (int64_t)b * a.nh * AD_C + h * AD_C + d;
  if (a.out_dtype == KCH_BF16) ((bf16*)a.out)[off] = __float2bfloat16_rn(o);
  else ((float*)a.out)[off] = o;
}

// =====================================================================================================
// Tensor-core variant for the production case: cosine scoring (rows carry norms), stored rows in bf16 or
// block-scaled 8 bits, ring in bf16.  The 16 heads are the M = 16 rows of mma.sync m16n8k16 tiles, as in the
// full-sequence kernel, but the operands are exact: the stored row (bf16, or the 8-bit payload, which bf16
// holds exactly) is the B operand as it lies in memory, and everything that is not representable in bf16 is
// moved to the fp32 side or split in two bf16 terms:
//   s_r   = scale * (Sa_r * va_r + Sb_r * vb_r),  Sa / Sb = q . payload over columns 0-63 / 64-127,
//           v*_r = block scale / ||row||  (1 / ||row|| for bf16 rows, 1 for ring rows),  q = q_hi + q_lo
//   O    += (p_r * va_r) . payload[:, 0:64]   and   (p_r * vb_r) . payload[:, 64:128],   p * v = hi + lo
// so the result has fp32-grade accuracy (dropped terms ~2^-17 relative).  Because |s| <= |scale| the softmax
// uses the fixed shift max(|scale|, sink_h): partial sums of different warps / CTAs simply add.
// Each warp streams 32-row tiles through a 3-stage cp.async ring (raw bytes; 8-bit tiles are expanded to a
// bf16 work tile in shared memory); a CTA is two warps, the entries of a query are split over gridDim.x CTAs.
// =====================================================================================================
#define ADM_WARPS 2
#define ADM_TILE 32
#define ADM_STAGES 3
#define ADM_STAGE_BYTES (ADM_TILE * AD_C * 2)   // one bf16 tile; an 8-bit tile uses the first half
#define ADM_QLD 136

__device__ __forceinline__ void adm_cp16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void adm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void adm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void adm_ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void adm_ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void adm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t adm_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// (x0, x1) -> packed bf16 pair of the leading terms and of the remainders
__device__ __forceinline__ void adm_split(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = adm_pack(x0, x1);
  lo = adm_pack(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xFFFF0000u));
}

template <bool Q8>
__global__ void __launch_bounds__(ADM_WARPS * 32) attn_decode_mma_kernel(AdArgs a) {
  extern __shared__ __align__(128) uint8_t adm_smem[];
  const int sp = blockIdx.x, S = gridDim.x, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  // shared memory: [q_hi 16 x 136 bf16][q_lo 16 x 136 bf16][per warp: 3 ring stages + one bf16 work tile]
  bf16* sq_hi = reinterpret_cast<bf16*>(adm_smem);
  bf16* sq_lo = sq_hi + 16 * ADM_QLD;
  uint8_t* wbase = adm_smem + 2 * 16 * ADM_QLD * 2 + (size_t)warp * ((ADM_STAGES + 1) * ADM_STAGE_BYTES);
  const uint32_t ring = smem_addr_u32(wbase);
  const uint32_t work = ring + ADM_STAGES * ADM_STAGE_BYTES;
  // ---- per-step geometry from the device counters -------------------------------------------------------
  const int nb = a.ctr[KCH_CTR_N_BLOCKS];
  int nvis = a.m > 0 ? a.ctr[KCH_CTR_TOKENS] / a.m : nb;
  nvis = a.comp ? min(nvis, nb) : 0;
  const int nw = (a.win && a.W > 0) ? min(a.ctr[KCH_CTR_RING_N], a.W) : 0;
  const int ns = a.sel ? a.topk : nvis;
  const int ns_pad = (ns + ADM_TILE - 1) & ~(ADM_TILE - 1);   // ring rows start on a tile boundary: tiles are homogeneous
  const int E = ns_pad + nw;
  const int tiles_total = (E + ADM_TILE - 1) / ADM_TILE;
  const int tiles_per = (tiles_total + S - 1) / S;
  const int tile_lo = sp * tiles_per, tile_hi = min(tiles_total, tile_lo + tiles_per);
  const int my_tiles = tile_hi > tile_lo + warp ? (tile_hi - tile_lo - warp + ADM_WARPS - 1) / ADM_WARPS : 0;
  const int32_t* selrow = a.sel ? a.sel + (int64_t)b * a.topk : nullptr;
  // ---- the query, normalised in fp32, as two bf16 terms (the whole CTA shares it) ----------------------------
  auto fetch_id = [&](int t_local) -> int {
    if (t_local >= my_tiles) return -1;
    const int tile = tile_lo + warp + t_local * ADM_WARPS;
    const int e = tile * ADM_TILE + lane;
    if (tile * ADM_TILE >= ns_pad || e >= ns) return -1;
    return selrow ? selrow[e] : e;
  };
  int id_pre[ADM_STAGES];
#pragma unroll
  for (int s2 = 0; s2 < ADM_STAGES; ++s2) id_pre[s2] = fetch_id(s2);       // with the query loads below: one round trip
  float qv[16 / ADM_WARPS][4];                         // every head's loads are in flight before the first norm
  if (a.q_dtype == KCH_BF16 && ((((uintptr_t)a.q) | (uintptr_t)(a.q_ld * 2)) & 7) == 0) {
    // raw 8-byte loads first, conversions after: a conversion next to its load would wait for it, head after head
    uint2 raw[16 / ADM_WARPS];
#pragma unroll
    for (int hh = 0; hh < 16 / ADM_WARPS; ++hh) {
      const int h = min(warp + hh * ADM_WARPS, a.nh - 1);
      raw[hh] = *reinterpret_cast<const uint2*>((const bf16*)a.q + (int64_t)b * a.q_ld + h * AD_C + lane * 4);
    }
#pragma unroll
    for (int hh = 0; hh < 16 / ADM_WARPS; ++hh) {
      const bool on = warp + hh * ADM_WARPS < a.nh;
      qv[hh][0] = on ? __uint_as_float(raw[hh].x << 16) : 0.f; qv[hh][1] = on ? __uint_as_float(raw[hh].x & 0xFFFF0000u) : 0.f;
      qv[hh][2] = on ? __uint_as_float(raw[hh].y << 16) : 0.f; qv[hh][3] = on ? __uint_as_float(raw[hh].y & 0xFFFF0000u) : 0.f;
    }
  } else if (a.q_dtype == KCH_F32 && ((((uintptr_t)a.q) | (uintptr_t)(a.q_ld * 4)) & 15) == 0) {
    float4 raw[16 / ADM_WARPS];
#pragma unroll
    for (int hh = 0; hh < 16 / ADM_WARPS; ++hh) {
      const int h = min(warp + hh * ADM_WARPS, a.nh - 1);
      raw[hh] = *reinterpret_cast<const float4*>((const float*)a.q + (int64_t)b * a.q_ld + h * AD_C + lane * 4);
    }
#pragma unroll
    for (int hh = 0; hh < 16 / ADM_WARPS; ++hh) {
      const bool on = warp + hh * ADM_WARPS < a.nh;
      qv[hh][0] = on ? raw[hh].x : 0.f; qv[hh][1] = on ? raw[hh].y : 0.f;
      qv[hh][2] = on ? raw[hh].z : 0.f; qv[hh][3] = on ? raw[hh].w : 0.f;
    }
  } else {
#pragma unroll
    for (int hh = 0; hh < 16 / ADM_WARPS; ++hh) {
      const int h = warp + hh * ADM_WARPS;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        qv[hh][i] = h < a.nh ? ld_any(a.q, (int64_t)b * a.q_ld + h * AD_C + lane * 4 + i, a.q_dtype) : 0.f;
    }
  }
#pragma unroll
  for (int hh = 0; hh < 16 / ADM_WARPS; ++hh) {
    const int h = warp + hh * ADM_WARPS;
    float v[4] = {qv[hh][0], qv[hh][1], qv[hh][2], qv[hh][3]};
    if (a.q_normalize) {
      const float nrm = fmaxf(sqrtf(warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3])), 1e-12f);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] /= nrm;
    }
    uint2 hi, lo;
    adm_split(v[0], v[1], hi.x, lo.x);
    adm_split(v[2], v[3], hi.y, lo.y);
    *reinterpret_cast<uint2*>(sq_hi + h * ADM_QLD + lane * 4) = hi;
    *reinterpret_cast<uint2*>(sq_lo + h * ADM_QLD + lane * 4) = lo;
  }
  __syncthreads();
  uint32_t qh[8][4], ql[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qh[ks][0] = *reinterpret_cast<const uint32_t*>(sq_hi + g * ADM_QLD + 16 * ks + 2 * j);
    qh[ks][1] = *reinterpret_cast<const uint32_t*>(sq_hi + (g + 8) * ADM_QLD + 16 * ks + 2 * j);
    qh[ks][2] = *reinterpret_cast<const uint32_t*>(sq_hi + g * ADM_QLD + 16 * ks + 8 + 2 * j);
    qh[ks][3] = *reinterpret_cast<const uint32_t*>(sq_hi + (g + 8) * ADM_QLD + 16 * ks + 8 + 2 * j);
    ql[ks][0] = *reinterpret_cast<const uint32_t*>(sq_lo + g * ADM_QLD + 16 * ks + 2 * j);
    ql[ks][1] = *reinterpret_cast<const uint32_t*>(sq_lo + (g + 8) * ADM_QLD + 16 * ks + 2 * j);
    ql[ks][2] = *reinterpret_cast<const uint32_t*>(sq_lo + g * ADM_QLD + 16 * ks + 8 + 2 * j);
    ql[ks][3] = *reinterpret_cast<const uint32_t*>(sq_lo + (g + 8) * ADM_QLD + 16 * ks + 8 + 2 * j);
  }
  // ---- tile streaming -----------------------------------------------------------------------------------
  // lane e of tile t resolves entry 32 t + e: row pointer (nullptr = invalid, zero-filled), value factors va / vb
  // The chain selected index -> row address -> row bytes is two dependent round trips per tile; they are taken apart:
  // the index of a tile is fetched one tile ahead of the copy that needs it (`fetch_id`), and the row's norm and scales
  // are only loaded at issue time -- the division happens when the tile is consumed, two tiles later.
  struct Meta { float va, vb, nrm; uint32_t valid; bool q8; };    // value factors are va / nrm, vb / nrm
  auto issue_tile = [&](int t_local, int id, Meta& mt) {
    const int tile = tile_lo + warp + t_local * ADM_WARPS;
    const int e = tile * ADM_TILE + lane;
    const bool comp_tile = tile * ADM_TILE < ns_pad;
    const uint8_t* p = nullptr;
    mt.va = mt.vb = 0.f;
    mt.nrm = 1.f;
    if (comp_tile) {
      if (e < ns) {
        if (id >= 0 && id < nvis) {
          const int64_t row = (int64_t)b * a.cap + id;
          p = (const uint8_t*)a.comp + row * (Q8 ? AD_C : AD_C * 2);
          mt.nrm = a.comp_norms[row];
          if (Q8) { mt.va = a.comp_scales[row * 2]; mt.vb = a.comp_scales[row * 2 + 1]; }
          else { mt.va = mt.vb = 1.f; }
        }
      }
    } else if (e - ns_pad < nw) {
      p = (const uint8_t*)a.win + ((int64_t)b * a.W + (e - ns_pad)) * (AD_C * 2);
      mt.va = mt.vb = 1.f;
    }
    mt.valid = __ballot_sync(0xffffffffu, p != nullptr);
    mt.q8 = Q8 && comp_tile;
    const uint32_t dst0 = ring + (uint32_t)(t_local % ADM_STAGES) * ADM_STAGE_BYTES;
    if (mt.q8) {
      // raw payload rows of 128 bytes, 8 chunks each, unswizzled (expanded to the work tile after arrival)
      const int ch = lane & 7;
#pragma unroll
      for (int it = 0; it < ADM_TILE / 4; ++it) {
        const int r = 4 * it + (lane >> 3);
        const uint8_t* rp = (const uint8_t*)__shfl_sync(0xffffffffu, (unsigned long long)p, r);
        adm_cp16(dst0 + r * AD_C + (ch << 4), rp ? (const void*)(rp + ch * 16) : (const void*)a.ctr, rp ? 16 : 0);
      }
    } else {
      const int ch = lane & 15;
#pragma unroll
      for (int it = 0; it < ADM_TILE / 2; ++it) {
        const int r = 2 * it + (lane >> 4);
        const uint8_t* rp = (const uint8_t*)__shfl_sync(0xffffffffu, (unsigned long long)p, r);
        adm_cp16(dst0 + r * (AD_C * 2) + ((ch ^ (r & 7)) << 4), rp ? (const void*)(rp + ch * 16) : (const void*)a.ctr,
                 rp ? 16 : 0);
      }
    }
    adm_commit();
  };
  Meta meta[ADM_STAGES];
#pragma unroll
  for (int s2 = 0; s2 < ADM_STAGES; ++s2) { meta[s2].va = meta[s2].vb = 0.f; meta[s2].nrm = 1.f; meta[s2].valid = 0; meta[s2].q8 = false; }
#pragma unroll
  for (int s2 = 0; s2 < ADM_STAGES - 1; ++s2) {
    if (s2 < my_tiles) issue_tile(s2, id_pre[s2], meta[s2]); else adm_commit();
  }
  int id_next = id_pre[ADM_STAGES - 1];                                    // index of tile t + ADM_STAGES - 1, fetched a tile ahead
  const float ascale = fabsf(a.scale);
  float sink0 = -INFINITY, sink1 = -INFINITY;
  if (a.sink) {
    if (g < a.nh) sink0 = ld_any(a.sink, g, a.sink_dtype);
    if (g + 8 < a.nh) sink1 = ld_any(a.sink, g + 8, a.sink_dtype);
  }
  const float shift0 = fmaxf(ascale, sink0), shift1 = fmaxf(ascale, sink1);
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float l0 = 0.f, l1 = 0.f;
  bool any_valid = false;

#pragma unroll 1
  for (int t = 0; t < my_tiles; ++t) {
    {
      const int nt = t + ADM_STAGES - 1;
      Meta mt; mt.va = mt.vb = 0.f; mt.nrm = 1.f; mt.valid = 0; mt.q8 = false;
      if (nt < my_tiles) issue_tile(nt, id_next, mt); else adm_commit();
      id_next = fetch_id(nt + 1);
      // the register array is indexed with compile-time constants only
      if (nt % ADM_STAGES == 0) meta[0] = mt; else if (nt % ADM_STAGES == 1) meta[1] = mt; else meta[2] = mt;
    }
    adm_wait<ADM_STAGES - 1>();
    __syncwarp();
    const int st = t % ADM_STAGES;
    Meta mt = st == 0 ? meta[0] : (st == 1 ? meta[1] : meta[2]);
    mt.va = mt.va / mt.nrm;                       // same operands as scale / norm (1 / norm for bf16 rows)
    mt.vb = mt.vb / mt.nrm;
    any_valid |= mt.valid != 0;
    uint32_t tb = ring + (uint32_t)st * ADM_STAGE_BYTES;
    if (Q8 && mt.q8) {
      // expand the 8-bit payload to bf16 (exact) into the swizzled work tile
      const uint8_t* raw = wbase + (size_t)st * ADM_STAGE_BYTES;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int idx = it * 32 + lane, r = idx >> 3, ch = idx & 7;
        const uint4 v = *reinterpret_cast<const uint4*>(raw + r * AD_C + (ch << 4));
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
        uint32_t ob[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float f0, f1, f2, f3;
          if (a.comp_dtype == KCH_FP8_E4M3) {
            __nv_fp8_e4m3 e0, e1, e2, e3;
            e0.__x = w4[k] & 0xFF; e1.__x = (w4[k] >> 8) & 0xFF; e2.__x = (w4[k] >> 16) & 0xFF; e3.__x = w4[k] >> 24;
            f0 = float(e0); f1 = float(e1); f2 = float(e2); f3 = float(e3);
          } else {
            f0 = (float)(int8_t)(w4[k] & 0xFF); f1 = (float)(int8_t)((w4[k] >> 8) & 0xFF);
            f2 = (float)(int8_t)((w4[k] >> 16) & 0xFF); f3 = (float)(int8_t)(w4[k] >> 24);
          }
          ob[2 * k] = adm_pack(f0, f1);
          ob[2 * k + 1] = adm_pack(f2, f3);
        }
        uint8_t* wt = wbase + (size_t)ADM_STAGES * ADM_STAGE_BYTES;
        *reinterpret_cast<uint4*>(wt + r * (AD_C * 2) + (((2 * ch) ^ (r & 7)) << 4)) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
        *reinterpret_cast<uint4*>(wt + r * (AD_C * 2) + (((2 * ch + 1) ^ (r & 7)) << 4)) = make_uint4(ob[4], ob[5], ob[6], ob[7]);
      }
      __syncwarp();
      tb = work;
    }
    // ---- S = Q X^T for the 32 rows, kept apart for the two 64-column halves --------------------------------
    uint32_t pah[2][4], pal[2][4], pbh[2][4], pbl[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
      const int krow = 8 * nt + (lane & 7);
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        const int ch = 4 * qd + (lane >> 3);
        uint32_t r0, r1, r2, r3;
        adm_ldsm4(tb + krow * (AD_C * 2) + ((ch ^ (krow & 7)) << 4), r0, r1, r2, r3);
        if (qd < 2) {
          adm_mma(sa, qh[2 * qd], r0, r1); adm_mma(sa, ql[2 * qd], r0, r1);
          adm_mma(sa, qh[2 * qd + 1], r2, r3); adm_mma(sa, ql[2 * qd + 1], r2, r3);
        } else {
          adm_mma(sb, qh[2 * qd], r0, r1); adm_mma(sb, ql[2 * qd], r0, r1);
          adm_mma(sb, qh[2 * qd + 1], r2, r3); adm_mma(sb, ql[2 * qd + 1], r2, r3);
        }
      }
      // this thread's columns: rows 8nt + 2j and 8nt + 2j + 1 of the tile
      const int k0 = 8 * nt + 2 * j;
      const float va0 = __shfl_sync(0xffffffffu, mt.va, k0), va1 = __shfl_sync(0xffffffffu, mt.va, k0 + 1);
      const float vb0 = __shfl_sync(0xffffffffu, mt.vb, k0), vb1 = __shfl_sync(0xffffffffu, mt.vb, k0 + 1);
      const bool v0 = (mt.valid >> k0) & 1u, v1 = (mt.valid >> (k0 + 1)) & 1u;
      const float p00 = v0 ? __expf(fminf((sa[0] * va0 + sb[0] * vb0) * a.scale - shift0, 80.f)) : 0.f;
      const float p01 = v1 ? __expf(fminf((sa[1] * va1 + sb[1] * vb1) * a.scale - shift0, 80.f)) : 0.f;
      const float p10 = v0 ? __expf(fminf((sa[2] * va0 + sb[2] * vb0) * a.scale - shift1, 80.f)) : 0.f;
      const float p11 = v1 ? __expf(fminf((sa[3] * va1 + sb[3] * vb1) * a.scale - shift1, 80.f)) : 0.f;
      l0 += p00 + p01;
      l1 += p10 + p11;
      const int ksx = nt >> 1, rx = (nt & 1) * 2;
      adm_split(p00 * va0, p01 * va1, pah[ksx][rx], pal[ksx][rx]);
      adm_split(p10 * va0, p11 * va1, pah[ksx][rx + 1], pal[ksx][rx + 1]);
      if (Q8) {
        adm_split(p00 * vb0, p01 * vb1, pbh[ksx][rx], pbl[ksx][rx]);
        adm_split(p10 * vb0, p11 * vb1, pbh[ksx][rx + 1], pbl[ksx][rx + 1]);
      }
    }
    // ---- O += (P v) X : 2 k-steps of 16 rows, 16 n-tiles of 8 channels -----------------------------------
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const int krow = 16 * ks + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int ch = 2 * dp + (lane >> 4);
        uint32_t r0, r1, r2, r3;
        adm_ldsm4t(tb + krow * (AD_C * 2) + ((ch ^ (krow & 7)) << 4), r0, r1, r2, r3);
        if (Q8 && dp >= 4) {
          adm_mma(o[2 * dp], pbh[ks], r0, r1); adm_mma(o[2 * dp], pbl[ks], r0, r1);
          adm_mma(o[2 * dp + 1], pbh[ks], r2, r3); adm_mma(o[2 * dp + 1], pbl[ks], r2, r3);
        } else {
          adm_mma(o[2 * dp], pah[ks], r0, r1); adm_mma(o[2 * dp], pal[ks], r0, r1);
          adm_mma(o[2 * dp + 1], pah[ks], r2, r3); adm_mma(o[2 * dp + 1], pal[ks], r2, r3);
        }
      }
    }
    __syncwarp();
  }
  adm_wait<0>();
  // ---- merge the warps and write the partial ----------------------------------------------------------------
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();                               // every warp is done with the query tile and its ring
  float* s_o = reinterpret_cast<float*>(adm_smem + 2 * 16 * ADM_QLD * 2);   // [warps][16][128] over the rings
  float* s_l = reinterpret_cast<float*>(adm_smem);                          // [warps][16] (+ any flags) over the query tile
  int* s_any = reinterpret_cast<int*>(adm_smem + ADM_WARPS * 16 * 4);
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    const int d = 8 * n + 2 * j;
    *reinterpret_cast<float2*>(s_o + ((size_t)warp * 16 + g) * AD_C + d) = make_float2(o[n][0], o[n][1]);
    *reinterpret_cast<float2*>(s_o + ((size_t)warp * 16 + g + 8) * AD_C + d) = make_float2(o[n][2], o[n][3]);
  }
  if (j == 0) { s_l[warp * 16 + g] = l0; s_l[warp * 16 + g + 8] = l1; }
  if (lane == 0) s_any[warp] = any_valid ? 1 : 0;
  __syncthreads();
  bool any = false;
#pragma unroll
  for (int w = 0; w < ADM_WARPS; ++w) any = any || s_any[w] != 0;
  float* wsb = a.ws + ((int64_t)b * S + sp) * a.nh * (AD_C + 2);
  for (int idx = tid; idx < a.nh * AD_C; idx += ADM_WARPS * 32) {
    const int h = idx >> 7, d = idx & 127;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < ADM_WARPS; ++w) v += s_o[((size_t)w * 16 + h) * AD_C + d];
    wsb[h * (AD_C + 2) + 2 + d] = v;
  }
  if (tid < a.nh) {
    float sk = -INFINITY;
    if (a.sink) sk = ld_any(a.sink, tid, a.sink_dtype);
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < ADM_WARPS; ++w) l += s_l[w * 16 + tid];
    wsb[tid * (AD_C + 2)] = any ? fmaxf(ascale, sk) : -INFINITY;
    wsb[tid * (AD_C + 2) + 1] = l;
  }
}

static bool attend_decode_mma_ok(const kch_attend_decode_args* p) {
  if (!p->comp || !p->comp_norms) return false;                       // cosine scoring only (bounded logits)
  if (p->comp_dtype != KCH_BF16 && p->comp_dtype != KCH_FP8_E4M3 && p->comp_dtype != KCH_INT8) return false;
  if (p->win && p->sliding_window > 0 && p->win_dtype != KCH_BF16) return false;
  if (!(fabsf(p->scale) <= 16.f)) return false;
  if (((uintptr_t)p->comp & 15) || (p->win && ((uintptr_t)p->win & 15))) return false;
  return true;
}

extern "C" int kch_attend_decode_splits(int B) {
  if (B < 1) return 1;
  static const int forced = [] { const char* e = getenv("KCH_DECODE_SPLITS"); return e ? atoi(e) : 0; }();
  // One wave of CTAs (three fit on an SM beside their tile rings): each warp then streams a few tiles through its
  // ring instead of paying the query set-up and a partial-result round trip for a single tile.
  // (KCH_DECODE_SPLITS=n overrides, for comparison.)
  int s = forced > 0 ? forced : (3 * 148) / B;
  return s < 1 ? 1 : (s > AD_MAX_SPLITS ? AD_MAX_SPLITS : s);
}

extern "C" int64_t kch_attend_decode_workspace_bytes(int B, int nh, int c) {
  if (B < 1 || nh < 1 || c < 1) return 0;
  return (int64_t)B * kch_attend_decode_splits(B) * nh * (c + 2) * (int64_t)sizeof(float);
}

extern "C" int kch_attend_decode(const kch_attend_decode_args* p, void* stream) {
  KCH_REQUIRE(p != nullptr, "kch_attend_decode: null args");
  KCH_REQUIRE(p->c == AD_C && p->nh >= 1 && p->nh <= AD_NH, "kch_attend_decode: c=%d nh=%d (needs c == 128, nh <= 16)",
              p->c, p->nh);
  KCH_REQUIRE(p->B >= 1, "B=%d must be >= 1", p->B);
  KCH_REQUIRE(p->counters != nullptr, "kch_attend_decode: the cache's device counters are required");
  KCH_REQUIRE(p->topk >= 0 && p->sliding_window >= 0, "kch_attend_decode: topk=%d sliding_window=%d", p->topk,
              p->sliding_window);
  KCH_REQUIRE(p->q_ld >= (int64_t)p->nh * p->c && p->q && p->out, "kch_attend_decode: q / out / q_ld");
  if (p->comp) {
    KCH_REQUIRE(p->comp_dtype == KCH_F32 || p->comp_dtype == KCH_BF16 || p->comp_dtype == KCH_FP8_E4M3 ||
                p->comp_dtype == KCH_INT8, "kch_attend_decode: comp_dtype=%d", p->comp_dtype);
    if (p->comp_dtype == KCH_FP8_E4M3 || p->comp_dtype == KCH_INT8)
      KCH_REQUIRE(p->comp_scales != nullptr, "block-scaled 8-bit rows need their scales");
    KCH_REQUIRE(p->m >= 1, "m=%d must be >= 1", p->m);
  }
  if (p->win) KCH_REQUIRE(p->win_dtype == KCH_F32 || p->win_dtype == KCH_BF16, "kch_attend_decode: win_dtype=%d", p->win_dtype);
  const int S = kch_attend_decode_splits(p->B);
  KCH_REQUIRE(p->workspace && p->workspace_bytes >= kch_attend_decode_workspace_bytes(p->B, p->nh, p->c),
              "kch_attend_decode: workspace of %lld bytes needed", (long long)kch_attend_decode_workspace_bytes(p->B, p->nh, p->c));
  AdArgs a;
  a.q = p->q; a.q_dtype = p->q_dtype; a.q_ld = p->q_ld; a.q_normalize = p->q_normalize;
  a.B = p->B; a.nh = p->nh;
  a.comp = p->comp; a.comp_dtype = p->comp_dtype; a.cap = p->capacity;
  a.comp_norms = p->comp_norms; a.comp_scales = p->comp_scales;
  a.sel = p->comp ? p->sel_indices : nullptr; a.topk = a.sel ? p->topk : 0; a.m = p->m;
  a.win = p->sliding_window > 0 ? p->win : nullptr; a.win_dtype = p->win_dtype; a.W = p->sliding_window;
  a.sink = p->sink; a.sink_dtype = p->sink_dtype; a.scale = p->scale;
  a.out = p->out; a.out_dtype = p->out_dtype; a.ctr = p->counters; a.ws = (float*)p->workspace;
  cudaStream_t s = kch_stream(stream);
  static const bool force_simt = [] { const char* e = getenv("KCH_ATTEND_DECODE"); return e && e[0] == 's'; }();
  if (!force_simt && attend_decode_mma_ok(p)) {
    const size_t smem = 2 * 16 * ADM_QLD * 2 + (size_t)ADM_WARPS * ((ADM_STAGES + 1) * ADM_STAGE_BYTES);
    if (p->comp_dtype == KCH_BF16) {
      KCH_CUDA_OK(cudaFuncSetAttribute(attn_decode_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      attn_decode_mma_kernel<false><<<dim3(S, p->B), ADM_WARPS * 32, smem, s>>>(a);
    } else {
      KCH_CUDA_OK(cudaFuncSetAttribute(attn_decode_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      attn_decode_mma_kernel<true><<<dim3(S, p->B), ADM_WARPS * 32, smem, s>>>(a);
    }
  } else {
    attn_decode_split_kernel<<<dim3(S, p->B), AD_THREADS, 0, s>>>(a);
  }
  KCH_LAUNCH_OK();
  attn_decode_combine_kernel<<<dim3(p->nh, p->B), AD_THREADS, 0, s>>>(a, S);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
