// Shared-KV multi-query attention core with ONE joint softmax over
//   [selected (CSA) or all visible (HCA) compressed entries]  U  [sliding-window entries]
// and an optional per-head attention-sink logit that only enters the denominator:
//   p_j = exp(s_j) / (sum_i exp(s_i) + exp(sink_h)),   out = sum_j p_j x_j   (values == keys)
// Follows naive_csa (ops_csa.py:923-1155), naive_hca (ops_hca.py:139-192) and the decode-time
// forward_step of both caches (ops_decoding_cache.py:891-1070, 1318-1395).
//
// Generic kernel: one CTA per query position; any head count / width (c <= 256); keys may be fp32,
// bf16 or block-scaled 8-bit (e4m3 / int8 with one fp32 scale per 64 elements), optionally divided
// by a per-row norm (decode caches keep the stored row and its norm instead of a normalised copy).
#include <math.h>
#include <stdlib.h>

#include "kch_common.cuh"

struct AttnArgs {
  const void* q; int q_dtype; int64_t q_ld; int q_normalize;
  int B, T, nh, c;
  const void* comp; int comp_dtype; int64_t comp_ld; int64_t comp_batch_rows; int n_comp;
  const float* comp_norms; const float* comp_scales;
  const int32_t* sel; int topk;
  int m; int64_t t0; int nvis_fixed;
  const void* win_ptr; int win_dtype; int64_t win_ld; int64_t win_batch_rows; int win_size; int win_mode; int win_len;
  int win_t0;
  const void* sink; int sink_dtype;
  float scale;
  void* out; int out_dtype;
};

__device__ __forceinline__ float key_elem(const void* base, int dtype, int64_t row, int64_t ld, int d,
                                          const float* scales, int c) {
  switch (dtype) {
    case KCH_F32: return ((const float*)base)[row * ld + d];
    case KCH_BF16: return __bfloat162float(((const bf16*)base)[row * ld + d]);
    case KCH_FP8_E4M3: {
      __nv_fp8_e4m3 v = ((const __nv_fp8_e4m3*)base)[row * ld + d];
      return float(v) * scales[row * (c / 64) + d / 64];
    }
    default: {  // KCH_INT8
      int8_t v = ((const int8_t*)base)[row * ld + d];
      return (float)v * scales[row * (c / 64) + d / 64];
    }
  }
}

template <int HB>
__global__ void __launch_bounds__(256) attn_generic_kernel(AttnArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int64_t bt = blockIdx.x;
  const int t = (int)(bt % a.T), b = (int)(bt / a.T);
  const int nh = a.nh, c = a.c;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // entry list geometry
  int64_t nv64 = a.nvis_fixed >= 0 ? a.nvis_fixed : (a.m > 0 ? (a.t0 + t + 1) / a.m : a.n_comp);
  const int nvis = (int)(nv64 < a.n_comp ? nv64 : a.n_comp);
  const int ns = a.sel ? a.topk : nvis;            // sparse slots or dense visible blocks
  int nw, wrow0;                                     // window entries and their first row
  if (a.win_size <= 0 || !a.win_ptr) { nw = 0; wrow0 = 0; }
  else if (a.win_mode == 1) { nw = a.win_len; wrow0 = 0; }
  else { const int tw = t + a.win_t0; int lo = tw - a.win_size + 1; if (lo < 0) lo = 0; nw = tw - lo + 1; wrow0 = lo; }
  const int E = ns + nw;
  float* sq = smem;                 // [nh][c]
  float* ss = sq + nh * c;          // [E][nh]   scores, then probabilities
  float* sred = ss + (size_t)(E > 0 ? E : 1) * nh;  // partial sums for the P.V reduction
  // ---- queries -----------------------------------------------------------------------
  for (int h = warp; h < nh; h += 8) {
    float ssum = 0.f;
    for (int d = lane; d < c; d += 32) {
      float v = ld_any(a.q, bt * a.q_ld + (int64_t)h * c + d, a.q_dtype);
      sq[h * c + d] = v;
      ssum += v * v;
    }
    if (a.q_normalize) {
      float nrm = fmaxf(sqrtf(warp_sum(ssum)), 1e-12f);
      for (int d = lane; d < c; d += 32) sq[h * c + d] /= nrm;
    }
  }
  __syncthreads();
  const int32_t* selrow = a.sel ? a.sel + bt * a.topk : nullptr;
  const int64_t comp_row0 = (int64_t)b * a.comp_batch_rows;
  const int64_t win_row0 = (int64_t)b * a.win_batch_rows + wrow0;
  // ---- scores: one warp per entry ------------------------------------------------------
  for (int e = warp; e < E; e += 8) {
    bool valid = true;
    const void* base; int dt; int64_t row, ld; const float* scales = nullptr; float div = 1.f;
    if (e < ns) {
      int id = selrow ? selrow[e] : e;
      valid = id >= 0 && id < nvis;
      row = comp_row0 + (valid ? id : 0);
      base = a.comp; dt = a.comp_dtype; ld = a.comp_ld; scales = a.comp_scales;
      if (a.comp_norms) div = a.comp_norms[row];
    } else {
      row = win_row0 + (e - ns);
      base = a.win_ptr; dt = a.win_dtype; ld = a.win_ld;
    }
    if (!valid) {
      for (int h = lane; h < nh; h += 32) ss[(size_t)e * nh + h] = -INFINITY;
      continue;
    }
    float kv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int d = lane + 32 * i;
      kv[i] = d < c ? key_elem(base, dt, row, ld, d, scales, c) / div : 0.f;
    }
    for (int h = 0; h < nh; ++h) {
      float p = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int d = lane + 32 * i;
        if (d < c) p = fmaf(sq[h * c + d], kv[i], p);
      }
      p = warp_sum(p);
      if (lane == 0) ss[(size_t)e * nh + h] = p * a.scale;
    }
  }
  __syncthreads();
  // ---- joint softmax per head (one warp per head) ----------------------------------------
  for (int h = warp; h < nh; h += 8) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, ss[(size_t)e * nh + h]);
    mx = warp_max(mx);
    const bool any = mx > -INFINITY;
    float sk = 0.f;
    if (a.sink) { sk = ld_any(a.sink, h, a.sink_dtype); if (any) mx = fmaxf(mx, sk); }
    float den = 0.f;
    for (int e = lane; e < E; e += 32) {
      float p = any ? expf(ss[(size_t)e * nh + h] - mx) : 0.f;
      ss[(size_t)e * nh + h] = p;
      den += p;
    }
    den = warp_sum(den);
    if (a.sink && any) den += expf(sk - mx);
    float inv = any ? 1.f / den : 0.f;
    for (int e = lane; e < E; e += 32) ss[(size_t)e * nh + h] *= inv;
  }
  __syncthreads();
  // ---- out = P . X : thread owns channel d, entry subsets are split across thread groups ----
  const int split = 256 / c > 0 ? 256 / c : 1;
  const int sp = tid / c, d = tid % c;
  const bool active = tid < split * c;
  for (int h0 = 0; h0 < nh; h0 += HB) {
    float acc[HB];
#pragma unroll
    for (int i = 0; i < HB; ++i) acc[i] = 0.f;
    if (active) {
      for (int e = sp; e < E; e += split) {
        const void* base; int dt; int64_t row, ld; const float* scales = nullptr; float div = 1.f;
        if (e < ns) {
          int id = selrow ? selrow[e] : e;
          if (id < 0 || id >= nvis) continue;
          row = comp_row0 + id;
          base = a.comp; dt = a.comp_dtype; ld = a.comp_ld; scales = a.comp_scales;
          if (a.comp_norms) div = a.comp_norms[row];
        } else {
          row = win_row0 + (e - ns);
          base = a.win_ptr; dt = a.win_dtype; ld = a.win_ld;
        }
        float kvv = key_elem(base, dt, row, ld, d, scales, c) / div;
#pragma unroll
        for (int i = 0; i < HB; ++i)
          if (h0 + i < nh) acc[i] = fmaf(ss[(size_t)e * nh + h0 + i], kvv, acc[i]);
      }
    }
    if (split > 1) {
      if (active)
#pragma unroll
        for (int i = 0; i < HB; ++i) sred[(sp * HB + i) * c + d] = acc[i];
      __syncthreads();
      if (tid < c) {
#pragma unroll
        for (int i = 0; i < HB; ++i) {
          float r = 0.f;
          for (int s2 = 0; s2 < split; ++s2) r += sred[(s2 * HB + i) * c + tid];
          acc[i] = r;
        }
      }
      __syncthreads();
    }
    if (tid < c) {
#pragma unroll
      for (int i = 0; i < HB; ++i)
        if (h0 + i < nh) {
          int64_t off = bt * ((int64_t)nh * c) + (int64_t)(h0 + i) * c + tid;
          if (a.out_dtype == KCH_BF16) ((bf16*)a.out)[off] = __float2bfloat16_rn(acc[i]);
          else ((float*)a.out)[off] = acc[i];
        }
    }
  }
}

bool kch_attend_mma_supported(const kch_attend_args* p);
int kch_attend_mma(const kch_attend_args* p, void* stream);
bool kch_attend_tc5_enabled();
int kch_attend_tc5(const kch_attend_args* p, void* stream);

extern "C" int kch_attend(const kch_attend_args* p, void* stream) {
  KCH_REQUIRE(p != nullptr, "kch_attend: null args");
  KCH_REQUIRE(p->nh >= 1, "nh=%d must be >= 1", p->nh);
  KCH_REQUIRE(p->c >= 1 && p->c <= 256, "c=%d must be in [1, 256]", p->c);
  KCH_REQUIRE(p->sliding_window >= 0, "sliding_window=%d must be >= 0 (0 disables the branch)", p->sliding_window);
  KCH_REQUIRE(p->B >= 0 && p->T >= 0, "kch_attend: B=%d T=%d", p->B, p->T);
  KCH_REQUIRE(p->topk >= 0, "topk=%d must be >= 0", p->topk);
  KCH_REQUIRE(p->win_t0 >= 0, "win_t0=%d must be >= 0", p->win_t0);
  if ((p->comp_dtype == KCH_FP8_E4M3 || p->comp_dtype == KCH_INT8))
    KCH_REQUIRE(p->comp_scales && p->c % 64 == 0, "block-scaled 8-bit rows need scales and c %% 64 == 0 (c=%d)", p->c);
  if (p->B == 0 || p->T == 0) return KCH_OK;
  // tensor-core kernel for the production geometry; KCH_ATTEND=generic forces the fp32 CUDA-core kernel
  static const bool force_generic = [] { const char* e = getenv("KCH_ATTEND"); return e && e[0] == 'g'; }();
  if (!force_generic && kch_attend_mma_supported(p))
    return kch_attend_tc5_enabled() ? kch_attend_tc5(p, stream) : kch_attend_mma(p, stream);
  AttnArgs a;
  a.q = p->q; a.q_dtype = p->q_dtype; a.q_ld = p->q_ld; a.q_normalize = p->q_normalize;
  a.B = p->B; a.T = p->T; a.nh = p->nh; a.c = p->c;
  a.comp = p->comp; a.comp_dtype = p->comp_dtype; a.comp_ld = p->comp_ld; a.comp_batch_rows = p->comp_batch_rows;
  a.n_comp = p->comp ? p->n_comp : 0;
  a.comp_norms = p->comp_norms; a.comp_scales = p->comp_scales;
  a.sel = p->sel_indices; a.topk = p->sel_indices ? p->topk : 0;
  a.m = p->m; a.t0 = p->t0; a.nvis_fixed = p->n_visible;
  a.win_ptr = p->win; a.win_dtype = p->win_dtype; a.win_ld = p->win_ld; a.win_batch_rows = p->win_batch_rows;
  a.win_size = p->win ? p->sliding_window : 0; a.win_mode = p->win_mode; a.win_len = p->win_len;
  a.win_t0 = p->win_t0;
  a.sink = p->sink; a.sink_dtype = p->sink_dtype; a.scale = p->scale; a.out = p->out; a.out_dtype = p->out_dtype;
  int nw_max = !p->win ? 0 : (p->win_mode == 1 ? p->win_len : p->sliding_window);
  // maximum entry count over all queries bounds the shared-memory need
  int64_t ns_max;
  if (p->sel_indices) ns_max = p->topk;
  else if (p->n_visible >= 0) ns_max = p->n_visible < a.n_comp ? p->n_visible : a.n_comp;
  else if (p->m > 0) { int64_t v = (p->t0 + p->T) / p->m; ns_max = v < a.n_comp ? v : a.n_comp; }
  else ns_max = a.n_comp;
  int64_t E = ns_max + nw_max;
  int split = 256 / p->c > 0 ? 256 / p->c : 1;
  int HB = p->nh >= 16 ? 16 : p->nh >= 8 ? 8 : p->nh >= 4 ? 4 : p->nh >= 2 ? 2 : 1;
  size_t smem = ((size_t)p->nh * p->c + (size_t)(E > 0 ? E : 1) * p->nh + (size_t)split * HB * p->c) * sizeof(float);
  KCH_REQUIRE(smem <= 220 * 1024, "kch_attend: %lld entries x %d heads exceed the shared-memory budget of the generic kernel",
              (long long)E, p->nh);
  const AttnArgs& k = a;
  cudaStream_t s = kch_stream(stream);
  unsigned grid = (unsigned)((int64_t)p->B * p->T);
#define GO(HB_)                                                                                      \
  do {                                                                                               \
    KCH_CUDA_OK(cudaFuncSetAttribute(attn_generic_kernel<HB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    attn_generic_kernel<HB_><<<grid, 256, smem, s>>>(k);                                             \
  } while (0)
  switch (HB) { case 16: GO(16); break; case 8: GO(8); break; case 4: GO(4); break; case 2: GO(2); break; default: GO(1); }
#undef GO
  KCH_LAUNCH_OK();
  return KCH_OK;
}
