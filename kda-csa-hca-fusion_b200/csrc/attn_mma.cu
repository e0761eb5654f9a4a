// Tensor-core path of the joint-softmax MQA core for the production geometry (c = 128, up to 16 heads,
// bf16 activations, cosine scoring): same mathematics as attn_core.cu.
//
// One warp owns one query position.  The 16 heads are the M=16 rows of mma.sync m16n8k16 tiles:
//   S[16 heads x 8 keys]  = Q[16 x 128] . X^T        (8 k-steps per 8 keys)
//   O[16 heads x 128]    += P[16 x 16 keys] . X      (values are the keys)
// The gathered key rows (selected compressed entries, or the dense visible prefix, then the window
// rows) are streamed L2 -> shared memory with 16-byte cp.async in a 2-stage ring of 32-row tiles, XOR
// swizzled so ldmatrix (plain for S, .trans for P.X) is conflict-free.  Because q and the keys are unit
// vectors, |s| <= |scale|, so the softmax uses the fixed shift max(|scale|, sink_h) instead of a running
// maximum; invalid slots get p = 0 and their rows are zero-filled.
// Bound: the gather, 256 B per (query, entry) out of L2; tensor work is 4*16*128 flop per entry.
#include <math.h>
#include <stdlib.h>

#include "kch_common.cuh"

#define AM_WARPS 4
#define AM_TILE 32
#define AM_C 128
#define AM_QLD 136   // padded row of the per-warp query tile (bf16 elements)

struct AttnMmaArgs {
  const bf16* q; int64_t q_ld;
  int B, T, nh;
  const bf16* comp; int64_t comp_batch_rows; int n_comp;
  const int32_t* sel; int topk;
  int m; int64_t t0; int nvis_fixed;
  const bf16* win; int64_t win_ld; int64_t win_batch_rows; int win_size; int win_t0;
  const void* sink; int sink_dtype;
  float scale;
  bf16* out;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int AM_STAGES, int MINB>
__global__ void __launch_bounds__(AM_WARPS * 32, MINB) attn_mma_kernel(AttnMmaArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t bt = (int64_t)blockIdx.x * AM_WARPS + warp;
  if (bt >= (int64_t)a.B * a.T) return;
  const int t = (int)(bt % a.T), b = (int)(bt / a.T);
  const int g = lane >> 2, j = lane & 3;
  // per-warp shared memory: the key ring; its last stage doubles as the query staging tile until the
  // query fragments are in registers (the prologue only fills stages 0 .. AM_STAGES-2)
  uint8_t* wbase = smem_raw + (size_t)warp * (AM_STAGES * AM_TILE * AM_C * 2);
  bf16* sq = reinterpret_cast<bf16*>(wbase + (AM_STAGES - 1) * AM_TILE * AM_C * 2);
  const uint32_t ring = smem_addr(wbase);
  // ---- entry list geometry ---------------------------------------------------------------
  int64_t nv64 = a.nvis_fixed >= 0 ? a.nvis_fixed : (a.m > 0 ? (a.t0 + t + 1) / a.m : a.n_comp);
  const int nvis = (int)(nv64 < a.n_comp ? nv64 : a.n_comp);
  const int ns = a.sel ? a.topk : nvis;
  int nw = 0, wrow0 = 0;
  if (a.win_size > 0 && a.win) { const int tw = t + a.win_t0; int lo = tw - a.win_size + 1; if (lo < 0) lo = 0; nw = tw - lo + 1; wrow0 = lo; }
  const int E = ns + nw;
  const int ntiles = (E + AM_TILE - 1) / AM_TILE;
  const int32_t* selrow = a.sel ? a.sel + bt * a.topk : nullptr;
  const bf16* comp_b = a.comp ? a.comp + (int64_t)b * a.comp_batch_rows * AM_C : nullptr;
  const bf16* win_b = a.win ? a.win + ((int64_t)b * a.win_batch_rows + wrow0) * a.win_ld : nullptr;

  // lane e of a tile resolves entry tile*32+e to a row pointer (nullptr = invalid -> zero fill)
  auto entry_ptr = [&](int e) -> const bf16* {
    if (e >= E) return nullptr;
    if (e < ns) {
      int id = selrow ? selrow[e] : e;
      if (id < 0 || id >= nvis) return nullptr;
      return comp_b + (int64_t)id * AM_C;
    }
    return win_b + (int64_t)(e - ns) * a.win_ld;
  };
  auto issue_tile = [&](int tile, uint32_t& valid_mask) {
    const bf16* p = entry_ptr(tile * AM_TILE + lane);
    valid_mask = __ballot_sync(0xffffffffu, p != nullptr);
    const uint32_t dst0 = ring + (uint32_t)(tile % AM_STAGES) * (AM_TILE * AM_C * 2);
    const int ch = lane & 15;
#pragma unroll
    for (int it = 0; it < AM_TILE / 2; ++it) {
      const int r = 2 * it + (lane >> 4);
      const bf16* rp = (const bf16*)__shfl_sync(0xffffffffu, (unsigned long long)p, r);
      const uint32_t dst = dst0 + r * (AM_C * 2) + ((ch ^ (r & 7)) << 4);
      cp_async16(dst, rp ? (const void*)(rp + ch * 8) : (const void*)a.q, rp ? 16 : 0);
    }
    cp_commit();
  };
  // ---- prologue: start the first tiles, then normalise the query while they fly -------------
  uint32_t vmask[AM_STAGES];
#pragma unroll
  for (int s = 0; s < AM_STAGES - 1; ++s) {
    if (s < ntiles) issue_tile(s, vmask[s]);
    else { vmask[s] = 0; cp_commit(); }
  }
  {
    const bf16* qrow = a.q + bt * a.q_ld;
    for (int h = 0; h < 16; ++h) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (h < a.nh) {
        uint2 raw = *reinterpret_cast<const uint2*>(qrow + h * AM_C + lane * 4);
        __nv_bfloat162 p0 = *reinterpret_cast<__nv_bfloat162*>(&raw.x), p1 = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
        v[0] = __bfloat162float(p0.x); v[1] = __bfloat162float(p0.y);
        v[2] = __bfloat162float(p1.x); v[3] = __bfloat162float(p1.y);
      }
      float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
      float nrm = fmaxf(sqrtf(ss), 1e-12f);
      uint2 o;
      o.x = pack_bf16(v[0] / nrm, v[1] / nrm);
      o.y = pack_bf16(v[2] / nrm, v[3] / nrm);
      *reinterpret_cast<uint2*>(sq + h * AM_QLD + lane * 4) = o;
    }
  }
  __syncwarp();
  uint32_t qa[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(sq + g * AM_QLD + 16 * ks + 2 * j);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(sq + (g + 8) * AM_QLD + 16 * ks + 2 * j);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(sq + g * AM_QLD + 16 * ks + 8 + 2 * j);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(sq + (g + 8) * AM_QLD + 16 * ks + 8 + 2 * j);
  }
  __syncwarp();
  // fixed softmax shift per head row (rows g and g+8 of this thread)
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

  for (int tile = 0; tile < ntiles; ++tile) {
    // keep AM_STAGES-1 tiles in flight
    {
      const int nt = tile + AM_STAGES - 1;
      uint32_t vm = 0;
      if (nt < ntiles) issue_tile(nt, vm); else cp_commit();
      vmask[nt % AM_STAGES] = vm;
    }
    cp_wait<AM_STAGES - 1>();
    __syncwarp();
    const uint32_t vm = vmask[tile % AM_STAGES];
    any_valid |= vm != 0;
    const uint32_t tb = ring + (uint32_t)(tile % AM_STAGES) * (AM_TILE * AM_C * 2);
    // ---- S = Q X^T for the 32 keys: 4 n-tiles of 8 keys --------------------------------------
    uint32_t pa[2][4];   // P as A fragments for the two 16-key k-steps of P.X
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const int krow = 8 * nt + (lane & 7);
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        const int ch = 4 * qd + (lane >> 3);
        uint32_t r0, r1, r2, r3;
        ldsm4(tb + krow * (AM_C * 2) + ((ch ^ (krow & 7)) << 4), r0, r1, r2, r3);
        mma16816(s, qa[2 * qd], r0, r1);
        mma16816(s, qa[2 * qd + 1], r2, r3);
      }
      // columns of this thread: keys 8nt + 2j, 8nt + 2j + 1
      const int k0 = 8 * nt + 2 * j;
      const bool v0 = (vm >> k0) & 1u, v1 = (vm >> (k0 + 1)) & 1u;
      float p00 = v0 ? __expf(s[0] * a.scale - shift0) : 0.f;
      float p01 = v1 ? __expf(s[1] * a.scale - shift0) : 0.f;
      float p10 = v0 ? __expf(s[2] * a.scale - shift1) : 0.f;
      float p11 = v1 ? __expf(s[3] * a.scale - shift1) : 0.f;
      l0 += p00 + p01;
      l1 += p10 + p11;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p00, p01);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p10, p11);
    }
    // ---- O += P X : 2 k-steps of 16 keys, 16 n-tiles of 8 channels ---------------------------
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const int krow = 16 * ks + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int ch = 2 * dp + (lane >> 4);
        uint32_t r0, r1, r2, r3;
        ldsm4t(tb + krow * (AM_C * 2) + ((ch ^ (krow & 7)) << 4), r0, r1, r2, r3);
        mma16816(o[2 * dp], pa[ks], r0, r1);
        mma16816(o[2 * dp + 1], pa[ks], r2, r3);
      }
    }
    __syncwarp();
  }
  cp_wait<0>();
  // ---- normalise and store ------------------------------------------------------------------
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (a.sink) { l0 += __expf(sink0 - shift0); l1 += __expf(sink1 - shift1); }
  const float inv0 = (any_valid && l0 > 0.f) ? 1.f / l0 : 0.f;
  const float inv1 = (any_valid && l1 > 0.f) ? 1.f / l1 : 0.f;
  bf16* orow = a.out + bt * ((int64_t)a.nh * AM_C);
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    const int d = 8 * n + 2 * j;
    if (g < a.nh) *reinterpret_cast<uint32_t*>(orow + g * AM_C + d) = pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
    if (g + 8 < a.nh) *reinterpret_cast<uint32_t*>(orow + (g + 8) * AM_C + d) = pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
  }
}

// Dense form (no selection list: every visible compressed block is attended, as in naive_hca): the AD_WARPS
// consecutive queries of a CTA see the same blocks (their visible counts differ by at most one step of the causal
// rule) and overlapping windows, so the CTA stages each key row ONCE in shared memory (16-byte cp.async by all
// threads, 3-stage ring of 32-row tiles, one block barrier per tile) and every warp scores it under its own
// validity mask.  Per-warp arithmetic is that of attn_mma_kernel; the L2 -> shared traffic per query drops by the
// number of warps.  Entry list of the CTA: blocks [0, nvis(last query)), then window rows
// [first query's window start, last query's position].
#define AD_WARPS 8
#define AD_STAGES 3

__global__ void __launch_bounds__(AD_WARPS * 32, 2) attn_dense_mma_kernel(AttnMmaArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int tiles_per_seq = (a.T + AD_WARPS - 1) / AD_WARPS;
  const int b = blockIdx.x / tiles_per_seq;
  const int tq0 = (blockIdx.x % tiles_per_seq) * AD_WARPS;
  const int t = tq0 + warp;
  const bool active = t < a.T;
  const int t_last = min(tq0 + AD_WARPS, a.T) - 1;
  const int64_t bt = (int64_t)b * a.T + t;
  const int g = lane >> 2, j = lane & 3;
  uint8_t* ringp = smem_raw;
  bf16* sq = reinterpret_cast<bf16*>(smem_raw + AD_STAGES * AM_TILE * AM_C * 2) + warp * (16 * AM_QLD);
  const uint32_t ring = smem_addr(ringp);
  auto nvis_of = [&](int tt) -> int {
    int64_t nv64 = a.nvis_fixed >= 0 ? a.nvis_fixed : (a.m > 0 ? (a.t0 + tt + 1) / a.m : a.n_comp);
    return (int)(nv64 < a.n_comp ? nv64 : a.n_comp);
  };
  const int nvis = active ? nvis_of(t) : 0;
  const int ns = a.comp ? nvis_of(t_last) : 0;                   // blocks staged for the CTA
  int nw = 0, wrow0 = 0;                                          // window rows staged for the CTA: [wrow0, wrow0 + nw)
  const bool has_win = a.win_size > 0 && a.win;
  if (has_win) { int lo = tq0 + a.win_t0 - a.win_size + 1; if (lo < 0) lo = 0; wrow0 = lo; nw = t_last + a.win_t0 - lo + 1; }
  const int tw = t + a.win_t0;                                    // this query's own window: rows [tw - win + 1, tw]
  const int E = ns + nw;
  const int ntiles = (E + AM_TILE - 1) / AM_TILE;
  const bf16* comp_b = a.comp ? a.comp + (int64_t)b * a.comp_batch_rows * AM_C : nullptr;
  const bf16* win_b = has_win ? a.win + ((int64_t)b * a.win_batch_rows + wrow0) * a.win_ld : nullptr;

  auto issue_tile = [&](int tile) {
    const uint32_t dst0 = ring + (uint32_t)(tile % AD_STAGES) * (AM_TILE * AM_C * 2);
#pragma unroll
    for (int it = 0; it < (AM_TILE * 16) / (AD_WARPS * 32); ++it) {
      const int idx = tid + it * (AD_WARPS * 32), r = idx >> 4, ch = idx & 15;
      const int e = tile * AM_TILE + r;
      const bf16* rp = nullptr;
      if (e < ns) rp = comp_b + (int64_t)e * AM_C;
      else if (e < E) rp = win_b + (int64_t)(e - ns) * a.win_ld;
      const uint32_t dst = dst0 + r * (AM_C * 2) + ((ch ^ (r & 7)) << 4);
      cp_async16(dst, rp ? (const void*)(rp + ch * 8) : (const void*)a.q, rp ? 16 : 0);
    }
    cp_commit();
  };
  // validity of entry tile*32 + lane for THIS warp's query
  auto valid_mask = [&](int tile) -> uint32_t {
    const int e = tile * AM_TILE + lane;
    bool ok = false;
    if (active) {
      if (e < ns) ok = e < nvis;
      else if (e < E) { const int r = wrow0 + (e - ns); ok = r <= tw && r > tw - a.win_size; }
    }
    return __ballot_sync(0xffffffffu, ok);
  };
#pragma unroll
  for (int s = 0; s < AD_STAGES - 1; ++s) {
    if (s < ntiles) issue_tile(s); else cp_commit();
  }
  // normalised query of this warp -> A fragments
  {
    const bf16* qrow = a.q + (active ? bt : (int64_t)b * a.T) * a.q_ld;
    for (int h = 0; h < 16; ++h) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (h < a.nh && active) {
        uint2 raw = *reinterpret_cast<const uint2*>(qrow + h * AM_C + lane * 4);
        __nv_bfloat162 p0 = *reinterpret_cast<__nv_bfloat162*>(&raw.x), p1 = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
        v[0] = __bfloat162float(p0.x); v[1] = __bfloat162float(p0.y);
        v[2] = __bfloat162float(p1.x); v[3] = __bfloat162float(p1.y);
      }
      float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
      float nrm = fmaxf(sqrtf(ss), 1e-12f);
      uint2 o;
      o.x = pack_bf16(v[0] / nrm, v[1] / nrm);
      o.y = pack_bf16(v[2] / nrm, v[3] / nrm);
      *reinterpret_cast<uint2*>(sq + h * AM_QLD + lane * 4) = o;
    }
  }
  __syncwarp();
  uint32_t qa[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(sq + g * AM_QLD + 16 * ks + 2 * j);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(sq + (g + 8) * AM_QLD + 16 * ks + 2 * j);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(sq + g * AM_QLD + 16 * ks + 8 + 2 * j);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(sq + (g + 8) * AM_QLD + 16 * ks + 8 + 2 * j);
  }
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

  for (int tile = 0; tile < ntiles; ++tile) {
    cp_wait<AD_STAGES - 2>();                      // this thread's copies of `tile` have landed ...
    __syncthreads();                               // ... and everybody's; all warps are done with tile - 1
    if (tile + AD_STAGES - 1 < ntiles) issue_tile(tile + AD_STAGES - 1); else cp_commit();
    const uint32_t vm = valid_mask(tile);
    if (vm == 0) continue;                         // nothing of this tile is visible to this warp's query
    any_valid = true;
    const uint32_t tb = ring + (uint32_t)(tile % AD_STAGES) * (AM_TILE * AM_C * 2);
    uint32_t pa[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const int krow = 8 * nt + (lane & 7);
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        const int ch = 4 * qd + (lane >> 3);
        uint32_t r0, r1, r2, r3;
        ldsm4(tb + krow * (AM_C * 2) + ((ch ^ (krow & 7)) << 4), r0, r1, r2, r3);
        mma16816(s, qa[2 * qd], r0, r1);
        mma16816(s, qa[2 * qd + 1], r2, r3);
      }
      const int k0 = 8 * nt + 2 * j;
      const bool v0 = (vm >> k0) & 1u, v1 = (vm >> (k0 + 1)) & 1u;
      float p00 = v0 ? __expf(s[0] * a.scale - shift0) : 0.f;
      float p01 = v1 ? __expf(s[1] * a.scale - shift0) : 0.f;
      float p10 = v0 ? __expf(s[2] * a.scale - shift1) : 0.f;
      float p11 = v1 ? __expf(s[3] * a.scale - shift1) : 0.f;
      l0 += p00 + p01;
      l1 += p10 + p11;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p00, p01);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p10, p11);
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const int krow = 16 * ks + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int ch = 2 * dp + (lane >> 4);
        uint32_t r0, r1, r2, r3;
        ldsm4t(tb + krow * (AM_C * 2) + ((ch ^ (krow & 7)) << 4), r0, r1, r2, r3);
        mma16816(o[2 * dp], pa[ks], r0, r1);
        mma16816(o[2 * dp + 1], pa[ks], r2, r3);
      }
    }
  }
  cp_wait<0>();
  if (!active) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (a.sink) { l0 += __expf(sink0 - shift0); l1 += __expf(sink1 - shift1); }
  const float inv0 = (any_valid && l0 > 0.f) ? 1.f / l0 : 0.f;
  const float inv1 = (any_valid && l1 > 0.f) ? 1.f / l1 : 0.f;
  bf16* orow = a.out + bt * ((int64_t)a.nh * AM_C);
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    const int d = 8 * n + 2 * j;
    if (g < a.nh) *reinterpret_cast<uint32_t*>(orow + g * AM_C + d) = pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
    if (g + 8 < a.nh) *reinterpret_cast<uint32_t*>(orow + (g + 8) * AM_C + d) = pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
  }
}

int kch_attend_dense_tc5(const bf16* q, int64_t q_ld, int B, int T, int nh, const bf16* comp, int64_t comp_batch_rows,
                         int n_comp, int m, int64_t t0, int nvis_fixed, const bf16* win, int64_t win_ld,
                         int64_t win_batch_rows, int win_size, int win_t0, const void* sink, int sink_dtype, float scale,
                         bf16* out, cudaStream_t s);

bool kch_attend_mma_supported(const kch_attend_args* p) {
  if (p->c != AM_C || p->nh > 16 || p->nh < 1) return false;
  if (p->q_dtype != KCH_BF16 || p->out_dtype != KCH_BF16 || !p->q_normalize) return false;
  if (p->comp && (p->comp_dtype != KCH_BF16 || p->comp_norms || p->comp_scales || p->comp_ld != AM_C)) return false;
  if (p->win && p->sliding_window > 0 && (p->win_dtype != KCH_BF16 || p->win_mode != 0 || (p->win_ld % 8) != 0)) return false;
  if (!(fabsf(p->scale) <= 16.f)) return false;
  if ((p->q_ld % 4) != 0 || ((uintptr_t)p->q & 7)) return false;
  if (p->comp && ((uintptr_t)p->comp & 15)) return false;
  if (p->win && ((uintptr_t)p->win & 15)) return false;
  return true;
}

int kch_attend_mma(const kch_attend_args* p, void* stream) {
  AttnMmaArgs a;
  a.q = (const bf16*)p->q; a.q_ld = p->q_ld;
  a.B = p->B; a.T = p->T; a.nh = p->nh;
  a.comp = (const bf16*)p->comp; a.comp_batch_rows = p->comp_batch_rows; a.n_comp = p->comp ? p->n_comp : 0;
  a.sel = p->sel_indices; a.topk = p->sel_indices ? p->topk : 0;
  a.m = p->m; a.t0 = p->t0; a.nvis_fixed = p->n_visible;
  const bool has_win = p->win && p->sliding_window > 0;
  a.win = has_win ? (const bf16*)p->win : nullptr; a.win_ld = p->win_ld; a.win_batch_rows = p->win_batch_rows;
  a.win_size = has_win ? p->sliding_window : 0; a.win_t0 = p->win_t0;
  a.sink = p->sink; a.sink_dtype = p->sink_dtype; a.scale = p->scale; a.out = (bf16*)p->out;
  static_assert(16 * AM_QLD * 2 <= AM_TILE * AM_C * 2, "query staging tile must fit one ring stage");
  // no selection list: the queries of a CTA share their staged keys (KCH_ATTEND_DENSE=w keeps one ring per warp)
  static const bool dense_per_warp = [] { const char* e = getenv("KCH_ATTEND_DENSE"); return e && e[0] == 'w'; }();
  // ... and on tcgen05 where nothing is gathered at all (KCH_ATTEND_DENSE=m keeps the mma.sync shared-ring kernel)
  static const bool dense_mma = [] { const char* e = getenv("KCH_ATTEND_DENSE"); return e && e[0] == 'm'; }();
  if (!a.sel && !dense_per_warp && !dense_mma) {
    const int rc = kch_attend_dense_tc5(a.q, a.q_ld, a.B, a.T, a.nh, a.comp, a.comp_batch_rows, a.n_comp, a.m, a.t0, a.nvis_fixed,
                                        a.win, a.win_ld, a.win_batch_rows, a.win_size, a.win_t0, a.sink, a.sink_dtype, a.scale,
                                        a.out, kch_stream(stream));
    if (rc != -100) return rc;
  }
  if (!a.sel && !dense_per_warp) {
    const size_t smem = (size_t)AD_STAGES * AM_TILE * AM_C * 2 + (size_t)AD_WARPS * 16 * AM_QLD * 2;
    KCH_CUDA_OK(cudaFuncSetAttribute(attn_dense_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t ctas = (int64_t)p->B * ((p->T + AD_WARPS - 1) / AD_WARPS);
    attn_dense_mma_kernel<<<(unsigned)ctas, AD_WARPS * 32, smem, kch_stream(stream)>>>(a);
    KCH_LAUNCH_OK();
    return KCH_OK;
  }
  int64_t nq = (int64_t)p->B * p->T;
  unsigned grid = (unsigned)((nq + AM_WARPS - 1) / AM_WARPS);
  // ring depth / resident CTAs per SM: two stages and three CTAs per SM (168 registers) measured fastest on
  // B200 (7.1 ms vs 8.0 ms for three stages / two CTAs at the benchmark size); KCH_ATTN_CFG = 0 | 2 selects
  // (3 stages, 2 CTAs) | (2 stages, 4 CTAs) for experiments
  static const int cfg = [] { const char* e = getenv("KCH_ATTN_CFG"); return e ? atoi(e) : 1; }();
#define AM_GO(ST, MB)                                                                                          \
  do {                                                                                                         \
    size_t smem = (size_t)AM_WARPS * (ST * AM_TILE * AM_C * 2);                                                \
    KCH_CUDA_OK(cudaFuncSetAttribute(attn_mma_kernel<ST, MB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    attn_mma_kernel<ST, MB><<<grid, AM_WARPS * 32, smem, kch_stream(stream)>>>(a);                             \
  } while (0)
  if (cfg == 1) AM_GO(2, 3);
  else if (cfg == 2) AM_GO(2, 4);
  else AM_GO(3, 2);
#undef AM_GO
  KCH_LAUNCH_OK();
  return KCH_OK;
}
