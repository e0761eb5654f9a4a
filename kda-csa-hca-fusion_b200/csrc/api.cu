// Error plumbing and dispatch shared by the C-ABI entry points.
#include <atomic>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "kch_common.cuh"

static thread_local char g_err[512] = "";

void kch_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<long long> g_launches{0};
void kch_note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long long kch_launch_count(int reset) {
  return reset ? g_launches.exchange(0) : g_launches.load();
}

extern "C" const char* kch_last_error(void) { return g_err; }
extern "C" int kch_abi_version(void) { return 1; }

int kch_linear_simt(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K,
                    int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype, void* stream);
bool kch_linear_tcgen05_supported(const void* A, const void* W, const void* C, const void* R, int64_t M, int N,
                                  int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype);
int kch_linear_tcgen05(const void* A, const void* W, void* C, const void* R, int64_t M, int N, int K, int64_t lda,
                       int64_t ldw, int64_t ldc, int64_t ldr, const kch_epilogue* e, void* stream, int slab_k = 0);
bool kch_linear_tcgen05_epilogue_ok(const kch_epilogue* e, int N);

extern "C" int kch_linear(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K,
                          int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype, void* stream) {
  return kch_linear_ex(A, W, C, residual, M, N, K, lda, ldw, ldc, ldr, dtype, nullptr, stream);
}

extern "C" int kch_linear_kslabs(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K,
                                 int n_slabs, int64_t ldw, int64_t ldc, int64_t ldr, int dtype, void* stream) {
  KCH_REQUIRE(M >= 0 && N >= 32 && K >= 1 && n_slabs >= 1, "kch_linear_kslabs: M=%lld N=%d K=%d n_slabs=%d",
              (long long)M, N, K, n_slabs);
  KCH_REQUIRE(dtype == KCH_BF16, "kch_linear_kslabs: bf16 only (dtype tag %d)", dtype);
  KCH_REQUIRE(K % n_slabs == 0 && (K / n_slabs) % 64 == 0,
              "kch_linear_kslabs: K=%d must split into n_slabs=%d slabs whose width is a multiple of 64", K, n_slabs);
  KCH_REQUIRE(ldw >= K && ldc >= N, "kch_linear_kslabs: leading dimensions ldw=%lld ldc=%lld too small", (long long)ldw,
              (long long)ldc);
  KCH_REQUIRE((int64_t)M * n_slabs <= 0x7FFFFFFFLL, "kch_linear_kslabs: M * n_slabs = %lld rows exceed the tensor-map range",
              (long long)M * n_slabs);
  if (M == 0) return KCH_OK;
  const int slab_k = K / n_slabs;
  KCH_REQUIRE(kch_linear_tcgen05_supported(A, W, C, residual, M, N, K, slab_k, ldw, ldc, ldr, dtype),
              "kch_linear_kslabs: operands must be 16-byte aligned with strides that are multiples of 8 elements");
  return kch_linear_tcgen05(A, W, C, residual, M, N, K, slab_k, ldw, ldc, ldr, nullptr, stream, n_slabs > 1 ? slab_k : 0);
}

extern "C" int kch_linear_ex(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K,
                             int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype, const kch_epilogue* ep,
                             void* stream) {
  KCH_REQUIRE(M >= 0 && N >= 0 && K >= 1, "kch_linear: M=%lld N=%d K=%d", (long long)M, N, K);
  KCH_REQUIRE(lda >= K && ldw >= K && ldc >= N, "kch_linear: leading dimensions lda=%lld ldw=%lld ldc=%lld too small",
              (long long)lda, (long long)ldw, (long long)ldc);
  KCH_REQUIRE(dtype == KCH_F32 || dtype == KCH_BF16, "kch_linear: unsupported dtype tag %d", dtype);
  if (M == 0 || N == 0) return KCH_OK;
  // CUDA-core kernel for fp32, for shapes the TMA descriptors cannot express, and for very narrow
  // outputs; KCH_LINEAR=simt forces it (a debugging aid: still a CUDA kernel, never a host path).
  static const bool force_simt = [] { const char* e = getenv("KCH_LINEAR"); return e && e[0] == 's'; }();
  if (ep && ep->n_segments) {
    KCH_REQUIRE(ep->n_segments <= 8, "kch_linear_ex: at most 8 epilogue segments (got %d)", ep->n_segments);
    KCH_REQUIRE(!residual, "kch_linear_ex: an activation epilogue and a residual cannot be combined");
    KCH_REQUIRE(ep->seg_end[ep->n_segments - 1] == N, "kch_linear_ex: the last segment must end at N=%d", N);
  }
  const bool tc = !force_simt && N >= 32 &&
                  kch_linear_tcgen05_supported(A, W, C, residual, M, N, K, lda, ldw, ldc, ldr, dtype);
  if (tc && kch_linear_tcgen05_epilogue_ok(ep, N))
    return kch_linear_tcgen05(A, W, C, residual, M, N, K, lda, ldw, ldc, ldr, ep, stream);
  int rc = tc ? kch_linear_tcgen05(A, W, C, residual, M, N, K, lda, ldw, ldc, ldr, nullptr, stream)
              : kch_linear_simt(A, W, C, residual, M, N, K, lda, ldw, ldc, ldr, dtype, stream);
  if (rc != KCH_OK || !ep || ep->n_segments == 0) return rc;
  // unfused epilogue: the same activations as separate in-place passes over the column segments
  const size_t es = dtype == KCH_BF16 ? 2 : 4;
  int start = 0;
  for (int i = 0; i < ep->n_segments; ++i) {
    const int end = ep->seg_end[i];
    KCH_REQUIRE(end > start && end <= N, "kch_linear_ex: segment %d ends at %d (previous end %d, N=%d)", i, end, start, N);
    if (ep->seg_act[i]) {
      void* p = (char*)C + (size_t)start * es;
      rc = kch_activation(p, p, M, end - start, ep->seg_act[i], ep->seg_param[i], ep->group, dtype, ldc, ldc, stream);
      if (rc != KCH_OK) return rc;
    }
    start = end;
  }
  return KCH_OK;
}
