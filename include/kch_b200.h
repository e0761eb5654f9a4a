/* kch_b200 — C ABI of the B200 (sm_100a) kernels for the forward path of the KDA + CSA + HCA
 * hybrid attention stack of 183600/kda-csa-hca-fusion.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless stated otherwise; the library never allocates or
 *    frees device memory (except kch_*_workspace_bytes helpers, which only compute sizes) and keeps
 *    no state between calls other than a cache of TMA descriptors and one device status word.
 *  - `stream` is a cudaStream_t passed as void*.  Calls are asynchronous on that stream.
 *  - dtype tags: KCH_F32, KCH_BF16 for activations / weights; KCH_FP8_E4M3, KCH_INT8 only for
 *    block-scaled compressed rows (one fp32 scale per 64 elements).
 *  - Return value: KCH_OK (0); KCH_ERR_INVALID (<0) for a rejected argument — the message
 *    (kch_last_error) names the offending parameter the way the reference's ValueError does;
 *    KCH_ERR_CUDA (>0) for a CUDA failure.  Device-side bounded waits that expire set a status word
 *    readable with kch_device_status.
 *  - Reference citations are file:line inside the reference project.
 */
#ifndef KCH_B200_H
#define KCH_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KCH_OK 0
#define KCH_ERR_INVALID (-1)
#define KCH_ERR_CUDA 1

#define KCH_F32 0
#define KCH_BF16 1
#define KCH_FP8_E4M3 2
#define KCH_INT8 3

#define KCH_ACT_SILU 1
#define KCH_ACT_SIGMOID 2
#define KCH_ACT_NEG_SOFTPLUS 3
#define KCH_ACT_SILU_L2NORM 4

/* Library / error plumbing. */
int kch_abi_version(void);
const char* kch_last_error(void);           /* host string, thread-local, valid until the next call */
unsigned int kch_device_status(int reset);  /* synchronising read of the device status word (0 = clean) */
long long kch_launch_count(int reset);      /* kernels launched by this library in this process so far */

/* Self-test of the failure path that replaces a hang: one CTA waits with the library's bounded mbarrier wait on a
 * barrier nothing arrives at, gives up after `limit_polls` (1 .. 2^20) polls, records KCH_STATUS_SELFTEST_WAIT in the
 * status word and returns; `polls_out` (device, optional) receives the number of polls spent.  Afterwards
 * kch_device_status(1) reports and clears the code.  While the word is set every other bounded wait of the library
 * returns at its first poll, so read and clear it before launching real work.  No counterpart in the reference
 * (it has no device code): its nearest relative is the non-finite-output warning, ops_kda.py:151-172. */
#define KCH_STATUS_SELFTEST_WAIT 0x5E1F
#define KCH_STATUS_GEMM_DECODE 0x6D01   /* status word: a wait of the decode-batch GEMM (operands / accumulator) expired */
#define KCH_STATUS_KDA_STEP 0x6D03       /* status word: the state copy of the one-token KDA step did not arrive */
#define KCH_STATUS_INDEXER_DECODE 0x6D02 /* status word: a wait of the one-token indexer (key tiles / accumulator) expired */
int kch_selftest_bounded_wait(unsigned int limit_polls, unsigned int* polls_out, void* stream);

/* ---- layer glue ---------------------------------------------------------------------------- */

/* _Fp32LayerNorm.forward, ops_fused.py:52-60: LayerNorm in fp32, stored in `dtype`. x,y [rows,d]. */
int kch_layernorm(const void* x, const void* weight, const void* bias, void* y, int64_t rows, int d,
                  float eps, int dtype, int wdtype, void* stream);

/* KDAHybridLayer short conv, ops_fused.py:505-527: causal depthwise kernel-3 convolution + bias.
 * x,y [B,T,d]; lookback [B,2,d] or NULL (zeros); weight [d,3]; bias [d]; all in `dtype`. */
int kch_short_conv(const void* x, const void* lookback, const void* weight, const void* bias, void* y,
                   int B, int T, int d, int dtype, void* stream);
/* LayerNorm (fp32 arithmetic, rounded to bf16) followed by the short convolution in one pass; bf16 only,
 * d a multiple of 256 up to 2048, T >= 2.  Same values as kch_layernorm then kch_short_conv.  `lookback` /
 * `lookback_out` [B,2,d] hold NORMALISED rows (what the convolution consumes); lookback_out receives the last
 * two normalised rows of the sequence.  ln_weight / ln_bias in wdtype, conv operands in bf16. */
int kch_layernorm_short_conv(const void* x, const void* ln_weight, const void* ln_bias, float eps,
                             const void* lookback, const void* conv_weight, const void* conv_bias, void* y,
                             void* lookback_out, int B, int T, int d, int dtype, int wdtype, void* stream);

/* One-token step of the same convolution (x,y [B,1,d]) that also slides `lookback` [B,2,d] by one token in
 * place: lookback <- [lookback[:,1], x] (the concatenation of ops_fused.py:560-569 without a new tensor). */
int kch_short_conv_step(const void* x, void* lookback, const void* weight, const void* bias, void* y, int B, int d,
                        int dtype, void* stream);

/* LayerNorm (ops_fused.py:52-60) and that one-token step in one launch, for the decode step of a KDA sub-layer:
 * x [B,1,d] is the un-normalised residual stream, `lookback` [B,2,d] holds NORMALISED rows and slides in place.
 * bf16, d % 256 == 0, d <= 2048; same rounding points as kch_layernorm followed by kch_short_conv_step. */
int kch_layernorm_short_conv_step(const void* x, const void* ln_weight, const void* ln_bias, float eps,
                                  void* lookback, const void* conv_weight, const void* conv_bias, void* y,
                                  int B, int d, int dtype, int wdtype, void* stream);

/* F.linear at ops_fused.py:571-581,609,713,739 and ops_csa.py:841-878, ops_hca.py:132-141:
 * C[M,N] = A[M,K] . W[N,K]^T, fp32 accumulation, rounded to `dtype`; if `residual` is given the
 * rounded product is added to it in fp32 and rounded again (x = residual + proj, ops_fused.py:1091).
 * Leading dimensions are in elements.  bf16 with K,lda,ldw multiples of 8 runs on tcgen05 tensor
 * cores; everything else on CUDA cores. */
int kch_linear(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K,
               int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype, void* stream);

/* kch_linear with activations fused into the store (ops_fused.py:571-581 applied to the fused q|k|v|g_down|beta
 * projection): columns [seg_end[s-1], seg_end[s]) get activation seg_act[s] (0 = none, else KCH_ACT_*),
 * with seg_param[s] (decay scale) and `group` (head width of KCH_ACT_SILU_L2NORM).  Rounding points are
 * those of the unfused chain.  Runs inside the tcgen05 epilogue when the segment boundaries allow it (with
 * fast exp/reciprocal intrinsics: at most one bf16 rounding away from the unfused chain), otherwise as
 * separate in-place passes.  Not combinable with `residual`. */
typedef struct kch_epilogue {
  int n_segments;      /* <= 8 */
  int seg_end[8];
  int seg_act[8];
  float seg_param[8];
  int group;
} kch_epilogue;
int kch_linear_ex(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K,
                  int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int dtype, const kch_epilogue* epilogue,
                  void* stream);

/* The output projection after an all-gather of per-GPU head slices (no counterpart in the reference, which has no
 * distributed code; mathematically F.linear(concat_heads(A), W), ops_fused.py:609/713/739): A holds the K input
 * columns as `n_slabs` slabs [n_slabs][M][K / n_slabs] one after the other -- the rank-major buffer ncclAllGather
 * leaves behind -- and the K loop walks the slabs, so the gathered tensor is never re-laid out.  bf16 only; the slab
 * width must be a multiple of 64.  C[M, N] = A_cat[M, K] W[N, K]^T (+ residual). */
int kch_linear_kslabs(const void* A, const void* W, void* C, const void* residual, int64_t M, int N, int K, int n_slabs,
                      int64_t ldw, int64_t ldc, int64_t ldr, int dtype, void* stream);

/* All-gather of per-GPU slabs by plain peer stores (no counterpart in the reference, which has no
 * distributed code): rank `rank` of `world` writes `slab_bytes` from `src` into slot `rank` of every rank's gather
 * buffer and the ranks meet on arrival / data flags next to the buffers (bounded waits; a wait that runs out records
 * KCH_STATUS_PEER_GATHER in the status word and the kernel returns).  `bufs[p]` / `flags[p]` (HOST arrays of `world`
 * device pointers) are rank p's buffer ([world][slab_bytes]) and flag block (kch_peer_gather_flag_words(world) zeroed
 * 32-bit words) as mapped on this GPU: memory every rank has mapped from every peer (CUDA VMM / IPC).  The call counter
 * lives in the flag block, so a captured CUDA graph replays it unchanged.  All ranks must make the
 * same sequence of calls on a buffer.  slab_bytes: multiple of 16; up to 1 MiB runs as one launch of one CTA, larger slabs as
 * three launches (arrival, a copy kernel over all SMs, data flags). */
#define KCH_STATUS_PEER_GATHER 0x9A7E
int64_t kch_peer_gather_flag_words(int world);
int kch_peer_allgather(const void* src, int64_t slab_bytes, void* const* bufs, void* const* flags, int rank, int world,
                       void* stream);

/* Activation epilogues with the reference's rounding points, ops_fused.py:571-581.
 * x,y [rows,cols] in `dtype`, rows ldx / ldy elements apart (x may be a column slice of a fused
 * projection); `param` is the decay scale for KCH_ACT_NEG_SOFTPLUS; `group` is the head width for
 * KCH_ACT_SILU_L2NORM. */
int kch_activation(const void* x, void* y, int64_t rows, int cols, int act, float param, int group,
                   int dtype, int64_t ldx, int64_t ldy, void* stream);

/* F.normalize(x.float(), dim=-1), ops_csa.py:927-936,1110-1113, ops_hca.py:135,141,155:
 * y[rows,c] = x / max(||x||,1e-12) evaluated in fp32 and stored as out_dtype (fp32, or bf16 for the
 * tensor-core attention path); x rows are `ld` elements apart.  `norms` (optional) receives the
 * clamped norms; y may be NULL. */
int kch_rownorm(const void* x, int64_t ld, void* y, float* norms, int64_t rows, int c, int dtype,
                int out_dtype, void* stream);

/* ---- KDA ----------------------------------------------------------------------------------- */

/* naive_recurrent_kda, ops_kda.py:175-267.  q,k [B,T,H,K]; v [B,T,HV,V]; g [B,T,HV,K];
 * beta [B,T,HV]; all `dtype`.  Heads are dense within a token; consecutive tokens are ld_qk / ld_v / ld_g /
 * ld_beta elements apart (0 = contiguous), so q, k, v, beta may be column slices of one fused projection.
 * initial_state / final_state fp32 [B,HV,K,V] (either may be NULL).  o [B,T,HV,V] contiguous in `dtype`.
 * g is clamped below at g_clamp_min (pass -INFINITY to disable). */
int kch_kda_recurrent(const void* q, const void* k, const void* v, const void* g, const void* beta,
                      const float* initial_state, void* o, float* final_state, int B, int T, int H,
                      int HV, int K, int V, float scale, float g_clamp_min, int dtype, int64_t ld_qk,
                      int64_t ld_v, int64_t ld_g, int64_t ld_beta, void* stream);

/* naive_chunk_kda, ops_kda.py:340-536 (prepare 375-424, chain 509-535, finalize 440-461).  Same
 * tensors as above.  Needs a workspace of kch_kda_chunk_workspace_bytes(...) bytes. */
int64_t kch_kda_chunk_workspace_bytes(int B, int T, int HV, int K, int V, int chunk_size);
int kch_kda_chunk(const void* q, const void* k, const void* v, const void* g, const void* beta,
                  const float* initial_state, void* o, float* final_state, int B, int T, int H, int HV,
                  int K, int V, int chunk_size, float scale, float g_clamp_min, int dtype, int64_t ld_qk,
                  int64_t ld_v, int64_t ld_g, int64_t ld_beta, void* workspace, int64_t workspace_bytes,
                  void* stream);

/* The same operator fed with the PRE-activation of the gate: g_pre is the output of g_up, and the decay is
 * g = round(-round(softplus(g_pre)) * gate_scale) evaluated on load with the layer's bf16 rounding points
 * (KDAHybridLayer, ops_fused.py:575-578), which saves the activation pass over [B,T,HV,K].  Tensor-core path only:
 * bf16, K = V = 128, chunk_size 64, g_clamp_min >= -10 (kch_kda_chunk_gate_supported tells). */
int kch_kda_chunk_gate_supported(int K, int V, int chunk_size, float g_clamp_min, int dtype);
int kch_kda_chunk_gate(const void* q, const void* k, const void* v, const void* g_pre, const void* beta,
                       const float* initial_state, void* o, float* final_state, int B, int T, int H, int HV,
                       int K, int V, int chunk_size, float scale, float g_clamp_min, float gate_scale, int dtype,
                       int64_t ld_qk, int64_t ld_v, int64_t ld_g, int64_t ld_beta, void* workspace,
                       int64_t workspace_bytes, void* stream);

/* ---- compression ------------------------------------------------------------------------------ */

/* csa_compress_kv, ops_csa.py:198-234.  C,Z: rows of c elements, `ld` apart, batch b starts at row
 * b*batch_stride_rows; B_pos [m,c]; out fp32, batch b at element b*out_batch_stride_elems. */
int kch_compress_kv(const void* C, const void* Z, const void* B_pos, float* out, int B, int64_t T, int c,
                    int m, int64_t ld, int64_t batch_stride_rows, int64_t out_batch_stride_elems,
                    int dtype, int bias_dtype, void* stream);

/* csa_compress_kv_overlapped, ops_csa.py:237-305.  prev_Cb/prev_Zb [B,m,c] (rows prev_ld apart)
 * supply the b-branch of the block preceding block 0 (NULL: none, as at the sequence start), which
 * is how _csa_compress_kv_overlapped_single (ops_decoding_cache.py:128-195) continues a stream. */
int kch_compress_kv_overlapped(const void* Ca, const void* Cb, const void* Za, const void* Zb,
                               const void* Ba, const void* Bb, const void* prev_Cb, const void* prev_Zb,
                               int64_t prev_ld, float* out, int B, int64_t T, int c, int m, int64_t ld,
                               int64_t batch_stride_rows, int64_t out_batch_stride_elems, int dtype,
                               int bias_dtype, void* stream);

/* ---- lightning indexer + top-k ------------------------------------------------------------------ */

/* csa_lightning_indexer, ops_csa.py:330-573 (scores 529-536, top-k 550-554).
 * q_idx fp32 [B,T,HI,DI], k_idx fp32 [B,n_blocks,DI] (both already normalised when cosine scoring is
 * on), w_idx fp32 [B,T,HI] or NULL.  Block n is visible to query row t iff n < (t0+t+1)/m, or iff
 * n < n_visible when n_visible >= 0 (m <= 0 and n_visible < 0: everything visible).
 * indices int32 [B,T,topk], -1 padded; ties go to the lower block index; `sorted` orders the picks
 * by descending logit as torch.topk does.  k_batch_stride: elements between the key blocks of
 * consecutive batch entries (0 = n_blocks*DI).  Workspace: kch_indexer_workspace_bytes. */
int64_t kch_indexer_workspace_bytes(int B, int T, int n_blocks, int HI, int DI);
int kch_indexer_topk(const float* q_idx, const float* k_idx, const float* w_idx, int32_t* indices, int B,
                     int T, int n_blocks, int HI, int DI, int topk, float scale, int m, int64_t t0,
                     int n_visible, int sorted, int64_t k_batch_stride, void* workspace,
                     int64_t workspace_bytes, void* stream);
/* Same selection with the queries read as the projection wrote them: q_idx [B,T,HI*DI] in q_dtype, tokens q_ld
 * elements apart.  KCH_BF16 (needs DI == 64): the un-normalised bf16 queries are exact tensor-core operands and,
 * with q_normalize, each head's dot products are divided by max(||q_h||, 1e-12) (the reference normalises the
 * query first, ops_csa.py:531-536: the same value up to one rounding).  KCH_F32: identical to kch_indexer_topk.
 * Workspace: kch_indexer_workspace_bytes_ex(B, T, n_blocks, q_dtype). */
int64_t kch_indexer_workspace_bytes_ex(int B, int T, int n_blocks, int q_dtype);
int kch_indexer_topk_ex(const void* q_idx, int q_dtype, int64_t q_ld, int q_normalize, const float* k_idx,
                        const float* w_idx, int32_t* indices, int B, int T, int n_blocks, int HI, int DI, int topk,
                        float scale, int m, int64_t t0, int n_visible, int sorted, int64_t k_batch_stride,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* No counterpart in the reference (it allocates freely through PyTorch).  Same selection as
 * kch_indexer_topk (unsorted picks), for callers that must not allocate device memory while serving:
 * the logits live in a 16 MiB array built into the library instead of a caller workspace.  Limit:
 * B*T*round_up(n_blocks,4) <= kch_indexer_topk_static_capacity() (4 Mi fp32); larger requests are
 * rejected.  The first call on each device resolves the array's device address (make it before any
 * stream capture); calls on one device share the array, so calls that overlap on the GPU race. */
int64_t kch_indexer_topk_static_capacity(void);
int kch_indexer_topk_static(const float* q_idx, const float* k_idx, const float* w_idx, int32_t* indices,
                            int B, int T, int n_blocks, int HI, int DI, int topk, float scale, int m,
                            int64_t t0, int n_visible, int64_t k_batch_stride, void* stream);

/* ---- attention core ------------------------------------------------------------------------------- */

/* Joint-softmax MQA over [selected | all visible] compressed entries and the sliding window, with
 * the sink logit in the denominator: naive_csa ops_csa.py:923-1155, naive_hca ops_hca.py:139-192,
 * CSADecodingCache.forward_step ops_decoding_cache.py:891-1070, HCADecodingCache.forward_step
 * 1318-1395. */
typedef struct kch_attend_args {
  const void* q;            /* [B*T, nh*c] rows q_ld apart, q_dtype */
  int q_dtype;
  int64_t q_ld;
  int q_normalize;          /* 1: L2-normalise each head's query in fp32 first */
  int B, T, nh, c;
  const void* comp;         /* compressed rows, comp_ld elements apart; batch b starts at row b*comp_batch_rows */
  int comp_dtype;           /* KCH_F32 / KCH_BF16 / KCH_FP8_E4M3 / KCH_INT8 */
  int64_t comp_ld;
  int64_t comp_batch_rows;
  int n_comp;               /* rows per batch element */
  const float* comp_norms;  /* optional per-row divisor (same row indexing as comp) */
  const float* comp_scales; /* [rows, c/64] for the 8-bit kinds */
  const int32_t* sel_indices; /* [B,T,topk] or NULL = dense over every visible row (HCA) */
  int topk;
  int m;                    /* visibility: row n visible to query t iff n < (t0+t+1)/m ... */
  int64_t t0;
  int n_visible;            /* ... or n < n_visible when >= 0 */
  const void* win;          /* window keys; NULL or sliding_window 0 disables */
  int win_dtype;
  int64_t win_ld;
  int64_t win_batch_rows;
  int sliding_window;
  int win_mode;             /* 0: row s of `win` is position s of the sequence; 1: ring buffer, rows 0..win_len-1 all valid */
  int win_len;
  const void* sink;         /* [nh] or NULL */
  int sink_dtype;
  float scale;
  void* out;                /* [B,T,nh*c] */
  int out_dtype;
  int win_t0;               /* win_mode 0: query t sits at row t + win_t0 of `win` (rows before it: earlier tokens,
                             * e.g. the tail of a cache's ring when a later chunk of a sequence is attended) */
} kch_attend_args;
int kch_attend(const kch_attend_args* args, void* stream);

/* ---- decode caches ---------------------------------------------------------------------------------- */

/* Device-resident mirror of a decode cache's counters (int32[8]; no counterpart in the reference, whose
 * counters are Python ints): with it a decode step has no host-side arguments that change from token to
 * token, so the whole step can be replayed from a CUDA graph.  kch_cache_advance applies the same update
 * the host makes after an append (ops_decoding_cache.py:764-779). */
#define KCH_CTR_ACC_LEN 0   /* tokens in the open block */
#define KCH_CTR_N_BLOCKS 1  /* completed compressed rows */
#define KCH_CTR_RING_N 2    /* tokens ever written to the window ring */
#define KCH_CTR_HAS_PREV 3  /* CSA: a previous block's b-branch is held */
#define KCH_CTR_TOKENS 4    /* tokens seen */
#define KCH_CTR_ARRIVALS 5  /* CTAs of a fused append that have finished (kch_cache_append_token_advance) */
#define KCH_CTR_WORDS 8
#define KCH_STATUS_CACHE_CAPACITY 64  /* device status: an append found its counters out of range / storage full */
int kch_cache_advance(int32_t* counters, int m, void* stream);

/* One appended token for every sequence of the batch: CSADecodingCache.append_step
 * (ops_decoding_cache.py:704-779) when Cb/Zb/K_idx/Z_idx are given, HCADecodingCache.append_step
 * (1238-1264) when they are NULL.  The counters (acc_len, n_blocks, ring_pos, has_prev) are host values
 * owned by the caller, as in the reference's cache objects, unless `counters` points at their device
 * mirror: then the kernel reads them there (ring_pos = ring_n % win), skips the append and raises
 * KCH_STATUS_CACHE_CAPACITY if a closing block finds no room, and the caller follows with
 * kch_cache_advance. */
typedef struct kch_cache_append_args {
  int B, c, c_I, m, win;
  int dtype;                 /* dtype of projections, accumulators, ring, kcomp (KCH_F32 / KCH_BF16) */
  const void *Ca, *Cb, *Za, *Zb, *K_idx, *Z_idx;  /* token rows: row b at element b*ld_c (b*ld_i) */
  int64_t ld_c, ld_i;
  void *acc_Ca, *acc_Cb, *acc_Za, *acc_Zb, *acc_K_idx, *acc_Z_idx;  /* [B,m,c] / [B,m,c_I] */
  int acc_len;
  void *prev_Cb, *prev_Zb;   /* [B,m,c] */
  int has_prev;
  const void *Ba, *Bb, *B_idx;  /* [m,c], [m,c], [m,c_I] in `dtype` */
  void* comp;                /* [B,capacity,c] in comp_kind */
  int comp_kind;             /* == dtype, or KCH_FP8_E4M3 / KCH_INT8 */
  float* comp_scales;        /* [B,capacity,c/64] for 8-bit kinds */
  float* comp_norms;         /* [B,capacity] */
  void* kcomp;               /* [B,capacity,c_I] in dtype */
  float* kcomp_norms;        /* [B,capacity] max(||stored indexer key||, 1e-12) */
  int64_t capacity;
  int n_blocks;
  void* ring;                /* [B,win,c] in dtype */
  int ring_pos;
  int normalize;
  const int32_t* counters;   /* optional device mirror, see above */
} kch_cache_append_args;
int kch_cache_append_token(const kch_cache_append_args* args, void* stream);
/* The same with kch_cache_advance folded in (needs `counters`): the CTA that finishes last advances the device
 * counters, one launch instead of two per layer and token. */
int kch_cache_append_token_advance(const kch_cache_append_args* args, void* stream);

/* Lightning indexer of one decode step over a cache's stored indexer keys
 * (CSADecodingCache.forward_step, ops_decoding_cache.py:903-1000): q_idx [B,HI*DI] rows q_ld apart in
 * q_dtype (read as fp32, normalised here when `normalize`), keys [B,capacity,DI] in k_dtype with k_norms
 * [B,capacity] (key_n = key / norm when `normalize`), w [B,HI] rows w_ld apart in w_dtype.  The visible prefix is min(tokens / m, n_blocks) read from `counters`.
 * Writes idx_out [B,topk] (ascending block index, -1 padded).  workspace: B * round_up(capacity,4) floats. */
int64_t kch_decode_indexer_workspace_bytes(int B, int64_t capacity);
int kch_decode_indexer_topk(const void* q_idx, int q_dtype, int64_t q_ld, const void* keys, int k_dtype,
                            const float* k_norms, const void* w, int w_dtype, int64_t w_ld,
                            int32_t* idx_out, int B, int64_t capacity, int HI, int DI, int topk, int normalize,
                            float scale, int m, const int32_t* counters, void* workspace, int64_t workspace_bytes,
                            void* stream);

/* Attention of one decode step (one query per sequence) straight over a cache's storage, split over the
 * entries so that a small batch still fills the GPU (CSADecodingCache.forward_step
 * ops_decoding_cache.py:1001-1070, HCADecodingCache.forward_step 1318-1395).  Same joint softmax as
 * kch_attend; rows are used as row / norm when comp_norms is given.  Entry counts come from `counters`:
 * visible rows = min(tokens / m, n_blocks), window rows = min(ring_n, sliding_window).
 * workspace: B * n_splits * nh * (c + 2) floats, n_splits = kch_attend_decode_splits(B). */
typedef struct kch_attend_decode_args {
  const void* q;             /* [B, nh*c] rows q_ld apart */
  int q_dtype;
  int64_t q_ld;
  int q_normalize;
  int B, nh, c;
  const void* comp;          /* [B,capacity,c] */
  int comp_dtype;
  int64_t capacity;
  const float* comp_norms;   /* [B,capacity] or NULL */
  const float* comp_scales;  /* [B,capacity,c/64] for the 8-bit kinds */
  const int32_t* sel_indices;/* [B,topk] or NULL = every visible row */
  int topk;
  int m;
  const void* win;           /* ring [B,sliding_window,c] or NULL */
  int win_dtype;
  int sliding_window;
  const void* sink;
  int sink_dtype;
  float scale;
  void* out;                 /* [B, nh*c] */
  int out_dtype;
  const int32_t* counters;
  void* workspace;
  int64_t workspace_bytes;
} kch_attend_decode_args;
int kch_attend_decode_splits(int B);
int64_t kch_attend_decode_workspace_bytes(int B, int nh, int c);
int kch_attend_decode(const kch_attend_decode_args* args, void* stream);

/* Block-scaled 8-bit encoding of rows (no counterpart in the reference; it stores the cache dtype only):
 * payload [rows,c], scales [rows,c/64], norms [rows] = max(||dequantised row||, 1e-12). */
int kch_quantize_rows(const void* x, int64_t ld, void* payload, float* scales, float* norms, int64_t rows,
                      int c, int kind, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KCH_B200_H */
