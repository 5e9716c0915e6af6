/*
 * argus_b200.h — C ABI of the B200 (sm_100a) attention path for argus-engine.
 *
 * Plain C: pointers, sizes and POD structs only. Each entry point names the reference interface it
 * stands behind (path inside the argus-engine tree : line). Device pointers are ordinary CUDA device
 * addresses (managed memory is accepted); `stream` is a CUstream / cudaStream_t, NULL = the legacy
 * default stream, used verbatim.
 *
 * Error convention (the engine builds with panic=abort, so nothing here aborts or traps):
 *   0  ARGUS_B200_OK            done (work is enqueued on `stream` unless a host output was requested)
 *  -1  ARGUS_B200_E_INVALID     bad argument
 *  -2  ARGUS_B200_E_UNSUPPORTED shape / dtype this library declines; the caller keeps its own route,
 *                               exactly like `Ok(false)` of Backend::flash_attention_prefill
 *  -3  ARGUS_B200_E_CUDA        a CUDA runtime call failed; see argus_b200_last_error()
 *  -4  ARGUS_B200_E_WORKSPACE   the problem needs more scratch than the context may hold
 */
#ifndef ARGUS_B200_H
#define ARGUS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ARGUS_B200_API __attribute__((visibility("default")))
#else
#define ARGUS_B200_API
#endif

#define ARGUS_B200_OK 0
#define ARGUS_B200_E_INVALID (-1)
#define ARGUS_B200_E_UNSUPPORTED (-2)
#define ARGUS_B200_E_CUDA (-3)
#define ARGUS_B200_E_WORKSPACE (-4)

#define ARGUS_B200_KV_F32 0
#define ARGUS_B200_KV_F16 1

#define ARGUS_B200_MAX_BATCH 64

/* Opaque per-device context: owns the split-KV scratch (partials, tickets, logit scratch) and the
 * launch plan cache. One per CUDA device; calls on one context must come from one thread at a time
 * (the engine's single inference thread, cf. engine/src/backend/cuda_pc.rs:254). */
typedef struct argus_b200_ctx argus_b200_ctx;

/* Replaces the JIT set-up of the reference backends (CudaKernels::compile,
 * engine/src/backend/cuda_pc/kernels.rs:96-180; KiviCudaBackend make, crates/techniques/kivi/src/
 * gpu_kivi_cuda.rs:387-437): kernels are ahead-of-time sm_100a code, so this only binds the current
 * device, raises the shared-memory limits and allocates `workspace_bytes` of scratch (0 = default
 * 64 MiB). The caller's context is borrowed, never destroyed. */
ARGUS_B200_API int argus_b200_create(int device, size_t workspace_bytes, argus_b200_ctx** out);
/* The same inside the CALLER'S CUDA context instead of the device's primary one: `cu_context` is the raw CUcontext the
 * engine's KV buffers live in - CudaQuantAttnMakeArgs.cu_context / cu_device (crates/argus-extension-api/src/lib.rs:
 * 2985-2994), which the reference's plugin rebuilds with CudaContext::from_raw_context
 * (crates/techniques/kivi/src/gpu_kivi_cuda.rs:387-399). It is pushed for the allocations and popped again, borrowed and
 * never destroyed. Later calls on the context object must come from a thread that has this CUDA context current, as
 * the engine's inference thread does. */
ARGUS_B200_API int argus_b200_create_in_context(void* cu_context, int device, size_t workspace_bytes, argus_b200_ctx** out);
ARGUS_B200_API void argus_b200_destroy(argus_b200_ctx* ctx);
/* Text of the last failure on this context ("" if none). Owned by the context. */
ARGUS_B200_API const char* argus_b200_last_error(const argus_b200_ctx* ctx);
/* Library version and the SM architecture the kernels were built for (100). */
ARGUS_B200_API int argus_b200_version(void);
ARGUS_B200_API int argus_b200_sm_arch(void);
/* Kernel launches issued through this context since creation (all entry points). */
ARGUS_B200_API uint64_t argus_b200_launch_count(const argus_b200_ctx* ctx);

/* One sequence of a decode call. K/V element (kv_head, t, c) lives at
 * base + kv_head*head_stride + t*pos_stride + c (strides in ELEMENTS), which covers both layouts of
 * engine/src/kv/kv_cache.rs:238-266: HeadMajor (head_stride = capacity*D, pos_stride = D) and
 * SeqMajor (head_stride = D, pos_stride = Hkv*D). */
typedef struct argus_b200_seq {
    const void* k;
    const void* v;
    int64_t seq_len;     /* cache_seq_len of this sequence; 0 is allowed (output zeros, lse = -inf) */
    int64_t head_stride; /* elements */
    int64_t pos_stride;  /* elements */
} argus_b200_seq;

/* Optional outputs of a decode call. All pointers may be NULL. Device pointers unless noted.
 *  scores      [n_seqs][Hq][score_stride]  post-softmax p_t per query head — the layout of
 *              `scores_out[h*stride + t]` in Backend::attention_gen (engine/src/backend.rs:376-383)
 *              and of the GPU accumulator's score_buf slice (engine/src/backend/cuda_pc.rs:1750-1759).
 *  head_scores [n_seqs][Hkv][score_stride] group mean (1/g)*sum_r p[kv*g+r][t] — one tracked layer of
 *              AttnScoreProducer::accumulate_layer_gqa (crates/techniques/attn-score/src/lib.rs:278-287),
 *              fused so that the Hq-wide score matrix never reaches HBM.
 *  flat_scores [n_seqs][score_stride]      sum over all query heads (same file :262-266).
 *  lse         [n_seqs][Hq]                natural-log sum-exp of the scaled logits (-inf if seq_len==0);
 *              with `out` this is the (o, lse) partial of engine/src/backend/cpu/neon.rs:1028-1043.
 *  scores_host HOST pointer [n_seqs][Hq][score_stride]; when set the call blocks until it is filled,
 *              like the `scores_out` read-back of CudaBackend::attention_gen (cuda_pc.rs:1867-1880). */
typedef struct argus_b200_decode_extras {
    float* scores;
    float* head_scores;
    float* flat_scores;
    float* lse;
    float* scores_host;
    int64_t score_stride; /* elements; >= max seq_len when any score output is set */
} argus_b200_decode_extras;

/* Single-query GQA decode attention = Backend::attention_gen (engine/src/backend.rs:284-295; CUDA
 * implementation engine/src/backend/cuda_pc.rs:1693-1885 + attention_gen_f16kv_naive,
 * engine/src/backend/cuda_pc/kernels.cu:471-540). q [Hq][D] F32, out [Hq][D] F32,
 * scale = 1/sqrt(D) computed inside, no mask. kv_dtype: ARGUS_B200_KV_F16, or ARGUS_B200_KV_F32 (the cache is
 * first rounded to a packed F16 copy in context scratch, 2*Hkv*T*D*2 bytes; strides then need only be
 * multiples of 4 elements). D in {64,128}; Hq/Hkv <= 8 per KV head group. */
ARGUS_B200_API int argus_b200_attention_gen(argus_b200_ctx* ctx, void* stream, const float* q, const void* k_cache,
                             const void* v_cache, float* out, int num_heads_q, int num_heads_kv,
                             int head_dim, int64_t cache_seq_len, int kv_dtype, int64_t head_stride,
                             int64_t pos_stride, const argus_b200_decode_extras* extras);

/* The same over n_seqs <= ARGUS_B200_MAX_BATCH independent sequences of different lengths in ONE
 * launch (the reference engine has no batched decode; it would loop attention_gen). q/out
 * [n_seqs][Hq][D]. `seqs` is a HOST array, read during the call. */
ARGUS_B200_API int argus_b200_attention_gen_batched(argus_b200_ctx* ctx, void* stream, const float* q,
                                     const argus_b200_seq* seqs, int n_seqs, float* out,
                                     int num_heads_q, int num_heads_kv, int head_dim, int kv_dtype,
                                     const argus_b200_decode_extras* extras);

/* One decode step of the engine's attention layer in one call: the new token's K/V row is written into the cache and
 * the query attends over the sequence INCLUDING it - the pair of calls the engine issues back to back
 * (engine/src/layers/transformer_layer/forward_gen_fmt.rs:207 KV write, :267-275 attention; kernels
 * kv_scatter_f32_to_f16, engine/src/backend/cuda_pc/kernels.cu:305-340, + attention_gen_f16kv_naive, :471-540).
 * k_new / v_new: F32 device rows [n_seqs][Hkv][D] (16-byte aligned), stored at position seqs[b].seq_len - the length
 * BEFORE the write, which must be below capacity[b] - rounded to F16 nearest-even exactly like argus_b200_kv_scatter;
 * the attention then runs over seq_len + 1 positions. With F16 caches both happen in ONE launch (the CTA that owns the
 * end of a sequence stores the row before it reads); F32 caches take the KV write kernel first. The caller advances
 * its sequence length afterwards. `seqs` and `capacity` are HOST arrays read during the call. */
ARGUS_B200_API int argus_b200_decode_step_batched(argus_b200_ctx* ctx, void* stream, const float* q, const float* k_new,
                                                  const float* v_new, const argus_b200_seq* seqs, const int64_t* capacity,
                                                  int n_seqs, float* out, int num_heads_q, int num_heads_kv, int head_dim,
                                                  int kv_dtype, const argus_b200_decode_extras* extras);
ARGUS_B200_API int argus_b200_decode_step(argus_b200_ctx* ctx, void* stream, const float* q, const float* k_new,
                                          const float* v_new, void* k_cache, void* v_cache, float* out, int num_heads_q,
                                          int num_heads_kv, int head_dim, int64_t cache_seq_len, int64_t capacity,
                                          int kv_dtype, int64_t head_stride, int64_t pos_stride,
                                          const argus_b200_decode_extras* extras);

/* The same over PAGED F16 caches (the paged layout option of a KVCacheFormat for batched serving; no counterpart in
 * the reference, whose caches are contiguous per sequence): K and V live in page pools; token t of sequence b is row
 * t % page_tokens of page seqs[b].page_table[t / page_tokens], and element (page, kv_head, row, c) sits at
 * pool + page*page_stride + kv_head*head_stride + row*pos_stride + c (strides in elements, multiples of 8; a page
 * laid out [Hkv][page_tokens][D] has head_stride = page_tokens*D, pos_stride = D, page_stride = Hkv*page_tokens*D).
 * page_tokens is a multiple of 16. `seqs` is a HOST array read during the call, the page tables are DEVICE arrays of
 * ceil(seq_len / page_tokens) page numbers. Same outputs, extras and split plan as argus_b200_attention_gen_batched:
 * for the same tokens the results are bit-identical to the contiguous form. */
typedef struct argus_b200_paged_seq {
    const int32_t* page_table;
    int64_t seq_len;
} argus_b200_paged_seq;
ARGUS_B200_API int argus_b200_attention_gen_paged(argus_b200_ctx* ctx, void* stream, const float* q, const void* k_pool,
                                                  const void* v_pool, const argus_b200_paged_seq* seqs, int n_seqs,
                                                  float* out, int num_heads_q, int num_heads_kv, int head_dim,
                                                  int page_tokens, int64_t page_stride, int64_t head_stride,
                                                  int64_t pos_stride, const argus_b200_decode_extras* extras);

/* ───────────── KIVI capability: CudaQuantAttnBackend (crates/argus-extension-api/src/lib.rs:3087-3104) ─────────────
 * The four structs below are byte-for-byte the #[repr(C)] PODs of the reference (same field order and
 * types; usize = size_t, u64 device pointers, bool = uint8_t); the Rust FFI crate passes them through
 * unchanged. All buffers are engine-owned and borrowed for the call. */

/* CudaQuantAttnArgs, lib.rs:3000-3026 */
typedef struct argus_b200_quant_attn_args {
    void* cu_stream;      /* NULL = default stream */
    uint64_t q_mem;       /* [Hq][D] F32 */
    uint64_t qk_mem;      /* packed K blocks [flush][Hkv][group][ch] */
    uint64_t qv_mem;      /* packed V blocks [flush][Hkv][token][D/32] */
    uint64_t res_k_mem;   /* F32 residual [Hkv][res_cap][D] */
    uint64_t res_v_mem;
    uint64_t out_mem;     /* [Hq][D] F32 */
    float* scores_out;    /* HOST pointer [Hq][scores_len/Hq], NULL = skip; filled when the call returns */
    size_t scores_len;
    size_t num_heads_q, num_heads_kv, head_dim, q_tokens, res_tokens, res_cap;
    float scale;
    uint8_t bits;         /* 2, 4 or 8 */
} argus_b200_quant_attn_args;

/* CudaQuantAttnGatherArgs, lib.rs:3031-3043 */
typedef struct argus_b200_quant_gather_args {
    void* cu_stream;
    uint64_t input_mem;    /* [seq_len][Hkv][D] F32 */
    uint64_t residual_mem; /* [Hkv][res_cap][D] F32, rows res_pos.. written */
    size_t kv_heads, res_cap, head_dim, seq_len, res_pos;
} argus_b200_quant_gather_args;

/* CudaQuantDequantFlushArgs, lib.rs:3048-3063 */
typedef struct argus_b200_quant_dequant_flush_args {
    void* cu_stream;
    uint64_t q_blocks_mem;
    uint64_t attn_mem;     /* F16 SeqMajor view [max_seq][Hkv][D] */
    size_t kv_heads, head_dim;
    size_t n_groups_or_tokens; /* K: groups per flush; V: flush tokens */
    size_t tok_base, block_start;
    uint8_t bits;
    uint8_t is_key;
} argus_b200_quant_dequant_flush_args;

/* CudaQuantScatterResidualArgs, lib.rs:3069-3081 */
typedef struct argus_b200_quant_scatter_residual_args {
    void* cu_stream;
    uint64_t res_mem;      /* F32 ring */
    uint64_t attn_mem;     /* F16 SeqMajor view */
    size_t kv_heads, res_cap, head_dim, res_pos, tok_base;
} argus_b200_quant_scatter_residual_args;

/* has_quant_attn_kernel(bits): 1 for bits in {2,4,8}, else 0. */
ARGUS_B200_API int argus_b200_kivi_has_quant_attn_kernel(const argus_b200_ctx* ctx, int bits);
/* attention_gen_quant — replaces KiviCudaBackend::attention_inner (crates/techniques/kivi/src/gpu_kivi_cuda.rs:126-223)
 * and kernel_attn_gen_kivi_q{2,4,8} (crates/techniques/kivi/src/kivi_attn.cu). No per-call allocation. */
ARGUS_B200_API int argus_b200_kivi_attention_gen_quant(argus_b200_ctx* ctx, const argus_b200_quant_attn_args* args);
/* gather_update_quant — kivi_gather_update (crates/techniques/kivi/src/kivi_q2.cu:117-138). */
ARGUS_B200_API int argus_b200_kivi_gather_update_quant(argus_b200_ctx* ctx, const argus_b200_quant_gather_args* args);
/* dequant_flush — kivi_dequantize_{key,value}_q2_f16 (kivi_q2.cu:19-91); the reference supports bits==2
 * only (gpu_kivi_cuda.rs:254-257), this one 2, 4 and 8. */
ARGUS_B200_API int argus_b200_kivi_dequant_flush(argus_b200_ctx* ctx, const argus_b200_quant_dequant_flush_args* args);
/* scatter_residual — kivi_scatter_residual_f16 (kivi_q2.cu:93-115). */
ARGUS_B200_API int argus_b200_kivi_scatter_residual(argus_b200_ctx* ctx,
                                                    const argus_b200_quant_scatter_residual_args* args);

/* Flush of the residual ring on the device: quantises n_groups*32 ring tokens into K blocks (order
 * `for h, for group, for ch`) at block index k_block_start and V blocks (`for h, for tok, for blk`) at
 * v_block_start — the work QuantizedRecentWindowCache::flush_residual does on the CPU before uploading
 * (engine/src/kv/quant_window_cache.rs:844-965, :1688-1866), bit-exact with BlockQ2_0/BlockKVQ4/BlockKVQ8::quantize
 * (crates/argus-kv-codec/src/lib.rs:36-73,125-157,175-202). res_k/res_v: F32 [Hkv][res_cap][D]. */
ARGUS_B200_API int argus_b200_kivi_flush_pack(argus_b200_ctx* ctx, void* stream, const float* res_k,
                                              const float* res_v, void* qk, void* qv, int kv_heads, int head_dim,
                                              int res_cap, int n_groups, int bits, int64_t k_block_start,
                                              int64_t v_block_start);

/* One KIVI-packed sequence of a batched call. */
typedef struct argus_b200_kivi_seq {
    const void* qk;
    const void* qv;
    const void* res_k;  /* [Hkv][res_cap][D], F32 or F16 (see res_dtype) */
    const void* res_v;
    int64_t q_tokens;   /* multiple of res_cap */
    int64_t res_tokens; /* <= res_cap */
} argus_b200_kivi_seq;

/* Fused dequant + decode over n_seqs packed sequences in one launch, with the optional outputs of
 * argus_b200_decode_extras (device score matrices, fused GQA group means for H2O, lse). `scale` is
 * applied to q·k as in CudaQuantAttnArgs. res_dtype: ARGUS_B200_KV_F32 (the engine's ring) or
 * ARGUS_B200_KV_F16. q/out [n_seqs][Hq][D] F32. */
ARGUS_B200_API int argus_b200_kivi_attention_batched(argus_b200_ctx* ctx, void* stream, const float* q,
                                                     const argus_b200_kivi_seq* seqs, int n_seqs, float* out,
                                                     int num_heads_q, int num_heads_kv, int head_dim, int res_cap,
                                                     int bits, int res_dtype, float scale,
                                                     const argus_b200_decode_extras* extras);

/* The same over PAGED packed caches (batched serving; no reference counterpart: the engine's packed cache is one
 * contiguous buffer per layer, engine/src/kv/quant_window_cache.rs:844-965). A page holds ONE flush of res_cap tokens
 * for all KV heads: its K blocks [Hkv][res_cap/32][D] sit at block index page * Hkv*(res_cap/32)*D of qk_pool and its
 * V blocks [Hkv][res_cap][D/32] at block index page * Hkv*res_cap*(D/32) of qv_pool - the layout one flush has in the
 * contiguous form, so a flush can be written with argus_b200_kivi_flush_pack at those block indices. flush_pages is a
 * DEVICE array of q_tokens / res_cap page numbers; `seqs` is a HOST array read during the call; the residual rings
 * stay per sequence. For the same tokens the results are bit-identical to argus_b200_kivi_attention_batched. */
typedef struct argus_b200_kivi_paged_seq {
    const int32_t* flush_pages;
    const void* res_k;
    const void* res_v;
    int64_t q_tokens;
    int64_t res_tokens;
} argus_b200_kivi_paged_seq;
ARGUS_B200_API int argus_b200_kivi_attention_paged(argus_b200_ctx* ctx, void* stream, const float* q, const void* qk_pool,
                                                   const void* qv_pool, const argus_b200_kivi_paged_seq* seqs, int n_seqs,
                                                   float* out, int num_heads_q, int num_heads_kv, int head_dim,
                                                   int res_cap, int bits, int res_dtype, float scale,
                                                   const argus_b200_decode_extras* extras);

/* ───────────── Score reducer: CudaScoreReduceBackend (lib.rs:2938-2948) ───────────── */

/* CudaScoreReduceArgs, lib.rs:2909-2933 (byte-for-byte). */
typedef struct argus_b200_score_reduce_args {
    void* cu_stream;
    uint64_t score_buf;        /* [n_layers][Hq][score_stride] post-softmax scores */
    uint64_t importance;       /* [max_seq_len], in place */
    uint64_t head_importance;  /* [Hkv * max_seq_len], in place */
    float decay_factor;        /* 1 - decay, clamped to [0,1] by the engine */
    size_t n_layers, n_heads_q, n_kv_heads, cache_seq_len, score_stride, max_seq_len;
    uint64_t layer_flat_importance; /* [n_layers * max_seq_len], 0 when unused */
} argus_b200_score_reduce_args;

/* reduce — kernel_score_fused_reduce (crates/techniques/attn-score/src/score_reduce.cu:13-64); no
 * 16-KV-head limit. Bit-identical to the CPU producer (AttnScoreProducer, crates/techniques/attn-score/src/lib.rs:
 * 175-359: decay as a rounded product, then a rounded sum); the reference's CUDA kernel contracts the two into one
 * FMA and can differ by one ulp when importance*decay_factor is inexact. */
ARGUS_B200_API int argus_b200_score_reduce(argus_b200_ctx* ctx, const argus_b200_score_reduce_args* args);
/* reduce_per_layer — kernel_score_fused_reduce_per_layer (score_reduce.cu:66-91). */
ARGUS_B200_API int argus_b200_score_reduce_per_layer(argus_b200_ctx* ctx, const argus_b200_score_reduce_args* args);

/* ───────────── Prefill: Backend::flash_attention_prefill (engine/src/backend.rs:1011-1027) ───────────── */

#define ARGUS_B200_PREFILL_F32Q_F16KV 0 /* the engine's entry: Q/O F32, K/V F16 (cuda_pc.rs:830-926) */
#define ARGUS_B200_PREFILL_BF16 1       /* Q, K, V, O all BF16 */
#define ARGUS_B200_PREFILL_F16 2        /* Q, K, V, O all F16 */

/* Causal GQA flash-attention prefill — replaces CudaBackend::flash_attention_prefill
 * (engine/src/backend/cuda_pc.rs:830-926) and flash_attn_prefill_f16kv_dk128
 * (engine/src/backend/cuda_pc/kernels.cu:691-816). Q/O [batch][seq_len][Hq][D]; K/V
 * [batch][Hkv][kv_capacity][D] when is_head_major, else [batch][kv_capacity][Hkv][D]. Query row r sees keys
 * 0..=cache_seq_len-seq_len+r; scale = 1/sqrt(D). Returns ARGUS_B200_E_UNSUPPORTED for head_dim != 128
 * (the reference's `Ok(false)`: the caller keeps its own route). In the F32-Q mode Q is first rounded to
 * F16 into context scratch (batch*seq_len*Hq*D*2 bytes).
 * In the BF16 mode V is multiplied as an F16 copy made tile by tile in shared memory (the probabilities need F16's 11
 * bits to hold the 2e-3 tolerance, and both operands of one MMA share a type): exact for |v| <= 65504, clamped to
 * +-65504 beyond. When that happens the status word reads 4 afterwards (argus_b200_check_status); the output is then
 * computed from the clamped values. */
ARGUS_B200_API int argus_b200_flash_attention_prefill(argus_b200_ctx* ctx, void* stream, const void* q,
                                                      const void* k_cache, const void* v_cache, void* out,
                                                      int n_heads_q, int n_heads_kv, int seq_len,
                                                      int cache_seq_len, int head_dim, int64_t kv_capacity,
                                                      int batch_size, int is_head_major, int dtype_mode);

/* ───────────── Sequence-sharded decode: merge of per-rank (o, lse) partials ─────────────
 * The reference is single-device; its only split/merge is the CPU chunk merge of
 * engine/src/backend/cpu/neon.rs:1028-1125, whose algebra this follows. Each rank runs
 * argus_b200_attention_gen over its slice of the KV sequence with `out` and `extras.lse` pointing into one
 * buffer of part_stride = Hq*D + Hq floats ([Hq][D] outputs, then [Hq] lse); the buffers of all ranks are
 * gathered (one NCCL all-gather) into `parts` [n_parts][part_stride] in this rank's own memory, and this call
 * writes out[Hq][D] (and optionally the merged lse[Hq]). Empty shards (lse = -inf) are skipped. */
ARGUS_B200_API int argus_b200_lse_merge(argus_b200_ctx* ctx, void* stream, const float* parts, int n_parts,
                                        int64_t part_stride, int num_heads_q, int head_dim, float* out,
                                        float* lse_out);

/* The whole step of a sequence-sharded decode in ONE launch: argus_b200_attention_gen over this rank's slice of the KV
 * sequence, whose split-merge epilogue also does the exchange. No counterpart in the reference (single device; the
 * algebra is the chunk merge of engine/src/backend/cpu/neon.rs:1028-1125). The CTA that completes a KV head stores the
 * head group's normalised rows and natural-log lse into slot `rank` of every other rank's receive buffer with plain
 * NVLink peer stores (no multicast, no bulk copy on peer memory), then collects - every wait bounded - the other
 * ranks' rows of those heads from its OWN receive buffer and writes the merged rows to `out` [Hq][D] (and `merged_lse`
 * [Hq] if set).
 *
 * Wire format: 128-byte lines of 30 data words followed by the step number twice. A line is written by one warp-wide
 * store (eight lanes x 16 bytes, one aligned 128-byte NVLink write) and read the same way, so a reader that finds the
 * current step number in both flag words has the data of the same write: no fence, no separate flag traffic, latency
 * of one store plus one NVLink crossing. A head group's g*(D+1) floats ([g][D] outputs, then [g] lse) take
 * ceil(g*(D+1)/30) lines, rounded up to a multiple of four; buffer sizes are counted in UNITS OF 16 BYTES:
 * lines_per_head = 8 x that line count (argus_b200_exchange_lines_per_head). A receive buffer is 128-byte aligned and
 * holds two sets (even / odd steps, `parity_stride_lines` units apart, a multiple of 8) of
 * [n_ranks][Hkv][lines_per_head] units, zero-initialised once (steps start at 1).
 * peer_lines[s] is the address, valid on this GPU, of rank s's receive buffer (e.g. a torch symmetric-memory
 * allocation). The step number lives in device memory: `step_counters` is an int[Hkv] array of this rank,
 * zero-initialised once and bumped by the kernel itself (one counter per KV head), so the call replays from a CUDA
 * graph; every rank must issue the same sequence of calls. Odd steps use the second buffer set, so a fast rank's next
 * push cannot overwrite what a slow rank still reads. phases: 3 normally; 1 = push only, after which
 * argus_b200_exchange_wait_merge (with the host's step number and this rank's own (o, lse) partial) does the second
 * half: the form single-GPU tests use, where no kernel may wait for a later launch. A shard may be empty (shard_len 0:
 * lse = -inf, skipped by the merge). A wait that runs out (about a second) zeroes the heads' output and sets the status
 * word to 3 (argus_b200_check_status). */
typedef struct argus_b200_exchange {
    void* const* peer_lines;
    int* step_counters;
    float* merged_lse;
    int64_t parity_stride_lines;
    int n_ranks;
    int rank;
    int phases;
} argus_b200_exchange;
ARGUS_B200_API int argus_b200_attention_gen_sharded(argus_b200_ctx* ctx, void* stream, const float* q, const void* k_shard,
                                                    const void* v_shard, float* out, int num_heads_q, int num_heads_kv,
                                                    int head_dim, int64_t shard_len, int kv_dtype, int64_t head_stride,
                                                    int64_t pos_stride, const argus_b200_exchange* exchange);
/* 16-byte units one head group occupies in a receive buffer (see above). */
ARGUS_B200_API int argus_b200_exchange_lines_per_head(int num_heads_q, int num_heads_kv, int head_dim);
/* The receiving half alone: one CTA per KV head waits (bounded) for the other ranks' lines of step `step` in this rank's
 * receive buffer and merges them with `own_part` ([Hq][D] outputs then [Hq] lse, as argus_b200_attention_gen with
 * extras.lse writes them) into out [Hq][D]. `exchange->step_counters` and `phases` are ignored. */
ARGUS_B200_API int argus_b200_exchange_wait_merge(argus_b200_ctx* ctx, void* stream, const float* own_part,
                                                  const argus_b200_exchange* exchange, int step, int num_heads_q,
                                                  int num_heads_kv, int head_dim, float* out);

/* Blocks until `stream` is idle and returns the status word the kernels set (0 = clean) and clears it:
 * 1 / 2 a bounded wait inside a decode / prefill kernel ran out (the call's output is not valid), 2 also: an invalid
 * entry in a compaction list, 3 a rank's flags never arrived in a sharded step (those heads are zero),
 * 4 a BF16 prefill clamped V values beyond the F16 range (informational, set only when no error is pending). */
ARGUS_B200_API int argus_b200_check_status(argus_b200_ctx* ctx, void* stream);

/* ───────────── KV write and eviction executors on a device-resident cache ─────────────
 * The callers either side of attention. K and V are addressed like in argus_b200_attention_gen: element
 * (head h, position t, channel c) at h*head_stride + t*pos_stride + c (HeadMajor [Hkv][cap][D]: head_stride =
 * cap*D, pos_stride = D); kv_dtype ARGUS_B200_KV_F16 or _F32. Pointers and row pitches must be 16-byte
 * aligned (else ARGUS_B200_E_UNSUPPORTED). All results are bit-identical to the reference's.
 *
 * argus_b200_kv_scatter replaces kv_scatter_f32_to_f16, kv_scatter_f32_to_f16_batch and
 * kv_scatter_f32_to_f32_batch (engine/src/backend/cuda_pc/kernels.cu:305-360, host side
 * engine/src/backend/cuda_pc.rs:1460-1570): the new rows k_src/v_src [seq_len][Hkv][D] F32 are written to
 * positions write_pos .. write_pos+seq_len-1 (F16: rounded to nearest even). seq_len = 1 is the decode step.
 *
 * argus_b200_kv_compact replaces KVCache::compact_keep_positions and compact_keep_positions_for_head
 * (engine/src/kv/kv_cache.rs:1266-1352), which exist on the CPU only: position write_start+i receives position
 * keep[i] for i < n_keep, in place. keep_dev is a DEVICE array, ascending, with keep[i] >= write_start+i and keep[i] < capacity (the
 * cache's row count; the reference's slice indexing would panic beyond it; an entry
 * that breaks any of this is skipped and sets the status word to 2, see argus_b200_check_status; the cache contents are
 * then unspecified). head = -1 moves
 * every KV head, head >= 0 only that one. Like the reference, the call does not touch the sequence length: the
 * caller sets it to write_start + n_keep. Rows move in ascending chunks, through the context's scratch where a
 * chunk's sources and destinations can overlap.
 *
 * argus_b200_kv_weighted_merge replaces apply_weighted_merges for F32 and F16 caches
 * (engine/src/kv/standard_format.rs:754-893; D2O Eq. 11): for merge m and every head and channel,
 * into <- into_weight[m]*into + sum_j from_weight[j]*row(from_pos[j]), j in [from_start[m], from_start[m+1]), in
 * list order, each product and each sum rounded on its own (F16: the F32 result is rounded once at the end).
 * All five arrays are DEVICE arrays (from_start has n_merges+1 entries); positions are pre-compaction ones; a
 * merge with an empty list leaves its row untouched. axis: 0 = K and V, 1 = K only, 2 = V only (MergeAxis). */
ARGUS_B200_API int argus_b200_kv_scatter(argus_b200_ctx* ctx, void* stream, const float* k_src, const float* v_src,
                                         void* k_dst, void* v_dst, int dst_dtype, int num_heads_kv, int head_dim,
                                         int64_t capacity, int64_t head_stride, int64_t pos_stride, int64_t write_pos,
                                         int64_t seq_len);
/* The decode-step form for a batch (no counterpart in the reference, which has no batched decode): ONE launch writes
 * the new row k_src/v_src [n_seqs][Hkv][D] F32 of every sequence into that sequence's own cache at position
 * seqs[b].seq_len (the sequence's length BEFORE the write, which must be below capacity[b]). `seqs` and `capacity`
 * are HOST arrays read during the call; seqs[b] is the descriptor argus_b200_attention_gen_batched takes. */
ARGUS_B200_API int argus_b200_kv_scatter_batched(argus_b200_ctx* ctx, void* stream, const float* k_src,
                                                 const float* v_src, const argus_b200_seq* seqs, const int64_t* capacity,
                                                 int n_seqs, int dst_dtype, int num_heads_kv, int head_dim);
ARGUS_B200_API int argus_b200_kv_compact(argus_b200_ctx* ctx, void* stream, void* k, void* v, int kv_dtype,
                                         int num_heads_kv, int head_dim, int64_t capacity, int64_t head_stride,
                                         int64_t pos_stride, const int32_t* keep_dev, int64_t n_keep, int64_t write_start,
                                         int head);
ARGUS_B200_API int argus_b200_kv_weighted_merge(argus_b200_ctx* ctx, void* stream, void* k, void* v, int kv_dtype,
                                                int num_heads_kv, int head_dim, int64_t head_stride, int64_t pos_stride,
                                                const int32_t* into_pos, const float* into_weight,
                                                const int32_t* from_start, const int32_t* from_pos,
                                                const float* from_weight, int n_merges, int axis);

/* ───────────── KV residency and the session prefix cache payload ─────────────
 * argus_b200_kv_snapshot_prefix / _restore_prefix move the per-layer payload of the session prefix cache file
 * ("ARGUSKV1" version 2, engine/src/session/prefix_cache.rs:1-30): for one layer, K bytes [Hkv][token_count][D] followed by
 * V bytes in the cache's own element type - byte for byte what SnapshotRestore::snapshot_prefix produces through
 * extract_packed_bytes and restore_prefix consumes through scatter_packed_bytes
 * (engine/src/kv/standard_format.rs:1796-1838, :1657-1790). The reference reads all `capacity` rows of every head back to
 * the host and packs on the CPU; here only the token_count prefix rows move. `dst` / `src` may be device memory or host
 * memory (pinned for an asynchronous copy); its size must be exactly 2*Hkv*token_count*D*elt bytes. The file header (magic,
 * hashes, token ids, logits) stays with the engine. Restoring does not touch rows at or beyond token_count, nor the
 * sequence length, which the caller sets. The cache is addressed as in argus_b200_attention_gen (HeadMajor: one
 * pitched copy per tensor; SeqMajor: a gather kernel, rows and pitches 16-byte aligned).
 *
 * argus_b200_kv_make_resident: the engine allocates KV buffers as managed memory (cuMemAllocManaged,
 * engine/src/backend/cuda_pc/memory.rs:36-44) and leaves page placement to first touch. Called once per buffer (after
 * allocation, or after the host wrote into it) this sets the device as the range's preferred location and prefetches
 * it on `stream`, so that the decode kernels stream it at the device-memory rate. Device memory is accepted and left
 * alone; any other kind of pointer returns ARGUS_B200_E_UNSUPPORTED. argus_b200_kv_alloc / _free are the matching
 * allocator for hosts that want the library to own the choice (managed != 0: cudaMallocManaged, else cudaMalloc). */
ARGUS_B200_API int argus_b200_kv_snapshot_prefix(argus_b200_ctx* ctx, void* stream, const void* k, const void* v, int kv_dtype,
                                                 int num_heads_kv, int head_dim, int64_t capacity, int64_t head_stride,
                                                 int64_t pos_stride, int64_t token_count, void* dst, size_t dst_bytes);
ARGUS_B200_API int argus_b200_kv_restore_prefix(argus_b200_ctx* ctx, void* stream, void* k, void* v, int kv_dtype,
                                                int num_heads_kv, int head_dim, int64_t capacity, int64_t head_stride,
                                                int64_t pos_stride, int64_t token_count, const void* src, size_t src_bytes);
ARGUS_B200_API int argus_b200_kv_make_resident(argus_b200_ctx* ctx, void* stream, const void* ptr, size_t bytes);
ARGUS_B200_API int argus_b200_kv_alloc(argus_b200_ctx* ctx, size_t bytes, int managed, void** out);
ARGUS_B200_API int argus_b200_kv_free(argus_b200_ctx* ctx, void* ptr);

/* D2O Eq. 8, find_nearest_layer_wide_via with cosine_similarity (crates/techniques/d2o/src/lib.rs:187-255; CPU-only in
 * the reference): for each evicted position the retained position whose K row (all KV heads concatenated) has the
 * largest cosine similarity - the first one in list order on ties, never the evicted position itself; no valid
 * target gives retain_pos[0] (or the evicted position when the list is empty) and similarity 0. Dot products and
 * squared norms are accumulated channel by channel with one rounding per product and per sum, as the reference
 * does, so similarities and selected positions are bit-identical. evict_pos / retain_pos / nearest_out / sim_out are
 * DEVICE arrays. head_dim must be a multiple of 32. */
ARGUS_B200_API int argus_b200_d2o_nearest(argus_b200_ctx* ctx, void* stream, const void* k_cache, int kv_dtype,
                                          int num_heads_kv, int head_dim, int64_t head_stride, int64_t pos_stride,
                                          const int32_t* evict_pos, int n_evict, const int32_t* retain_pos, int n_retain,
                                          int32_t* nearest_out, float* sim_out);

/* prefill_attention_scores (engine/src/kv/standard_format.rs:1400-1510; the H2O prefill seed, CPU-only in the
 * reference, which reads K back from the device for it): for the trailing min(q_window, seq_len) query rows of a
 * prefill chunk, row r at absolute position p = q_start_pos + r, the softmax probabilities of every query head over
 * keys lo..=p (scale 1/sqrt(head_dim), GQA head h reads KV head h / (Hq/Hkv)); lo = 0, or max(0, p - (window-1))
 * with a sliding window (`window` > 0).
 *   q        [seq_len][Hq][D] F32 (device), the chunk's queries
 *   sum_out  [Hq][cache_seq_len] += sum over the rows (nullable)                      -- IMP-2
 *   per_row  per_row_per_head != 0: [q_window][Hq][cache_seq_len] = the row's probabilities;
 *            per_row_per_head == 0: [q_window][cache_seq_len] += mean over heads (nullable) -- IMP-4
 * As in the reference the caller zeroes the buffers first and entries behind a row's position are not written.
 * Within the decode tolerance of the reference (its own test is bit-exact against a scalar loop; a GPU softmax is
 * not), accumulation orders as the reference's. F32 caches are declined (ARGUS_B200_E_UNSUPPORTED). K and V are addressed as in argus_b200_attention_gen; V is read by the decode
 * kernel this call is built on. */
ARGUS_B200_API int argus_b200_prefill_attention_scores(argus_b200_ctx* ctx, void* stream, const float* q,
                                                       const void* k_cache, const void* v_cache, int kv_dtype,
                                                       int num_heads_q, int num_heads_kv, int head_dim, int seq_len,
                                                       int cache_seq_len, int64_t head_stride, int64_t pos_stride,
                                                       int q_start_pos, int q_window, int window, float* sum_out,
                                                       float* per_row, int per_row_per_head);

/* ───────────── Decode without any allocation ─────────────
 * No counterpart in the reference (its CUDA backend allocates freely: managed KV buffers, a lazily grown
 * score scratch, a per-call score buffer in the KIVI plugin). This entry point is for hosts of this library
 * that cannot call cudaMalloc - code running under a stream capture or in a serving loop where an allocation
 * would synchronise the device, and embedders whose device memory comes once from their own pool.
 *
 * Same computation as argus_b200_attention_gen for one sequence (F16 K/V, D in {64,128}, Hq/Hkv <= 8) with an
 * optional natural-log lse[Hq] output and no score outputs. No context: the split-KV scratch lives in a fixed
 * array of argus_b200_static_scratch_bytes() = 4 MiB inside the library image, one per device that loads the
 * library, held until the process exits. A call whose split plan needs more (about 4 KB per (split, KV head)
 * at D=128; in practice Hkv up to 256 and any sequence length) returns ARGUS_B200_E_WORKSPACE.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and the SM count
 * with that device current: make that first call before any stream capture begins. All calls on a device
 * share the array and it keeps the last call's contents; the words that must start at zero are cleared on
 * `stream` at the start of every call. Calls whose kernels may overlap on the GPU race on the array: issue
 * them on one stream, or otherwise order them. Calls cudaMemsetAsync and one kernel launch, nothing that
 * allocates. Error text: argus_b200_static_last_error() (per host thread). */
ARGUS_B200_API int argus_b200_attention_gen_static(void* stream, const float* q, const void* k_cache,
                                                   const void* v_cache, float* out, float* lse, int num_heads_q,
                                                   int num_heads_kv, int head_dim, int64_t cache_seq_len,
                                                   int kv_dtype, int64_t head_stride, int64_t pos_stride);
ARGUS_B200_API size_t argus_b200_static_scratch_bytes(void);
ARGUS_B200_API const char* argus_b200_static_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* ARGUS_B200_H */
