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
 * scale = 1/sqrt(D) computed inside, no mask. kv_dtype: ARGUS_B200_KV_F16 (F32 is declined with
 * E_UNSUPPORTED in this version). D in {64,128}; Hq/Hkv <= 8 per KV head group. */
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

#ifdef __cplusplus
}
#endif
#endif /* ARGUS_B200_H */
