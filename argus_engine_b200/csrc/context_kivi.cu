// Host side of the KIVI capability and of the score reducer: argument checks, split planning over the
// packed part and the residual window, scratch binding, launches. Counterpart of KiviCudaBackend
// (crates/techniques/kivi/src/gpu_kivi_cuda.rs:33-446) and AttnScoreCudaReducer
// (crates/techniques/attn-score/src/gpu_reduce_cuda.rs:25-265) without their run-time nvcc step and
// without the per-call cuMemAlloc/cuMemFree of a score buffer.
#include <cuda_fp16.h>
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "context.h"

// The PODs must match the reference's #[repr(C)] structs byte for byte.
static_assert(sizeof(argus_b200_quant_attn_args) == 128, "CudaQuantAttnArgs layout");
static_assert(offsetof(argus_b200_quant_attn_args, scores_out) == 56, "CudaQuantAttnArgs layout");
static_assert(offsetof(argus_b200_quant_attn_args, scale) == 120, "CudaQuantAttnArgs layout");
static_assert(offsetof(argus_b200_quant_attn_args, bits) == 124, "CudaQuantAttnArgs layout");
static_assert(sizeof(argus_b200_quant_gather_args) == 64, "CudaQuantAttnGatherArgs layout");
static_assert(sizeof(argus_b200_quant_dequant_flush_args) == 72, "CudaQuantDequantFlushArgs layout");
static_assert(offsetof(argus_b200_quant_dequant_flush_args, bits) == 64, "CudaQuantDequantFlushArgs layout");
static_assert(sizeof(argus_b200_quant_scatter_residual_args) == 64, "CudaQuantScatterResidualArgs layout");
static_assert(sizeof(argus_b200_score_reduce_args) == 96, "CudaScoreReduceArgs layout");
static_assert(offsetof(argus_b200_score_reduce_args, n_layers) == 40, "CudaScoreReduceArgs layout");

namespace argus {

static int block_bytes(int bits) { return bits == 2 ? 12 : bits == 4 ? 20 : bits == 8 ? 36 : -1; }

int kivi_entry(Context* ctx, cudaStream_t st, const float* q, const argus_b200_kivi_seq* seqs, int n_seqs, float* out,
               int hq, int hkv, int d, int res_cap, int bits, int res_dtype, float scale,
               const argus_b200_decode_extras* ex, const int32_t* const* flush_pages) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    if (!q || !seqs || !out || n_seqs <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || n_seqs > kMaxBatch) {
        ctx->set_error("kivi attention: null pointer, bad head counts or more than %d sequences", kMaxBatch);
        return ARGUS_B200_E_INVALID;
    }
    if (res_cap <= 0 || res_cap % 32 != 0 || d % 32 != 0) {
        ctx->set_error("kivi attention: res_cap (%d) and head_dim (%d) must be positive multiples of 32", res_cap, d);
        return ARGUS_B200_E_INVALID;
    }
    const int g = hq / hkv;
    if (block_bytes(bits) < 0 || (d != 64 && d != 128) || g > kMaxGroup) {
        ctx->set_error("kivi attention: unsupported (bits=%d head_dim=%d group=%d)", bits, d, g);
        return ARGUS_B200_E_UNSUPPORTED;
    }
    KiviBatch bt;
    memset(&bt, 0, sizeof(bt));
    bt.res_cap = res_cap;
    bt.res_is_f16 = (res_dtype == ARGUS_B200_KV_F16);
    bt.res_chunk = 32;   // 8 token steps per warp: the residual rows go through plain F32 arithmetic, one token at a time
    int64_t qlens[kMaxBatch];
    int64_t max_len = 0, max_res = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const argus_b200_kivi_seq& s = seqs[i];
        if (s.q_tokens < 0 || s.res_tokens < 0 || s.q_tokens % res_cap != 0 || s.res_tokens > res_cap ||
            s.q_tokens + s.res_tokens > 0x7fffffff - 4096) {
            ctx->set_error("kivi attention: sequence %d: q_tokens must be a multiple of res_cap and res_tokens <= res_cap", i);
            return ARGUS_B200_E_INVALID;
        }
        if (s.q_tokens > 0 && (!s.qk || !s.qv || (reinterpret_cast<uintptr_t>(s.qk) & 15) ||
                               (reinterpret_cast<uintptr_t>(s.qv) & 15))) {
            ctx->set_error("kivi attention: sequence %d: packed K/V must be 16-byte aligned", i);
            return ARGUS_B200_E_INVALID;
        }
        if (s.res_tokens > 0 && (!s.res_k || !s.res_v)) {
            ctx->set_error("kivi attention: sequence %d: residual pointers are null", i);
            return ARGUS_B200_E_INVALID;
        }
        bt.qk[i] = static_cast<const uint8_t*>(s.qk);
        bt.qv[i] = static_cast<const uint8_t*>(s.qv);
        bt.res_k[i] = s.res_k;
        bt.res_v[i] = s.res_v;
        if (flush_pages) {
            if (s.q_tokens > 0 && !flush_pages[i]) {
                ctx->set_error("kivi attention: sequence %d: page table is null", i);
                return ARGUS_B200_E_INVALID;
            }
            bt.flush_pages[i] = flush_pages[i];
        }
        bt.q_tokens[i] = (int32_t)s.q_tokens;
        bt.res_tokens[i] = (int32_t)s.res_tokens;
        qlens[i] = s.q_tokens;
        max_len = std::max(max_len, s.q_tokens + s.res_tokens);
        max_res = std::max(max_res, s.res_tokens);
    }
    // A very long residual window (the bits==16 "residual only" mode of the container) gets longer chunks.
    while ((max_res + bt.res_chunk - 1) / bt.res_chunk > 64) bt.res_chunk *= 2;

    const bool want_scores = ex && (ex->scores || ex->head_scores || ex->flat_scores || ex->scores_host);
    if (want_scores && ex->score_stride < max_len) {
        ctx->set_error("kivi attention: score_stride %lld is shorter than the longest sequence %lld",
                       (long long)ex->score_stride, (long long)max_len);
        return ARGUS_B200_E_INVALID;
    }

    // Packed part: the same proportional planner as the F16 path, in tokens, then expressed in 32-token groups.
    int32_t chunk[kMaxBatch], nsplit[kMaxBatch];
    // The planner fills decode_kivi_plan_slots_per_sm() CTA slots per SM (measured there); ARGUS_B200_KIVI_WAVES / _SLOTS
    // override for experiments.
    const int waves = ctx->opt.kivi_waves > 0 ? ctx->opt.kivi_waves : 1;
    const int slots_per_sm = ctx->opt.kivi_slots > 0 ? ctx->opt.kivi_slots : decode_kivi_plan_slots_per_sm(d, bits);
    plan_splits(qlens, n_seqs, hkv, ctx->num_sms * slots_per_sm, waves, 4 * 32 * 2, chunk, nsplit);
    int items = 0, res_items = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const int groups = (int)(qlens[i] / 32);
        int cg = std::max(1, (chunk[i] + 31) / 32);
        int nq = groups > 0 ? (groups + cg - 1) / cg : 0;
        const int nr = (int)((bt.res_tokens[i] + bt.res_chunk - 1) / bt.res_chunk);
        if (nq + nr == 0) nq = 1;   // empty sequence: one empty split writes zeros and lse = -inf
        bt.chunk_groups[i] = cg;
        bt.n_qsplits[i] = nq;
        bt.item_start[i] = items;
        bt.res_start[i] = res_items;
        items += nq + nr;
        res_items += nr;
        if (nq + nr > kMaxSplits) {
            ctx->set_error("kivi attention: sequence %d needs %d splits (max %d)", i, nq + nr, kMaxSplits);
            return ARGUS_B200_E_WORKSPACE;
        }
    }
    bt.item_start[n_seqs] = items;
    bt.res_start[n_seqs] = res_items;

    size_t cur = 0;
    if ((size_t)n_seqs * hkv > ctx->n_tickets) return ARGUS_B200_E_WORKSPACE;
    float* part_o = ctx->scratch(&cur, (size_t)items * hkv * 8 * d * sizeof(float));
    float* part_ml = ctx->scratch(&cur, (size_t)items * hkv * 8 * sizeof(float2));
    float* lse2 = ctx->scratch(&cur, (size_t)n_seqs * hq * sizeof(float));
    float* logits = nullptr;
    float* scores_dev = ex ? ex->scores : nullptr;
    int64_t logit_stride = 0;
    if (want_scores) {
        logit_stride = ex->score_stride;
        if (scores_dev) logits = scores_dev;
        else {
            logits = ctx->scratch(&cur, (size_t)n_seqs * hq * logit_stride * sizeof(float));
            if (ex->scores_host) scores_dev = logits;
        }
    }
    if (!part_o || !part_ml || !lse2 || (want_scores && !logits)) {
        ctx->set_error("kivi attention: scratch of %zu bytes is too small for this call", ctx->ws_bytes);
        return ARGUS_B200_E_WORKSPACE;
    }

    DecodeParams p;
    memset(&p, 0, sizeof(p));
    p.q = q;
    p.out = out;
    p.lse = ex ? ex->lse : nullptr;
    p.n_seqs = n_seqs;
    p.hq = hq;
    p.hkv = hkv;
    p.group = g;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.part_o = part_o;
    p.part_ml = reinterpret_cast<float2*>(part_ml);
    p.tickets = ctx->tickets;
    p.logits = logits;
    p.logit_stride = logit_stride;
    p.lse2 = lse2;
    p.status = ctx->status;

    cudaError_t e = launch_decode_kivi(p, bt, d, bits, items, st);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "decode_kivi launch");
    ctx->launches += 1;

    if (want_scores) {
        FinalizeParams f;
        memset(&f, 0, sizeof(f));
        f.logits = logits;
        f.logit_stride = logit_stride;
        f.lse2 = lse2;
        f.scores = scores_dev;
        f.head_scores = ex->head_scores;
        f.flat_scores = ex->flat_scores;
        f.score_stride = ex->score_stride;
        f.n_seqs = n_seqs;
        f.hq = hq;
        f.hkv = hkv;
        f.group = g;
        for (int i = 0; i < n_seqs; ++i) f.seq_len[i] = bt.q_tokens[i] + bt.res_tokens[i];
        e = launch_finalize_scores(f, (int)max_len, st);
        if (e != cudaSuccess) return ctx->cuda_fail(e, "finalize_scores launch");
        ctx->launches += 1;
        if (ex->scores_host) {
            e = cudaMemcpyAsync(ex->scores_host, scores_dev, (size_t)n_seqs * hq * ex->score_stride * sizeof(float),
                                cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) return ctx->cuda_fail(e, "score read-back");
        }
    }
    return ARGUS_B200_OK;
}

}  // namespace argus

using argus::Context;
static inline Context* C_(argus_b200_ctx* c) { return reinterpret_cast<Context*>(c); }

extern "C" {

int argus_b200_kivi_has_quant_attn_kernel(const argus_b200_ctx* ctx, int bits) {
    return (ctx && (bits == 2 || bits == 4 || bits == 8)) ? 1 : 0;
}

int argus_b200_kivi_attention_batched(argus_b200_ctx* ctx, void* stream, const float* q, const argus_b200_kivi_seq* seqs,
                                      int n_seqs, float* out, int num_heads_q, int num_heads_kv, int head_dim,
                                      int res_cap, int bits, int res_dtype, float scale,
                                      const argus_b200_decode_extras* extras) {
    return argus::kivi_entry(C_(ctx), static_cast<cudaStream_t>(stream), q, seqs, n_seqs, out, num_heads_q, num_heads_kv,
                             head_dim, res_cap, bits, res_dtype, scale, extras, nullptr);
}

int argus_b200_kivi_attention_paged(argus_b200_ctx* ctx, void* stream, const float* q, const void* qk_pool,
                                    const void* qv_pool, const argus_b200_kivi_paged_seq* seqs, int n_seqs, float* out,
                                    int num_heads_q, int num_heads_kv, int head_dim, int res_cap, int bits,
                                    int res_dtype, float scale, const argus_b200_decode_extras* extras) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    if (!seqs || n_seqs <= 0 || n_seqs > argus::kMaxBatch) {
        C_(ctx)->set_error("kivi paged attention: null sequence table or more than %d sequences", argus::kMaxBatch);
        return ARGUS_B200_E_INVALID;
    }
    argus_b200_kivi_seq flat[argus::kMaxBatch];
    const int32_t* tables[argus::kMaxBatch];
    for (int i = 0; i < n_seqs; ++i) {
        flat[i].qk = qk_pool;
        flat[i].qv = qv_pool;
        flat[i].res_k = seqs[i].res_k;
        flat[i].res_v = seqs[i].res_v;
        flat[i].q_tokens = seqs[i].q_tokens;
        flat[i].res_tokens = seqs[i].res_tokens;
        tables[i] = seqs[i].flush_pages;
    }
    return argus::kivi_entry(C_(ctx), static_cast<cudaStream_t>(stream), q, flat, n_seqs, out, num_heads_q, num_heads_kv,
                             head_dim, res_cap, bits, res_dtype, scale, extras, tables);
}

int argus_b200_kivi_attention_gen_quant(argus_b200_ctx* ctx, const argus_b200_quant_attn_args* a) {
    if (!ctx || !a) return ARGUS_B200_E_INVALID;
    if (a->num_heads_q == 0 || a->num_heads_kv == 0) {
        C_(ctx)->set_error("attention_gen_quant: num_heads_q/kv must be > 0");
        return ARGUS_B200_E_INVALID;
    }
    argus_b200_kivi_seq s;
    s.qk = reinterpret_cast<const void*>(a->qk_mem);
    s.qv = reinterpret_cast<const void*>(a->qv_mem);
    s.res_k = reinterpret_cast<const void*>(a->res_k_mem);
    s.res_v = reinterpret_cast<const void*>(a->res_v_mem);
    s.q_tokens = (int64_t)a->q_tokens;
    s.res_tokens = (int64_t)a->res_tokens;
    argus_b200_decode_extras ex;
    memset(&ex, 0, sizeof(ex));
    const bool want = a->scores_out != nullptr && a->scores_len > 0;
    if (want) {
        ex.scores_host = a->scores_out;
        ex.score_stride = (int64_t)(a->scores_len / a->num_heads_q);
    }
    return argus::kivi_entry(C_(ctx), static_cast<cudaStream_t>(a->cu_stream), reinterpret_cast<const float*>(a->q_mem),
                             &s, 1, reinterpret_cast<float*>(a->out_mem), (int)a->num_heads_q, (int)a->num_heads_kv,
                             (int)a->head_dim, (int)a->res_cap, a->bits, ARGUS_B200_KV_F32, a->scale, want ? &ex : nullptr,
                             nullptr);
}

int argus_b200_kivi_gather_update_quant(argus_b200_ctx* ctx, const argus_b200_quant_gather_args* a) {
    if (!ctx || !a) return ARGUS_B200_E_INVALID;
    if (a->res_pos + a->seq_len > a->res_cap) {
        C_(ctx)->set_error("gather_update_quant: res_pos + seq_len exceeds res_cap");
        return ARGUS_B200_E_INVALID;
    }
    cudaError_t e = argus::launch_kivi_gather_update(reinterpret_cast<const float*>(a->input_mem),
                                                     reinterpret_cast<float*>(a->residual_mem), (int)a->kv_heads,
                                                     (int)a->res_cap, (int)a->head_dim, (int)a->seq_len, (int)a->res_pos,
                                                     static_cast<cudaStream_t>(a->cu_stream));
    if (e != cudaSuccess) return C_(ctx)->cuda_fail(e, "gather_update launch");
    C_(ctx)->launches += (a->seq_len > 0);
    return ARGUS_B200_OK;
}

int argus_b200_kivi_dequant_flush(argus_b200_ctx* ctx, const argus_b200_quant_dequant_flush_args* a) {
    if (!ctx || !a) return ARGUS_B200_E_INVALID;
    if (argus::block_bytes(a->bits) < 0 || a->head_dim % 32 != 0) {
        C_(ctx)->set_error("dequant_flush: unsupported bits=%d / head_dim=%zu", a->bits, a->head_dim);
        return ARGUS_B200_E_UNSUPPORTED;
    }
    cudaError_t e = argus::launch_kivi_dequant_flush(reinterpret_cast<const uint8_t*>(a->q_blocks_mem),
                                                     reinterpret_cast<__half*>(a->attn_mem), (int)a->kv_heads,
                                                     (int)a->head_dim, (int)a->n_groups_or_tokens, (int)a->tok_base,
                                                     (long long)a->block_start, a->bits, a->is_key ? 1 : 0,
                                                     static_cast<cudaStream_t>(a->cu_stream));
    if (e != cudaSuccess) return C_(ctx)->cuda_fail(e, "dequant_flush launch");
    C_(ctx)->launches += 1;
    return ARGUS_B200_OK;
}

int argus_b200_kivi_scatter_residual(argus_b200_ctx* ctx, const argus_b200_quant_scatter_residual_args* a) {
    if (!ctx || !a) return ARGUS_B200_E_INVALID;
    cudaError_t e = argus::launch_kivi_scatter_residual(reinterpret_cast<const float*>(a->res_mem),
                                                        reinterpret_cast<__half*>(a->attn_mem), (int)a->kv_heads,
                                                        (int)a->res_cap, (int)a->head_dim, (int)a->res_pos,
                                                        (int)a->tok_base, static_cast<cudaStream_t>(a->cu_stream));
    if (e != cudaSuccess) return C_(ctx)->cuda_fail(e, "scatter_residual launch");
    C_(ctx)->launches += (a->res_pos > 0);
    return ARGUS_B200_OK;
}

int argus_b200_kivi_flush_pack(argus_b200_ctx* ctx, void* stream, const float* res_k, const float* res_v, void* qk,
                               void* qv, int kv_heads, int head_dim, int res_cap, int n_groups, int bits,
                               int64_t k_block_start, int64_t v_block_start) {
    if (!ctx || !res_k || !res_v || !qk || !qv) return ARGUS_B200_E_INVALID;
    if (argus::block_bytes(bits) < 0 || head_dim % 32 != 0 || res_cap % 32 != 0 || n_groups < 0 ||
        n_groups * 32 > res_cap || kv_heads <= 0) {
        C_(ctx)->set_error("flush_pack: bad geometry (bits=%d head_dim=%d res_cap=%d n_groups=%d)", bits, head_dim, res_cap, n_groups);
        return ARGUS_B200_E_INVALID;
    }
    cudaError_t e = argus::launch_kivi_pack(res_k, res_v, static_cast<uint8_t*>(qk), static_cast<uint8_t*>(qv), kv_heads,
                                            head_dim, res_cap, n_groups, bits, k_block_start, v_block_start,
                                            static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return C_(ctx)->cuda_fail(e, "flush_pack launch");
    C_(ctx)->launches += 2 * (n_groups > 0);
    return ARGUS_B200_OK;
}

static int reduce_common(argus_b200_ctx* ctx, const argus_b200_score_reduce_args* a, bool per_layer) {
    if (!ctx || !a) return ARGUS_B200_E_INVALID;
    if (a->n_kv_heads == 0 || a->n_heads_q % a->n_kv_heads != 0 || a->cache_seq_len > a->score_stride ||
        a->cache_seq_len > a->max_seq_len) {
        C_(ctx)->set_error("score_reduce: bad head counts or cache_seq_len beyond the strides");
        return ARGUS_B200_E_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(a->cu_stream);
    cudaError_t e;
    if (per_layer) {
        if (a->layer_flat_importance == 0) return ARGUS_B200_E_INVALID;
        e = argus::launch_score_reduce_per_layer(reinterpret_cast<const float*>(a->score_buf),
                                                 reinterpret_cast<float*>(a->layer_flat_importance), a->decay_factor,
                                                 (int)a->n_layers, (int)a->n_heads_q, (int)a->cache_seq_len,
                                                 (long long)a->score_stride, (long long)a->max_seq_len, st);
    } else {
        if (a->n_kv_heads > 96) return ARGUS_B200_E_UNSUPPORTED;
        e = argus::launch_score_fused_reduce(reinterpret_cast<const float*>(a->score_buf),
                                             reinterpret_cast<float*>(a->importance),
                                             reinterpret_cast<float*>(a->head_importance), a->decay_factor,
                                             (int)a->n_layers, (int)a->n_heads_q, (int)a->n_kv_heads,
                                             (int)a->cache_seq_len, (long long)a->score_stride,
                                             (long long)a->max_seq_len, st);
    }
    if (e != cudaSuccess) return C_(ctx)->cuda_fail(e, "score_reduce launch");
    C_(ctx)->launches += (a->cache_seq_len > 0);
    return ARGUS_B200_OK;
}

int argus_b200_score_reduce(argus_b200_ctx* ctx, const argus_b200_score_reduce_args* a) { return reduce_common(ctx, a, false); }
int argus_b200_score_reduce_per_layer(argus_b200_ctx* ctx, const argus_b200_score_reduce_args* a) {
    return reduce_common(ctx, a, true);
}

int argus_b200_flash_attention_prefill(argus_b200_ctx* ctx, void* stream, const void* q, const void* k_cache,
                                       const void* v_cache, void* out, int n_heads_q, int n_heads_kv, int seq_len,
                                       int cache_seq_len, int head_dim, int64_t kv_capacity, int batch_size,
                                       int is_head_major, int dtype_mode) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    Context* c = C_(ctx);
    c->err[0] = 0;
    if (!q || !k_cache || !v_cache || !out || n_heads_q <= 0 || n_heads_kv <= 0 || n_heads_q % n_heads_kv != 0 ||
        seq_len <= 0 || cache_seq_len < seq_len || kv_capacity < cache_seq_len || batch_size <= 0 || dtype_mode < 0 ||
        dtype_mode > 2) {
        c->set_error("flash_attention_prefill: bad arguments (S=%d T=%d cap=%lld B=%d)", seq_len, cache_seq_len,
                     (long long)kv_capacity, batch_size);
        return ARGUS_B200_E_INVALID;
    }
    if (head_dim != 128) {
        c->set_error("flash_attention_prefill: head_dim %d is declined (128 only)", head_dim);
        return ARGUS_B200_E_UNSUPPORTED;
    }
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
         reinterpret_cast<uintptr_t>(out)) & 15) {
        c->set_error("flash_attention_prefill: pointers must be 16-byte aligned");
        return ARGUS_B200_E_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const void* q16 = q;
    if (dtype_mode == ARGUS_B200_PREFILL_F32Q_F16KV) {
        const long long n = (long long)batch_size * seq_len * n_heads_q * head_dim;
        size_t cur = 0;
        float* buf = c->scratch(&cur, (size_t)n * 2);
        if (!buf) {
            c->set_error("flash_attention_prefill: %lld bytes of scratch needed for the F16 copy of Q", n * 2);
            return ARGUS_B200_E_WORKSPACE;
        }
        cudaError_t e = argus::launch_cast_f32_to_f16(static_cast<const float*>(q), buf, n, st);
        if (e != cudaSuccess) return c->cuda_fail(e, "q cast launch");
        c->launches += 1;
        q16 = buf;
    }
    const int64_t pos_stride = is_head_major ? head_dim : (int64_t)n_heads_kv * head_dim;
    const int64_t head_stride = is_head_major ? kv_capacity * head_dim : head_dim;
    const int64_t batch_stride = kv_capacity * n_heads_kv * head_dim;
    cudaError_t e = argus::launch_prefill_tc(q16, k_cache, v_cache, out, dtype_mode == ARGUS_B200_PREFILL_BF16,
                                             dtype_mode == ARGUS_B200_PREFILL_F32Q_F16KV, batch_size, seq_len,
                                             cache_seq_len, n_heads_q, n_heads_kv, cache_seq_len, pos_stride, head_stride,
                                             batch_stride, c->opt.prefill_bf16_p, c->status, st);
    if (e == cudaErrorNotSupported) {
        c->set_error("flash_attention_prefill: the driver does not export cuTensorMapEncodeTiled");
        return ARGUS_B200_E_UNSUPPORTED;
    }
    if (e != cudaSuccess) return c->cuda_fail(e, "prefill launch");
    c->launches += 1;
    return ARGUS_B200_OK;
}

int argus_b200_lse_merge(argus_b200_ctx* ctx, void* stream, const float* parts, int n_parts, int64_t part_stride,
                         int num_heads_q, int head_dim, float* out, float* lse_out) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    if (!parts || !out || n_parts <= 0 || num_heads_q <= 0 || head_dim <= 0 ||
        part_stride < (int64_t)num_heads_q * head_dim + num_heads_q) {
        C_(ctx)->set_error("lse_merge: bad arguments (n_parts=%d part_stride=%lld)", n_parts, (long long)part_stride);
        return ARGUS_B200_E_INVALID;
    }
    cudaError_t e = argus::launch_lse_merge(parts, n_parts, (long long)part_stride, num_heads_q, head_dim, out, lse_out,
                                            static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return C_(ctx)->cuda_fail(e, "lse_merge launch");
    C_(ctx)->launches += 1;
    return ARGUS_B200_OK;
}

int argus_b200_exchange_wait_merge(argus_b200_ctx* ctx, void* stream, const float* own_part, const argus_b200_exchange* xc,
                                   int step, int num_heads_q, int num_heads_kv, int head_dim, float* out) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    Context* c = C_(ctx);
    c->err[0] = 0;
    if (!own_part || !xc || !out || !xc->peer_lines || xc->n_ranks <= 0 || xc->n_ranks > argus::kMaxRanks || xc->rank < 0 ||
        xc->rank >= xc->n_ranks || step <= 0 || num_heads_q <= 0 || num_heads_kv <= 0 || num_heads_q % num_heads_kv != 0 ||
        head_dim <= 0 || !xc->peer_lines[xc->rank]) {
        c->set_error("exchange_wait_merge: bad arguments (n_ranks=%d rank=%d step=%d)", xc ? xc->n_ranks : 0, xc ? xc->rank : 0,
                     step);
        return ARGUS_B200_E_INVALID;
    }
    argus::ExchangeWaitParams p;
    memset(&p, 0, sizeof(p));
    for (int s = 0; s < xc->n_ranks; ++s) p.xc.lines[s] = xc->peer_lines[s];
    p.xc.merged_lse = xc->merged_lse;
    p.xc.parity_stride_lines = xc->parity_stride_lines;
    p.xc.n_ranks = xc->n_ranks;
    p.xc.rank = xc->rank;
    p.out = out;
    p.status = c->status;
    p.hq = num_heads_q;
    p.hkv = num_heads_kv;
    p.d = head_dim;
    p.step = step;
    cudaError_t e = argus::launch_exchange_wait_merge(p, own_part, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return c->cuda_fail(e, "exchange_wait_merge launch");
    c->launches += 1;
    return ARGUS_B200_OK;
}

int argus_b200_check_status(argus_b200_ctx* ctx, void* stream) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    Context* c = C_(ctx);
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, c->status, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(c->status, 0, sizeof(int), static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return c->cuda_fail(e, "check_status");
    return host;
}

}  // extern "C"
