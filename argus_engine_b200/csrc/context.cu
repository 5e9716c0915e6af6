// Host side of the C ABI: context, scratch management, split planning and argument checking.
//
// This is the B200-native counterpart of the host code in CudaBackend::attention_gen
// (engine/src/backend/cuda_pc.rs:1693-1885): pointer/dtype gates, launch shape, score-buffer binding
// and the blocking score read-back — minus the run-time nvcc step, since kernels are ahead-of-time
// sm_100a code, and with a split-KV plan instead of one CTA per query head.
#include "context.h"
#include "decode_epilogue.cuh"

#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

namespace argus {

void Context::set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, sizeof(err), fmt, ap);
    va_end(ap);
}

int Context::cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return ARGUS_B200_E_CUDA;
}

// Scratch is carved from one allocation made at create time; nothing on the decode path allocates.
float* Context::scratch(size_t* cursor, size_t bytes) {
    const size_t at = (*cursor + 255) & ~size_t(255);
    if (at + bytes > ws_bytes - ws_tail_reserved) return nullptr;
    *cursor = at + bytes;
    return reinterpret_cast<float*>(ws + at);
}

// Split planning. Every (split, KV head) is a CTA. The split budget S = slots*waves/Hkv is shared out in
// proportion to the sequence lengths, so that all splits of a batch are close to the same length and a wave
// of CTAs starts and ends together; leftover splits go to the sequences whose splits are longest. A split
// is never shorter than `min_chunk` tokens (pipeline fill) and a sequence never has more than kMaxSplits.
void plan_splits(const int64_t* lens, int n, int hkv, int slots, int waves, int min_chunk, int32_t* chunk,
                 int32_t* nsplit) {
    int64_t total = 0;
    for (int i = 0; i < n; ++i) total += lens[i];
    const int64_t S = std::max<int64_t>(1, (int64_t)slots * waves / hkv);
    const double ideal = std::max<double>(min_chunk, (double)total / (double)S);
    int64_t used = 0;
    for (int i = 0; i < n; ++i) {
        int64_t k = (int64_t)((double)lens[i] / ideal);
        k = std::min<int64_t>(std::max<int64_t>(k, 1), kMaxSplits);
        nsplit[i] = (int32_t)k;
        used += k;
    }
    while (used < S) {
        int best = -1;
        double best_len = 0.0;
        for (int i = 0; i < n; ++i) {
            const double per = (double)lens[i] / nsplit[i];
            if (per > best_len && nsplit[i] < kMaxSplits && lens[i] / (nsplit[i] + 1) >= min_chunk) {
                best_len = per;
                best = i;
            }
        }
        if (best < 0) break;
        nsplit[best] += 1;
        used += 1;
    }
    for (int i = 0; i < n; ++i) {
        int64_t c = (lens[i] + nsplit[i] - 1) / nsplit[i];
        c = std::max<int64_t>(16, ((c + 15) / 16) * 16);
        chunk[i] = (int32_t)c;
        nsplit[i] = (int32_t)std::max<int64_t>(1, (lens[i] + c - 1) / c);
    }
}

int env_int(const char* name, int dflt) {
    const char* s = getenv(name);
    return (s && *s) ? atoi(s) : dflt;
}

int decode_f16_entry(Context* ctx, cudaStream_t st, const float* q, const argus_b200_seq* seqs, int n_seqs,
                     float* out, int hq, int hkv, int d, int kv_dtype, const argus_b200_decode_extras* ex,
                     const PagedInfo* paged, const argus_b200_exchange* xc, const float* k_new, const float* v_new) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    if (!q || !seqs || !out || n_seqs <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || d <= 0) {
        ctx->set_error("attention_gen: null pointer or bad head counts (hq=%d hkv=%d d=%d n_seqs=%d)", hq, hkv, d, n_seqs);
        return ARGUS_B200_E_INVALID;
    }
    if (n_seqs > kMaxBatch) {
        ctx->set_error("attention_gen: %d sequences exceed the per-launch maximum of %d", n_seqs, kMaxBatch);
        return ARGUS_B200_E_INVALID;
    }
    const int g = hq / hkv;
    if ((kv_dtype != ARGUS_B200_KV_F16 && kv_dtype != ARGUS_B200_KV_F32) || (d != 64 && d != 128) || g > kMaxGroup) {
        ctx->set_error("attention_gen: unsupported (kv_dtype=%d head_dim=%d group=%d)", kv_dtype, d, g);
        return ARGUS_B200_E_UNSUPPORTED;
    }
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) {
        ctx->set_error("attention_gen: q/out must be 16-byte aligned");
        return ARGUS_B200_E_INVALID;
    }

    DecodeBatch bt;
    memset(&bt, 0, sizeof(bt));
    if (paged) {
        if (kv_dtype != ARGUS_B200_KV_F16 || paged->page_tokens <= 0 || paged->page_tokens % 16 != 0 ||
            (paged->page_stride & 7) || !paged->page_tables) {
            ctx->set_error("attention_gen_paged: F16 pools, page_tokens a positive multiple of 16 and a page stride that is a "
                           "multiple of 8 elements are required");
            return ARGUS_B200_E_UNSUPPORTED;
        }
        bt.page_tokens = paged->page_tokens;
        bt.page_stride = paged->page_stride;
    }
    int64_t lens[kMaxBatch];
    int64_t max_len = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const argus_b200_seq& s = seqs[i];
        if (s.seq_len < 0 || s.seq_len > 0x7fffffff - 4096) {
            ctx->set_error("attention_gen: sequence %d has an invalid length", i);
            return ARGUS_B200_E_INVALID;
        }
        if (s.seq_len > 0) {
            if (!s.k || !s.v || (reinterpret_cast<uintptr_t>(s.k) & 15) || (reinterpret_cast<uintptr_t>(s.v) & 15) ||
                (s.head_stride & (kv_dtype == ARGUS_B200_KV_F16 ? 7 : 3)) || (s.pos_stride & (kv_dtype == ARGUS_B200_KV_F16 ? 7 : 3)) ||
                s.pos_stride < d) {
                ctx->set_error("attention_gen: sequence %d: K/V must be 16-byte aligned with strides that are multiples of 8 elements", i);
                return ARGUS_B200_E_INVALID;
            }
        }
        if (paged) {
            if (s.seq_len > 0 && !paged->page_tables[i]) {
                ctx->set_error("attention_gen_paged: sequence %d has no page table", i);
                return ARGUS_B200_E_INVALID;
            }
            bt.page_table[i] = paged->page_tables[i];
        }
        bt.k[i] = s.k;
        bt.v[i] = s.v;
        bt.head_stride[i] = s.head_stride;
        bt.pos_stride[i] = s.pos_stride;
        bt.seq_len[i] = (int32_t)s.seq_len;
        lens[i] = s.seq_len;
        max_len = std::max(max_len, s.seq_len);
    }

    const bool want_scores = ex && (ex->scores || ex->head_scores || ex->flat_scores || ex->scores_host);
    if (want_scores && ex->score_stride < max_len) {
        ctx->set_error("attention_gen: score_stride %lld is shorter than the longest sequence %lld",
                       (long long)(ex ? ex->score_stride : 0), (long long)max_len);
        return ARGUS_B200_E_INVALID;
    }

    if (xc) {
        // sequence-sharded form: one sequence, the (o, lse) partial goes to the peers from inside the kernel
        if (n_seqs != 1 || paged || want_scores || xc->n_ranks <= 0 || xc->n_ranks > kMaxRanks || xc->rank < 0 ||
            xc->rank >= xc->n_ranks || !xc->peer_lines || !xc->step_counters || (xc->phases & 3) == 0 ||
            xc->parity_stride_lines < (int64_t)xc->n_ranks * hkv * xc_lines_per_head(g, d) || (xc->parity_stride_lines & 7)) {
            ctx->set_error("attention_gen_sharded: one contiguous sequence, no score outputs, 1..%d ranks and a parity stride "
                           "of at least n_ranks*Hkv*lines_per_head units (a multiple of 8) are required", kMaxRanks);
            return ARGUS_B200_E_INVALID;
        }
        if (xc_smem_end(xc->n_ranks, g, d) > (size_t)decode_f16_smem_bytes(d)) {
            ctx->set_error("attention_gen_sharded: %d ranks of %d query heads per KV head do not fit the kernel's shared memory",
                           xc->n_ranks, g);
            return ARGUS_B200_E_UNSUPPORTED;
        }
        for (int s = 0; s < xc->n_ranks; ++s)
            if (!xc->peer_lines[s] || (reinterpret_cast<uintptr_t>(xc->peer_lines[s]) & 127)) {
                ctx->set_error("attention_gen_sharded: receive buffer of rank %d is null or not 128-byte aligned", s);
                return ARGUS_B200_E_INVALID;
            }
    }
    const int waves = ctx->opt.decode_waves > 0 ? ctx->opt.decode_waves : 1;
    const int min_chunk = ctx->opt.decode_min_chunk > 0 ? ctx->opt.decode_min_chunk : 2 * decode_f16_cta_tokens(d);
    int32_t nsplit[kMaxBatch];
    // Two CTAs per SM, except for one long sequence (at least 4096 tokens per CTA even then): one CTA of four warps per
    // SM keeps enough bytes in flight and streams a little faster (1M tokens: 601 us against 620 us; 128K: 87.3 / 88.4),
    // and halves the split partials the last CTA of a KV head has to merge.
    int64_t total_len = 0;
    for (int i = 0; i < n_seqs; ++i) total_len += lens[i];
    const bool one_long = n_seqs == 1 && total_len * hkv >= (int64_t)ctx->num_sms * 4096;
    const int slots_per_sm = ctx->opt.decode_slots > 0 ? ctx->opt.decode_slots : (one_long ? 1 : 2);
    plan_splits(lens, n_seqs, hkv, ctx->num_sms * slots_per_sm, waves, min_chunk, bt.chunk, nsplit);
    int items = 0;
    for (int i = 0; i < n_seqs; ++i) {
        bt.item_start[i] = items;
        items += nsplit[i];
    }
    bt.item_start[n_seqs] = items;

    // scratch carve-up
    size_t cur = 0;
    if (kv_dtype == ARGUS_B200_KV_F32) {
        // F32 cache: the kernel runs on a packed F16 HeadMajor copy made in scratch
        for (int i = 0; i < n_seqs; ++i) {
            if (lens[i] == 0) continue;
            const size_t bytes = (size_t)hkv * lens[i] * d * sizeof(__half);
            float* kc = ctx->scratch(&cur, bytes);
            float* vc = ctx->scratch(&cur, bytes);
            if (!kc || !vc) {
                ctx->set_error("attention_gen: the F16 copy of an F32 cache needs more scratch than %zu bytes", ctx->ws_bytes);
                return ARGUS_B200_E_WORKSPACE;
            }
            cudaError_t ce = launch_kv_f32_to_f16(static_cast<const float*>(bt.k[i]), kc, hkv, lens[i], d, bt.head_stride[i],
                                                  bt.pos_stride[i], st);
            if (ce == cudaSuccess)
                ce = launch_kv_f32_to_f16(static_cast<const float*>(bt.v[i]), vc, hkv, lens[i], d, bt.head_stride[i],
                                          bt.pos_stride[i], st);
            if (ce != cudaSuccess) return ctx->cuda_fail(ce, "kv cast launch");
            ctx->launches += 2;
            bt.k[i] = kc;
            bt.v[i] = vc;
            bt.head_stride[i] = lens[i] * d;
            bt.pos_stride[i] = d;
        }
    }
    int* tickets = ctx->tickets;  // persistent, zero between calls
    if ((size_t)n_seqs * hkv > ctx->n_tickets) {
        ctx->set_error("attention_gen: %d ticket slots needed, %zu available", n_seqs * hkv, ctx->n_tickets);
        return ARGUS_B200_E_WORKSPACE;
    }
    float* part_o = ctx->scratch(&cur, (size_t)items * hkv * 8 * d * sizeof(float));
    float* part_ml = ctx->scratch(&cur, (size_t)items * hkv * 8 * sizeof(float2));
    float* lse2 = ctx->scratch(&cur, (size_t)n_seqs * hq * sizeof(float));
    float* logits = nullptr;
    int64_t logit_stride = 0;
    float* scores_dev = ex ? ex->scores : nullptr;
    if (want_scores) {
        logit_stride = ex->score_stride;
        if (scores_dev) {
            logits = scores_dev;   // probabilities replace the logits in place
        } else {
            logits = ctx->scratch(&cur, (size_t)n_seqs * hq * logit_stride * sizeof(float));
            if (ex->scores_host) scores_dev = logits;
        }
    }
    if (!part_o || !part_ml || !lse2 || (want_scores && !logits)) {
        ctx->set_error("attention_gen: scratch of %zu bytes is too small for this call", ctx->ws_bytes);
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
    p.scale_log2 = (1.0f / sqrtf((float)d)) * 1.4426950408889634f;
    p.part_o = part_o;
    p.part_ml = reinterpret_cast<float2*>(part_ml);
    p.tickets = tickets;
    p.logits = logits;
    p.logit_stride = logit_stride;
    p.lse2 = lse2;
    p.status = ctx->status;
    p.k_new = k_new;   // F16 contiguous caches only; the callers route the other cases through the KV write kernel
    p.v_new = v_new;
    if (xc) {
        for (int s = 0; s < xc->n_ranks; ++s) p.xc.lines[s] = xc->peer_lines[s];
        p.xc.step_ctr = xc->step_counters;
        p.xc.merged_lse = xc->merged_lse;
        p.xc.parity_stride_lines = xc->parity_stride_lines;
        p.xc.n_ranks = xc->n_ranks;
        p.xc.rank = xc->rank;
        p.xc.phases = xc->phases & 3;
    }

    cudaError_t e = launch_decode_f16(p, bt, d, items, st);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "decode_f16 launch");
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
        for (int i = 0; i < n_seqs; ++i) f.seq_len[i] = bt.seq_len[i];
        e = launch_finalize_scores(f, (int)max_len, st);
        if (e != cudaSuccess) return ctx->cuda_fail(e, "finalize_scores launch");
        ctx->launches += 1;
        if (ex->scores_host) {
            // Blocking read-back, as the reference does for a host `scores_out`.
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

extern "C" {

int argus_b200_version(void) { return 1; }
int argus_b200_sm_arch(void) { return 100; }

// cuCtxPushCurrent / cuCtxPopCurrent through the runtime's driver entry-point lookup (no link against libcuda).
typedef int (*CtxPushFn)(void*);
typedef int (*CtxPopFn)(void**);
static bool ctx_push(void* cu_context) {
    static CtxPushFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuCtxPushCurrent", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<CtxPushFn>(sym);
    }
    return fn && fn(cu_context) == 0;
}
static void ctx_pop() {
    static CtxPopFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuCtxPopCurrent", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<CtxPopFn>(sym);
    }
    void* old = nullptr;
    if (fn) fn(&old);
}

// Allocations and device queries of a new context; the CUDA context they land in is whatever is current.
static int create_in_current(int device, size_t workspace_bytes, argus_b200_ctx** out) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return ARGUS_B200_E_CUDA;
    if (prop.major != 10) return ARGUS_B200_E_UNSUPPORTED;   // sm_100a code only
    Context* c = new Context();
    c->device = device;
    c->num_sms = prop.multiProcessorCount;
    c->ws_bytes = workspace_bytes ? workspace_bytes : (size_t(64) << 20);
    c->opt.decode_waves = argus::env_int("ARGUS_B200_DECODE_WAVES", 0);
    c->opt.decode_min_chunk = argus::env_int("ARGUS_B200_DECODE_MIN_CHUNK", 0);
    c->opt.decode_slots = argus::env_int("ARGUS_B200_DECODE_SLOTS", 0);
    c->opt.kivi_waves = argus::env_int("ARGUS_B200_KIVI_WAVES", 0);
    c->opt.kivi_slots = argus::env_int("ARGUS_B200_KIVI_SLOTS", 0);
    c->opt.prefill_bf16_p = argus::env_int("ARGUS_B200_PREFILL_BF16_P", 2);
    c->n_tickets = 4096;
    e = cudaMalloc(&c->ws, c->ws_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->tickets, c->n_tickets * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->tickets, 0, c->n_tickets * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&c->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->status, 0, sizeof(int));
    if (e != cudaSuccess) {
        if (c->ws) cudaFree(c->ws);
        if (c->tickets) cudaFree(c->tickets);
        if (c->status) cudaFree(c->status);
        delete c;
        return ARGUS_B200_E_CUDA;
    }
    *out = reinterpret_cast<argus_b200_ctx*>(c);
    return ARGUS_B200_OK;
}

int argus_b200_create(int device, size_t workspace_bytes, argus_b200_ctx** out) {
    if (!out) return ARGUS_B200_E_INVALID;
    *out = nullptr;
    cudaError_t e = cudaSetDevice(device);   // binds the device's primary context
    if (e != cudaSuccess) return ARGUS_B200_E_CUDA;
    return create_in_current(device, workspace_bytes, out);
}

int argus_b200_create_in_context(void* cu_context, int device, size_t workspace_bytes, argus_b200_ctx** out) {
    if (!out) return ARGUS_B200_E_INVALID;
    *out = nullptr;
    if (!cu_context) return ARGUS_B200_E_INVALID;
    if (!ctx_push(cu_context)) return ARGUS_B200_E_CUDA;   // the caller's context: borrowed, never destroyed
    const int rc = create_in_current(device, workspace_bytes, out);
    if (rc == ARGUS_B200_OK) reinterpret_cast<Context*>(*out)->cu_context = cu_context;
    ctx_pop();
    return rc;
}

void argus_b200_destroy(argus_b200_ctx* ctx) {
    Context* c = reinterpret_cast<Context*>(ctx);
    if (!c) return;
    const bool pushed = c->cu_context != nullptr && ctx_push(c->cu_context);
    cudaFree(c->ws);
    cudaFree(c->tickets);
    cudaFree(c->status);
    if (pushed) ctx_pop();
    delete c;
}

const char* argus_b200_last_error(const argus_b200_ctx* ctx) {
    return ctx ? reinterpret_cast<const Context*>(ctx)->err : "null context";
}

uint64_t argus_b200_launch_count(const argus_b200_ctx* ctx) {
    return ctx ? reinterpret_cast<const Context*>(ctx)->launches : 0;
}

int argus_b200_attention_gen_batched(argus_b200_ctx* ctx, void* stream, const float* q, const argus_b200_seq* seqs,
                                     int n_seqs, float* out, int num_heads_q, int num_heads_kv, int head_dim,
                                     int kv_dtype, const argus_b200_decode_extras* extras) {
    return argus::decode_f16_entry(reinterpret_cast<Context*>(ctx), static_cast<cudaStream_t>(stream), q, seqs, n_seqs,
                                   out, num_heads_q, num_heads_kv, head_dim, kv_dtype, extras);
}

int argus_b200_attention_gen_paged(argus_b200_ctx* ctx, void* stream, const float* q, const void* k_pool,
                                   const void* v_pool, const argus_b200_paged_seq* seqs, int n_seqs, float* out,
                                   int num_heads_q, int num_heads_kv, int head_dim, int page_tokens, int64_t page_stride,
                                   int64_t head_stride, int64_t pos_stride, const argus_b200_decode_extras* extras) {
    Context* c = reinterpret_cast<Context*>(ctx);
    if (!c) return ARGUS_B200_E_INVALID;
    if (!seqs || n_seqs <= 0 || n_seqs > argus::kMaxBatch) {
        c->set_error("attention_gen_paged: null sequence table or more than %d sequences", argus::kMaxBatch);
        return ARGUS_B200_E_INVALID;
    }
    argus_b200_seq flat[argus::kMaxBatch];
    const int32_t* tables[argus::kMaxBatch];
    for (int i = 0; i < n_seqs; ++i) {
        flat[i].k = k_pool;
        flat[i].v = v_pool;
        flat[i].seq_len = seqs[i].seq_len;
        flat[i].head_stride = head_stride;
        flat[i].pos_stride = pos_stride;
        tables[i] = seqs[i].page_table;
    }
    argus::PagedInfo pg{tables, page_tokens, page_stride};
    return argus::decode_f16_entry(c, static_cast<cudaStream_t>(stream), q, flat, n_seqs, out, num_heads_q, num_heads_kv,
                                   head_dim, ARGUS_B200_KV_F16, extras, &pg);
}

// Decode step = write the new token's K/V row, then attend over the sequence including it: what the engine's decode
// layer does back to back (engine/src/layers/transformer_layer/forward_gen_fmt.rs:207,267-275). For F16 caches the
// write happens inside the decode kernel (one launch); F32 caches take the KV write kernel first (two launches).
int argus_b200_decode_step_batched(argus_b200_ctx* ctx, void* stream, const float* q, const float* k_new,
                                   const float* v_new, const argus_b200_seq* seqs, const int64_t* capacity, int n_seqs,
                                   float* out, int num_heads_q, int num_heads_kv, int head_dim, int kv_dtype,
                                   const argus_b200_decode_extras* extras) {
    Context* c = reinterpret_cast<Context*>(ctx);
    if (!c) return ARGUS_B200_E_INVALID;
    c->err[0] = 0;
    if (!k_new || !v_new || !seqs || !capacity || n_seqs <= 0 || n_seqs > argus::kMaxBatch ||
        ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new)) & 15)) {
        c->set_error("decode_step: null or misaligned new rows, or more than %d sequences", argus::kMaxBatch);
        return ARGUS_B200_E_INVALID;
    }
    argus_b200_seq after[argus::kMaxBatch];
    for (int i = 0; i < n_seqs; ++i) {
        if (!seqs[i].k || !seqs[i].v || seqs[i].seq_len < 0 || seqs[i].seq_len >= capacity[i]) {
            c->set_error("decode_step: sequence %d: null cache or write position %lld outside capacity %lld", i,
                         (long long)seqs[i].seq_len, (long long)capacity[i]);
            return ARGUS_B200_E_INVALID;
        }
        after[i] = seqs[i];
        after[i].seq_len = seqs[i].seq_len + 1;
    }
    if (kv_dtype != ARGUS_B200_KV_F16) {
        const int rc = argus_b200_kv_scatter_batched(ctx, stream, k_new, v_new, seqs, capacity, n_seqs, kv_dtype, num_heads_kv,
                                                     head_dim);
        if (rc != ARGUS_B200_OK) return rc;
        return argus::decode_f16_entry(c, static_cast<cudaStream_t>(stream), q, after, n_seqs, out, num_heads_q, num_heads_kv,
                                       head_dim, kv_dtype, extras);
    }
    return argus::decode_f16_entry(c, static_cast<cudaStream_t>(stream), q, after, n_seqs, out, num_heads_q, num_heads_kv,
                                   head_dim, kv_dtype, extras, nullptr, nullptr, k_new, v_new);
}

int argus_b200_decode_step(argus_b200_ctx* ctx, void* stream, const float* q, const float* k_new, const float* v_new,
                           void* k_cache, void* v_cache, float* out, int num_heads_q, int num_heads_kv, int head_dim,
                           int64_t cache_seq_len, int64_t capacity, int kv_dtype, int64_t head_stride, int64_t pos_stride,
                           const argus_b200_decode_extras* extras) {
    argus_b200_seq s;
    s.k = k_cache;
    s.v = v_cache;
    s.seq_len = cache_seq_len;
    s.head_stride = head_stride;
    s.pos_stride = pos_stride;
    return argus_b200_decode_step_batched(ctx, stream, q, k_new, v_new, &s, &capacity, 1, out, num_heads_q, num_heads_kv,
                                          head_dim, kv_dtype, extras);
}

int argus_b200_exchange_lines_per_head(int num_heads_q, int num_heads_kv, int head_dim) {
    if (num_heads_q <= 0 || num_heads_kv <= 0 || num_heads_q % num_heads_kv != 0 || head_dim <= 0) return ARGUS_B200_E_INVALID;
    return argus::xc_lines_per_head(num_heads_q / num_heads_kv, head_dim);
}

int argus_b200_attention_gen_sharded(argus_b200_ctx* ctx, void* stream, const float* q, const void* k_shard,
                                     const void* v_shard, float* out, int num_heads_q, int num_heads_kv, int head_dim,
                                     int64_t shard_len, int kv_dtype, int64_t head_stride, int64_t pos_stride,
                                     const argus_b200_exchange* exchange) {
    Context* c = reinterpret_cast<Context*>(ctx);
    if (!c) return ARGUS_B200_E_INVALID;
    if (!exchange) {
        c->set_error("attention_gen_sharded: null exchange descriptor");
        return ARGUS_B200_E_INVALID;
    }
    argus_b200_seq s;
    s.k = k_shard;
    s.v = v_shard;
    s.seq_len = shard_len;
    s.head_stride = head_stride;
    s.pos_stride = pos_stride;
    return argus::decode_f16_entry(c, static_cast<cudaStream_t>(stream), q, &s, 1, out, num_heads_q, num_heads_kv, head_dim,
                                   kv_dtype, nullptr, nullptr, exchange);
}

int argus_b200_attention_gen(argus_b200_ctx* ctx, void* stream, const float* q, const void* k_cache,
                             const void* v_cache, float* out, int num_heads_q, int num_heads_kv, int head_dim,
                             int64_t cache_seq_len, int kv_dtype, int64_t head_stride, int64_t pos_stride,
                             const argus_b200_decode_extras* extras) {
    argus_b200_seq s;
    s.k = k_cache;
    s.v = v_cache;
    s.seq_len = cache_seq_len;
    s.head_stride = head_stride;
    s.pos_stride = pos_stride;
    return argus::decode_f16_entry(reinterpret_cast<Context*>(ctx), static_cast<cudaStream_t>(stream), q, &s, 1, out,
                                   num_heads_q, num_heads_kv, head_dim, kv_dtype, extras);
}

}  // extern "C"
