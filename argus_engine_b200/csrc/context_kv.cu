// C-ABI entry points of the KV write and eviction executors (kv_ops.cu).
#include <stdint.h>
#include <string.h>

#include <algorithm>

#include "context.h"

using namespace argus;

namespace {

int elt_bytes(int dtype) { return dtype == ARGUS_B200_KV_F16 ? 2 : dtype == ARGUS_B200_KV_F32 ? 4 : -1; }

// Rows are moved as 16-byte vectors: base pointers, the row pitch and the head pitch must allow that.
bool rows_are_vector_aligned(const void* k, const void* v, int64_t head_stride, int64_t pos_stride, int d, int eb) {
    return ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0 && (head_stride * eb) % 16 == 0 &&
           (pos_stride * eb) % 16 == 0 && ((int64_t)d * eb) % 16 == 0;
}

}  // namespace

extern "C" int argus_b200_kv_scatter(argus_b200_ctx* c, void* stream, const float* k_src, const float* v_src, void* k_dst,
                                     void* v_dst, int dst_dtype, int num_heads_kv, int head_dim, int64_t capacity,
                                     int64_t head_stride, int64_t pos_stride, int64_t write_pos, int64_t seq_len) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    const int eb = elt_bytes(dst_dtype);
    if (!k_src || !v_src || !k_dst || !v_dst || eb < 0 || num_heads_kv <= 0 || head_dim <= 0 || seq_len < 0 ||
        write_pos < 0 || write_pos + seq_len > capacity) {
        ctx->set_error("kv_scatter: null pointer, bad dtype, or rows [%lld, %lld) outside capacity %lld",
                       (long long)write_pos, (long long)(write_pos + seq_len), (long long)capacity);
        return ARGUS_B200_E_INVALID;
    }
    if (head_dim % 4 != 0 || ((reinterpret_cast<uintptr_t>(k_src) | reinterpret_cast<uintptr_t>(v_src)) & 15) ||
        ((reinterpret_cast<uintptr_t>(k_dst) | reinterpret_cast<uintptr_t>(v_dst)) & 15) || (head_stride * eb) % 16 ||
        (pos_stride * eb) % 16) {
        ctx->set_error("kv_scatter: head_dim %% 4, 16-byte aligned pointers and row pitches are required");
        return ARGUS_B200_E_UNSUPPORTED;
    }
    cudaError_t e = launch_kv_scatter(k_src, v_src, k_dst, v_dst, dst_dtype == ARGUS_B200_KV_F16, num_heads_kv, head_dim,
                                      head_stride, pos_stride, write_pos, seq_len, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_scatter launch");
    ctx->launches += seq_len > 0 ? 1 : 0;
    return ARGUS_B200_OK;
}

extern "C" int argus_b200_kv_scatter_batched(argus_b200_ctx* c, void* stream, const float* k_src, const float* v_src,
                                             const argus_b200_seq* seqs, const int64_t* capacity, int n_seqs, int dst_dtype,
                                             int num_heads_kv, int head_dim) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    const int eb = elt_bytes(dst_dtype);
    if (!k_src || !v_src || !seqs || !capacity || eb < 0 || n_seqs < 0 || n_seqs > kMaxBatch || num_heads_kv <= 0 ||
        head_dim <= 0) {
        ctx->set_error("kv_scatter_batched: null pointer, bad dtype or more than %d sequences", kMaxBatch);
        return ARGUS_B200_E_INVALID;
    }
    void* kd[kMaxBatch];
    void* vd[kMaxBatch];
    long long hs[kMaxBatch], ps[kMaxBatch], wp[kMaxBatch];
    bool aligned = head_dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(k_src) | reinterpret_cast<uintptr_t>(v_src)) & 15) == 0;
    for (int i = 0; i < n_seqs; ++i) {
        if (!seqs[i].k || !seqs[i].v || seqs[i].seq_len < 0 || seqs[i].seq_len >= capacity[i]) {
            ctx->set_error("kv_scatter_batched: sequence %d: null cache or position %lld outside capacity %lld", i,
                           (long long)seqs[i].seq_len, (long long)capacity[i]);
            return ARGUS_B200_E_INVALID;
        }
        kd[i] = const_cast<void*>(seqs[i].k);
        vd[i] = const_cast<void*>(seqs[i].v);
        hs[i] = seqs[i].head_stride;
        ps[i] = seqs[i].pos_stride;
        wp[i] = seqs[i].seq_len;
        aligned = aligned && ((reinterpret_cast<uintptr_t>(kd[i]) | reinterpret_cast<uintptr_t>(vd[i])) & 15) == 0 &&
                  (hs[i] * eb) % 16 == 0 && (ps[i] * eb) % 16 == 0;
    }
    if (!aligned) {
        ctx->set_error("kv_scatter_batched: head_dim %% 4, 16-byte aligned pointers and row pitches are required");
        return ARGUS_B200_E_UNSUPPORTED;
    }
    cudaError_t e = launch_kv_scatter_rows(k_src, v_src, kd, vd, hs, ps, wp, n_seqs, dst_dtype == ARGUS_B200_KV_F16,
                                           num_heads_kv, head_dim, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_scatter_batched launch");
    ctx->launches += n_seqs > 0 ? 1 : 0;
    return ARGUS_B200_OK;
}

extern "C" int argus_b200_kv_compact(argus_b200_ctx* c, void* stream, void* k, void* v, int kv_dtype, int num_heads_kv,
                                     int head_dim, int64_t capacity, int64_t head_stride, int64_t pos_stride,
                                     const int32_t* keep_dev, int64_t n_keep, int64_t write_start, int head) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    const int eb = elt_bytes(kv_dtype);
    if (!k || !v || eb < 0 || num_heads_kv <= 0 || head_dim <= 0 || n_keep < 0 || write_start < 0 || head < -1 ||
        head >= num_heads_kv || (n_keep > 0 && !keep_dev) || capacity <= 0 || write_start + n_keep > capacity) {
        ctx->set_error("kv_compact: null pointer, bad dtype, head index %d (of %d) or %lld rows from %lld beyond capacity %lld",
                       head, num_heads_kv, (long long)n_keep, (long long)write_start, (long long)capacity);
        return ARGUS_B200_E_INVALID;
    }
    if (n_keep == 0) return ARGUS_B200_OK;   // compact_keep_positions returns early on an empty list
    if (!rows_are_vector_aligned(k, v, head_stride, pos_stride, head_dim, eb)) {
        ctx->set_error("kv_compact: rows must be 16-byte aligned (pointers, head_dim, row and head pitch)");
        return ARGUS_B200_E_UNSUPPORTED;
    }
    const int head0 = head < 0 ? 0 : head, n_heads = head < 0 ? num_heads_kv : 1;
    const int64_t row_bytes = (int64_t)head_dim * eb;
    // Chunks of at most 32768 rows: a chunk whose first row moves at least that far needs no staging, and with an
    // H2O-like keep list the distance passes the chunk length after the first chunk or two.
    const int64_t rows_per_pass = std::min<int64_t>(32768, (int64_t)(ctx->ws_bytes / (size_t)(row_bytes * n_heads)));
    if (rows_per_pass < 1) {
        ctx->set_error("kv_compact: scratch of %zu bytes does not hold one row of every head", ctx->ws_bytes);
        return ARGUS_B200_E_WORKSPACE;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int64_t i0 = 0; i0 < n_keep; i0 += rows_per_pass) {
        const int64_t n = std::min(rows_per_pass, n_keep - i0);
        for (int which = 0; which < 2; ++which) {
            void* cache = which == 0 ? k : v;
            for (int first = 1; first >= 0; --first) {
                cudaError_t e = launch_kv_compact_pass(cache, ctx->ws, keep_dev, i0, n, write_start, head0, n_heads,
                                                       (int)row_bytes, head_stride * eb, pos_stride * eb, first, capacity,
                                                       ctx->status, st);
                if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_compact launch");
                ctx->launches += 1;
            }
        }
    }
    return ARGUS_B200_OK;
}

// Payload of one layer of the session prefix cache: K bytes [Hkv][token_count][D] then V bytes, the packed form of
// extract_packed_bytes / scatter_packed_bytes (engine/src/kv/standard_format.rs:1657-1790). The reference reads the
// whole buffer (capacity rows per head) back to the host and packs there; here only the prefix rows move.
static int prefix_payload(Context* ctx, cudaStream_t st, void* k, void* v, int kv_dtype, int hkv, int d, int64_t capacity,
                          int64_t head_stride, int64_t pos_stride, int64_t token_count, void* buf, size_t buf_bytes,
                          bool to_packed, const char* who) {
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    const int eb = elt_bytes(kv_dtype);
    if (!k || !v || !buf || eb < 0 || hkv <= 0 || d <= 0 || token_count < 0 || capacity <= 0 || token_count > capacity) {
        ctx->set_error("%s: null pointer, bad dtype or token_count %lld beyond capacity %lld", who, (long long)token_count,
                       (long long)capacity);
        return ARGUS_B200_E_INVALID;
    }
    const size_t half = (size_t)hkv * token_count * d * eb;
    if (buf_bytes != 2 * half) {
        ctx->set_error("%s: the payload of %lld tokens is %zu bytes, the buffer has %zu", who, (long long)token_count, 2 * half,
                       buf_bytes);
        return ARGUS_B200_E_INVALID;
    }
    if (token_count == 0) return ARGUS_B200_OK;
    uint8_t* pk = static_cast<uint8_t*>(buf);
    const size_t row = (size_t)d * eb;
    cudaError_t e = cudaSuccess;
    if (pos_stride == d) {
        // rows of a head are contiguous: one pitched copy per tensor (device, pinned or pageable host on the packed side)
        const size_t width = (size_t)token_count * row, pitch = (size_t)head_stride * eb;
        if (to_packed) {
            e = cudaMemcpy2DAsync(pk, width, k, pitch, width, hkv, cudaMemcpyDefault, st);
            if (e == cudaSuccess) e = cudaMemcpy2DAsync(pk + half, width, v, pitch, width, hkv, cudaMemcpyDefault, st);
        } else {
            e = cudaMemcpy2DAsync(k, pitch, pk, width, width, hkv, cudaMemcpyDefault, st);
            if (e == cudaSuccess) e = cudaMemcpy2DAsync(v, pitch, pk + half, width, width, hkv, cudaMemcpyDefault, st);
        }
        if (e != cudaSuccess) return ctx->cuda_fail(e, who);
        return ARGUS_B200_OK;
    }
    if (!rows_are_vector_aligned(k, v, head_stride, pos_stride, d, eb) || (reinterpret_cast<uintptr_t>(buf) & 15) || (half & 15)) {
        ctx->set_error("%s: strided rows need 16-byte aligned pointers, rows and pitches", who);
        return ARGUS_B200_E_UNSUPPORTED;
    }
    e = launch_kv_prefix_rows(k, pk, token_count, hkv, (int)row, head_stride * eb, pos_stride * eb, to_packed ? 1 : 0, st);
    if (e == cudaSuccess)
        e = launch_kv_prefix_rows(v, pk + half, token_count, hkv, (int)row, head_stride * eb, pos_stride * eb, to_packed ? 1 : 0, st);
    if (e != cudaSuccess) return ctx->cuda_fail(e, who);
    ctx->launches += 2;
    return ARGUS_B200_OK;
}

extern "C" int argus_b200_kv_snapshot_prefix(argus_b200_ctx* c, void* stream, const void* k, const void* v, int kv_dtype,
                                             int num_heads_kv, int head_dim, int64_t capacity, int64_t head_stride,
                                             int64_t pos_stride, int64_t token_count, void* dst, size_t dst_bytes) {
    return prefix_payload(reinterpret_cast<Context*>(c), static_cast<cudaStream_t>(stream), const_cast<void*>(k),
                          const_cast<void*>(v), kv_dtype, num_heads_kv, head_dim, capacity, head_stride, pos_stride, token_count,
                          dst, dst_bytes, true, "kv_snapshot_prefix");
}

extern "C" int argus_b200_kv_restore_prefix(argus_b200_ctx* c, void* stream, void* k, void* v, int kv_dtype, int num_heads_kv,
                                            int head_dim, int64_t capacity, int64_t head_stride, int64_t pos_stride,
                                            int64_t token_count, const void* src, size_t src_bytes) {
    return prefix_payload(reinterpret_cast<Context*>(c), static_cast<cudaStream_t>(stream), k, v, kv_dtype, num_heads_kv,
                          head_dim, capacity, head_stride, pos_stride, token_count, const_cast<void*>(src), src_bytes, false,
                          "kv_restore_prefix");
}

// KV residency. The engine's CUDA backend allocates KV buffers as managed memory and lets the driver migrate pages on
// first touch (engine/src/backend/cuda_pc/memory.rs:1-44); a decode kernel that faults pages in while it streams runs
// far below the device-memory rate. argus_b200_kv_make_resident states the preferred location once and prefetches.
extern "C" int argus_b200_kv_make_resident(argus_b200_ctx* c, void* stream, const void* ptr, size_t bytes) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    if (!ptr || bytes == 0) {
        ctx->set_error("kv_make_resident: null pointer or zero size");
        return ARGUS_B200_E_INVALID;
    }
    cudaPointerAttributes at;
    cudaError_t e = cudaPointerGetAttributes(&at, ptr);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_make_resident: pointer attributes");
    if (at.type == cudaMemoryTypeDevice) return ARGUS_B200_OK;   // already where the kernels want it
    if (at.type != cudaMemoryTypeManaged) {
        ctx->set_error("kv_make_resident: the range is neither device nor managed memory");
        return ARGUS_B200_E_UNSUPPORTED;
    }
    e = cudaMemAdvise(ptr, bytes, cudaMemAdviseSetPreferredLocation, ctx->device);
    if (e == cudaSuccess) e = cudaMemPrefetchAsync(ptr, bytes, ctx->device, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_make_resident: advise / prefetch");
    return ARGUS_B200_OK;
}

extern "C" int argus_b200_kv_alloc(argus_b200_ctx* c, size_t bytes, int managed, void** out) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx || !out || bytes == 0) return ARGUS_B200_E_INVALID;
    *out = nullptr;
    cudaError_t e = managed ? cudaMallocManaged(out, bytes, cudaMemAttachGlobal) : cudaMalloc(out, bytes);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_alloc");
    return ARGUS_B200_OK;
}

extern "C" int argus_b200_kv_free(argus_b200_ctx* c, void* ptr) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    if (!ptr) return ARGUS_B200_OK;
    cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_free");
    return ARGUS_B200_OK;
}

extern "C" int argus_b200_kv_weighted_merge(argus_b200_ctx* c, void* stream, void* k, void* v, int kv_dtype,
                                            int num_heads_kv, int head_dim, int64_t head_stride, int64_t pos_stride,
                                            const int32_t* into_pos, const float* into_weight, const int32_t* from_start,
                                            const int32_t* from_pos, const float* from_weight, int n_merges, int axis) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    const int eb = elt_bytes(kv_dtype);
    if (!k || !v || eb < 0 || num_heads_kv <= 0 || num_heads_kv > 65535 || head_dim <= 0 || n_merges < 0 || axis < 0 ||
        axis > 2 || (n_merges > 0 && (!into_pos || !into_weight || !from_start || !from_pos || !from_weight))) {
        ctx->set_error("kv_weighted_merge: null pointer, bad dtype or axis %d", axis);
        return ARGUS_B200_E_INVALID;
    }
    cudaError_t e = launch_kv_weighted_merge(k, v, kv_dtype == ARGUS_B200_KV_F16, num_heads_kv, head_dim, head_stride,
                                             pos_stride, into_pos, into_weight, from_start, from_pos, from_weight,
                                             n_merges, axis != 2, axis != 1, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return ctx->cuda_fail(e, "kv_weighted_merge launch");
    ctx->launches += n_merges > 0 ? 1 : 0;
    return ARGUS_B200_OK;
}

// prefill_attention_scores (engine/src/kv/standard_format.rs:1400-1510): for the trailing q_window query rows of a
// prefill chunk, the exact softmax probabilities of every head over keys 0..=p, summed over the rows and/or kept per
// row. Row r is a single-query decode over the first q_start_pos + r + 1 keys with score export, so the rows run as
// ONE batched decode launch over the same cache (it stays in L2) followed by the accumulation kernel.
extern "C" int argus_b200_prefill_attention_scores(argus_b200_ctx* c, void* stream, const float* q, const void* k_cache,
                                                   const void* v_cache, int kv_dtype, int num_heads_q, int num_heads_kv,
                                                   int head_dim, int seq_len, int cache_seq_len, int64_t head_stride,
                                                   int64_t pos_stride, int q_start_pos, int q_window, int window,
                                                   float* sum_out, float* per_row, int per_row_per_head) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    if (!q || !k_cache || !v_cache || num_heads_q <= 0 || num_heads_kv <= 0 || num_heads_q % num_heads_kv != 0 ||
        head_dim <= 0 || seq_len < 0 || cache_seq_len < 0 || q_start_pos < 0 || q_window < 0 ||
        q_start_pos + seq_len > cache_seq_len) {
        ctx->set_error("prefill_attention_scores: null pointer, bad head counts, or q_start_pos + seq_len (%d + %d) beyond "
                       "cache_seq_len %d", q_start_pos, seq_len, cache_seq_len);
        return ARGUS_B200_E_INVALID;
    }
    if (kv_dtype != ARGUS_B200_KV_F16) {
        ctx->set_error("prefill_attention_scores: F32 caches are not handled here");
        return ARGUS_B200_E_UNSUPPORTED;
    }
    const int qwin = std::min(q_window, seq_len);
    if (qwin == 0 || (!sum_out && !per_row)) return ARGUS_B200_OK;
    const int qwin_start = seq_len - qwin;
    const int64_t prefix = cache_seq_len;
    const size_t row_bytes = (size_t)num_heads_q * prefix * sizeof(float);   // probabilities of one query row
    const bool direct = per_row && per_row_per_head;                          // the caller's buffer has the decode's layout
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // Top of the scratch: decode outputs (discarded) and, unless the caller's per-row buffer can take them, the rows.
    const size_t out_bytes_per_row = (size_t)num_heads_q * head_dim * sizeof(float);
    const size_t budget = ctx->ws_bytes / 2;
    int rows_per_pass = std::min(qwin, kMaxBatch);
    // Sliding window (lo = p - (w-1) > 0 for some row): the rows start at different keys, so each row is its own call on
    // a cache pointer moved to its first key, with its probabilities landing at offset lo of its score row.
    if (window > 0) rows_per_pass = 1;
    if (!direct) rows_per_pass = (int)std::min<size_t>(rows_per_pass, budget / (row_bytes + out_bytes_per_row));
    if (rows_per_pass < 1) {
        ctx->set_error("prefill_attention_scores: scratch of %zu bytes cannot stage one row of %zu bytes", ctx->ws_bytes, row_bytes);
        return ARGUS_B200_E_WORKSPACE;
    }
    const size_t tail = (((size_t)rows_per_pass * (out_bytes_per_row + (direct ? 0 : row_bytes))) + 511) & ~size_t(255);
    if (tail > ctx->ws_bytes) return ARGUS_B200_E_WORKSPACE;
    uint8_t* tail_base = ctx->ws + ((ctx->ws_bytes - tail) & ~size_t(255));
    float* out_buf = reinterpret_cast<float*>(tail_base);
    float* rows_buf = reinterpret_cast<float*>(tail_base + (((size_t)rows_per_pass * out_bytes_per_row + 255) & ~size_t(255)));
    struct Guard {
        Context* c;
        ~Guard() { c->ws_tail_reserved = 0; }
    } guard{ctx};
    ctx->ws_tail_reserved = tail + 256;

    for (int r0 = 0; r0 < qwin; r0 += rows_per_pass) {
        const int nb = std::min(rows_per_pass, qwin - r0);
        float* rows = direct ? per_row + (size_t)r0 * num_heads_q * prefix : rows_buf;
        if (!direct) {
            cudaError_t e = cudaMemsetAsync(rows, 0, (size_t)nb * row_bytes, st);   // keys behind a row's position stay zero
            if (e != cudaSuccess) return ctx->cuda_fail(e, "prefill_attention_scores memset");
        }
        argus_b200_seq seqs[kMaxBatch];
        int64_t lo = 0;   // first visible key (sliding window; one row per pass then)
        if (window > 0) {
            const int64_t pos = (int64_t)q_start_pos + qwin_start + r0;
            lo = std::max<int64_t>(0, pos - (window - 1));
        }
        for (int i = 0; i < nb; ++i) {
            seqs[i].k = static_cast<const __half*>(k_cache) + lo * pos_stride;
            seqs[i].v = static_cast<const __half*>(v_cache) + lo * pos_stride;
            seqs[i].seq_len = (int64_t)q_start_pos + qwin_start + r0 + i + 1 - lo;
            seqs[i].head_stride = head_stride;
            seqs[i].pos_stride = pos_stride;
        }
        argus_b200_decode_extras ex;
        memset(&ex, 0, sizeof(ex));
        ex.scores = rows + lo;
        ex.score_stride = prefix;
        int rc = decode_f16_entry(ctx, st, q + (size_t)(qwin_start + r0) * num_heads_q * head_dim, seqs, nb, out_buf,
                                  num_heads_q, num_heads_kv, head_dim, kv_dtype, &ex);
        if (rc != ARGUS_B200_OK) return rc;
        float* mean = (per_row && !per_row_per_head) ? per_row + (size_t)r0 * prefix : nullptr;
        cudaError_t e = launch_pfa_reduce(rows, sum_out, mean, nb, num_heads_q, prefix, (long long)q_start_pos + qwin_start + r0,
                                          window, st);
        if (e != cudaSuccess) return ctx->cuda_fail(e, "prefill_attention_scores reduce launch");
        ctx->launches += (sum_out || mean) ? 1 : 0;
    }
    return ARGUS_B200_OK;
}

extern "C" int argus_b200_d2o_nearest(argus_b200_ctx* c, void* stream, const void* k_cache, int kv_dtype, int num_heads_kv,
                                      int head_dim, int64_t head_stride, int64_t pos_stride, const int32_t* evict_pos,
                                      int n_evict, const int32_t* retain_pos, int n_retain, int32_t* nearest_out,
                                      float* sim_out) {
    Context* ctx = reinterpret_cast<Context*>(c);
    if (!ctx) return ARGUS_B200_E_INVALID;
    ctx->err[0] = 0;
    const int eb = elt_bytes(kv_dtype);
    if (!k_cache || eb < 0 || num_heads_kv <= 0 || head_dim <= 0 || n_evict < 0 || n_retain < 0 ||
        (n_evict > 0 && (!evict_pos || !nearest_out || !sim_out)) || (n_retain > 0 && !retain_pos)) {
        ctx->set_error("d2o_nearest: null pointer, bad dtype or negative counts");
        return ARGUS_B200_E_INVALID;
    }
    if (head_dim % 32 != 0 || (n_evict + 31) / 32 > 65535) {
        ctx->set_error("d2o_nearest: head_dim must be a multiple of 32 and at most 2M evicted positions per call");
        return ARGUS_B200_E_UNSUPPORTED;
    }
    if (n_evict == 0) return ARGUS_B200_OK;
    size_t cur = 0;
    float* norms = ctx->scratch(&cur, (size_t)(n_evict + n_retain) * sizeof(float));
    float* best = ctx->scratch(&cur, (size_t)n_evict * sizeof(unsigned long long));
    if (!norms || !best) {
        ctx->set_error("d2o_nearest: scratch of %zu bytes is too small", ctx->ws_bytes);
        return ARGUS_B200_E_WORKSPACE;
    }
    cudaError_t e = launch_d2o_nearest(k_cache, kv_dtype == ARGUS_B200_KV_F16, head_stride, pos_stride, num_heads_kv, head_dim,
                                       evict_pos, n_evict, retain_pos, n_retain, norms,
                                       reinterpret_cast<unsigned long long*>(best), nearest_out, sim_out,
                                       static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return ctx->cuda_fail(e, "d2o_nearest launch");
    ctx->launches += n_retain > 0 ? 3 : 2;
    return ARGUS_B200_OK;
}
