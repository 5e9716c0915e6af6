// Internal: the object behind argus_b200_ctx and the kernel launchers the entry points call.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/argus_b200.h"
#include "decode_params.h"

namespace argus {

struct Context {
    int device = 0;
    void* cu_context = nullptr;   // the caller's CUcontext when created through argus_b200_create_in_context (borrowed)
    int num_sms = 148;
    uint8_t* ws = nullptr;      // scratch: partials, log-sum-exp, logit scratch
    size_t ws_bytes = 0;
    int* tickets = nullptr;     // arrival counters of the split merge; all zero between calls
    size_t n_tickets = 0;
    int* status = nullptr;      // device word set by a kernel whose bounded wait ran out
    uint64_t launches = 0;
    size_t ws_tail_reserved = 0;   // bytes at the top of `ws` a composite call keeps for itself while it calls an entry
    char err[512] = {0};
    // Tuning knobs, read from the environment ONCE at argus_b200_create (0 = the built-in choice).
    struct Options {
        int decode_waves = 0, decode_min_chunk = 0, decode_slots = 0;   // ARGUS_B200_DECODE_{WAVES,MIN_CHUNK,SLOTS}
        int kivi_waves = 0, kivi_slots = 0;                             // ARGUS_B200_KIVI_{WAVES,SLOTS}
        int prefill_bf16_p = 2;                                         // ARGUS_B200_PREFILL_BF16_P
    } opt;

    void set_error(const char* fmt, ...);
    int cuda_fail(cudaError_t e, const char* what);
    float* scratch(size_t* cursor, size_t bytes);
};

// context.cu: the body of argus_b200_attention_gen[_batched]
struct PagedInfo {   // paged form: seqs[i].k / .v are the page pools, strides address a row inside a page
    const int32_t* const* page_tables;   // host array of n_seqs device pointers
    int page_tokens;
    int64_t page_stride;
};
int decode_f16_entry(Context* ctx, cudaStream_t st, const float* q, const argus_b200_seq* seqs, int n_seqs, float* out,
                     int hq, int hkv, int d, int kv_dtype, const argus_b200_decode_extras* ex,
                     const PagedInfo* paged = nullptr, const argus_b200_exchange* xc = nullptr,
                     const float* k_new = nullptr, const float* v_new = nullptr);

// cudaFuncSetAttribute applies to the current device only, so the "already raised" memo of a kernel's dynamic
// shared-memory limit is kept per device (a process may hold one context per GPU).
constexpr int kMaxDevices = 64;
inline cudaError_t ensure_dynamic_smem(const void* kernel, int bytes, bool (&done)[kMaxDevices]) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < kMaxDevices && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < kMaxDevices) done[dev] = true;
    return e;
}

int env_int(const char* name, int dflt);
void plan_splits(const int64_t* lens, int n, int hkv, int slots, int waves, int min_chunk, int32_t* chunk,
                 int32_t* nsplit);

// decode_f16.cu
int decode_f16_cta_tokens(int head_dim);
cudaError_t launch_decode_f16(const DecodeParams& p, const DecodeBatch& bt, int head_dim, int n_items, cudaStream_t st);
cudaError_t launch_finalize_scores(const FinalizeParams& f, int max_len, cudaStream_t st);

// kivi_ops.cu
cudaError_t launch_kivi_pack(const float* res_k, const float* res_v, uint8_t* qk, uint8_t* qv, int hkv, int d,
                             int res_cap, int n_groups, int bits, long long k_block_start, long long v_block_start,
                             cudaStream_t st);
cudaError_t launch_kivi_dequant_flush(const uint8_t* q, __half* attn, int hkv, int d, int n, int tok_base,
                                      long long block_start, int bits, int is_key, cudaStream_t st);
cudaError_t launch_kivi_scatter_residual(const float* res, __half* attn, int hkv, int res_cap, int d, int res_pos,
                                         int tok_base, cudaStream_t st);
cudaError_t launch_kivi_gather_update(const float* in, float* res, int hkv, int res_cap, int d, int seq_len, int res_pos,
                                      cudaStream_t st);
// score_reduce.cu
cudaError_t launch_score_fused_reduce(const float* scores, float* importance, float* head_importance, float decay,
                                      int n_layers, int hq, int hkv, int T, long long stride, long long max_seq,
                                      cudaStream_t st);
cudaError_t launch_score_reduce_per_layer(const float* scores, float* layer_flat, float decay, int n_layers, int hq,
                                          int T, long long stride, long long max_seq, cudaStream_t st);
// prefill_sm100.cu
cudaError_t launch_prefill_tc(const void* q16, const void* k, const void* v, void* out, bool bf16, bool out_f32, int B,
                              int S, int T, int hq, int hkv, int64_t cap_rows, int64_t kv_pos_stride,
                              int64_t kv_head_stride, int64_t kv_batch_stride, int p_mode, int* status, cudaStream_t st);
cudaError_t launch_cast_f32_to_f16(const float* src, void* dst, long long n, cudaStream_t st);
// exchange_merge.cu
cudaError_t launch_exchange_wait_merge(const ExchangeWaitParams& p, const float* own_rows, cudaStream_t st);
int decode_f16_smem_bytes(int head_dim);
// kv_cast.cu
cudaError_t launch_kv_f32_to_f16(const float* src, void* dst, int hkv, long long T, int d, long long head_stride,
                                 long long pos_stride, cudaStream_t st);
// kv_ops.cu
cudaError_t launch_kv_scatter(const float* k_src, const float* v_src, void* k_dst, void* v_dst, bool dst_f16, int hkv,
                              int d, long long head_stride, long long pos_stride, long long write_pos, long long seq_len,
                              cudaStream_t st);
cudaError_t launch_kv_scatter_rows(const float* k_src, const float* v_src, void* const* k_dst, void* const* v_dst,
                                   const long long* head_stride, const long long* pos_stride, const long long* write_pos,
                                   int n, bool dst_f16, int hkv, int d, cudaStream_t st);
cudaError_t launch_kv_compact_pass(void* cache, void* scratch, const int* keep, long long i0, long long n_rows,
                                   long long write_start, int head0, int n_heads, int row_bytes, long long head_stride_bytes,
                                   long long pos_stride_bytes, int first, long long capacity, int* status,
                                   cudaStream_t st);
cudaError_t launch_kv_prefix_rows(void* cache, void* packed, long long n_tok, int hkv, int row_bytes,
                                  long long head_stride_bytes, long long pos_stride_bytes, int to_packed, cudaStream_t st);
cudaError_t launch_kv_weighted_merge(void* k, void* v, bool f16, int hkv, int d, long long head_stride,
                                     long long pos_stride, const int* into_pos, const float* into_w, const int* from_start,
                                     const int* from_pos, const float* from_w, int n_merges, int do_k, int do_v,
                                     cudaStream_t st);
cudaError_t launch_d2o_nearest(const void* k, bool f16, long long head_stride, long long pos_stride, int hkv, int d,
                               const int* evict, int n_evict, const int* retain, int n_retain, float* norms,
                               unsigned long long* best, int* nearest, float* sim_out, cudaStream_t st);
cudaError_t launch_pfa_reduce(const float* rows, float* sum_out, float* mean_out, int n_rows, int hq, long long prefix_len,
                              long long row0_pos, int window, cudaStream_t st);
// lse_merge.cu
cudaError_t launch_lse_merge(const float* parts, int n_parts, long long part_stride, int hq, int d, float* out,
                             float* lse_out, cudaStream_t st);
// decode_kivi.cu
cudaError_t launch_decode_kivi(const DecodeParams& p, const KiviBatch& bt, int head_dim, int bits, int n_items,
                               cudaStream_t st);
int decode_kivi_ctas_per_sm(int head_dim, int bits);
int decode_kivi_plan_slots_per_sm(int head_dim, int bits);
}  // namespace argus
