// Launch parameters shared by the split-KV decode kernels (F16 cache and KIVI-packed cache), the
// score finalize kernel and the host planner.
#pragma once
#include <stdint.h>

namespace argus {

constexpr int kMaxBatch = 64;   // sequences per launch (descriptor table travels as a kernel parameter)
constexpr int kMaxGroup = 8;    // query heads per KV head handled by one MMA row block
constexpr int kMaxSplits = 512; // splits of one sequence (bounds the merge table in shared memory)

// Work decomposition: item = (sequence b, split s of that sequence, kv head). Items of sequence b
// start at item_start[b]; it has item_start[b+1]-item_start[b] splits of chunk[b] tokens (the last one ragged).
// blockIdx.x enumerates items as ((item_start[b] + s) * Hkv + kv).
struct DecodeBatch {
    const void* k[kMaxBatch];
    const void* v[kMaxBatch];
    int64_t head_stride[kMaxBatch];  // elements
    int64_t pos_stride[kMaxBatch];   // elements
    int32_t seq_len[kMaxBatch];
    int32_t chunk[kMaxBatch];           // tokens per split of this sequence (multiple of 16)
    int32_t item_start[kMaxBatch + 1];  // prefix sum of splits per sequence
    // Paged caches (page_tokens > 0): k/v point at page pools; token t of sequence b lives in page
    // page_table[b][t / page_tokens] at row t % page_tokens: base + page*page_stride + head*head_stride + row*pos_stride.
    const int32_t* page_table[kMaxBatch];
    int64_t page_stride;                // elements
    int32_t page_tokens;                // multiple of 16, so that a 16-token warp tile never straddles two pages
};

// KIVI-packed sequences. Splits [0, n_qsplits[b]) of sequence b cover chunk_groups[b] 32-token groups of the
// packed part each; the remaining splits cover res_chunk tokens of the residual window each. The grid runs the
// residual splits of ALL sequences first (res_start = their prefix sum) and the packed splits after them: a residual
// split is the slowest CTA per token, and one that starts last is a tail nothing overlaps.
struct KiviBatch {
    const uint8_t* qk[kMaxBatch];
    const uint8_t* qv[kMaxBatch];
    const void* res_k[kMaxBatch];   // [Hkv][res_cap][D] F32 or F16
    const void* res_v[kMaxBatch];
    const int32_t* flush_pages[kMaxBatch];   // paged form: flush f of sequence b lives in page flush_pages[b][f]; null = flush f
    int32_t q_tokens[kMaxBatch];
    int32_t res_tokens[kMaxBatch];
    int32_t chunk_groups[kMaxBatch];
    int32_t n_qsplits[kMaxBatch];
    int32_t item_start[kMaxBatch + 1];
    int32_t res_start[kMaxBatch + 1];
    int32_t res_cap;
    int32_t res_chunk;
    int32_t res_is_f16;
};

// Sequence-sharded decode (one sequence, one KV slice per GPU): the CTA that completes a KV head pushes the head
// group's normalised rows and lse into slot `rank` of every rank's receive buffer and (phase 2) collects the other
// ranks' rows from its own buffer and merges. n_ranks == 0 switches all of it off. Layout: decode_epilogue.cuh.
constexpr int kMaxRanks = 16;
struct PeerExchange {
    void* lines[kMaxRanks];          // receive buffer of every rank: 2 sets of [n_ranks][Hkv][lines_per_head] 16-byte lines
    int* step_ctr;                   // [Hkv] step counters in this rank's memory; the completing CTA of a KV head bumps its own
    float* merged_lse;               // [Hq] natural-log lse of the merged result, nullable
    long long parity_stride_lines;   // lines between the even-step and the odd-step buffer set
    int n_ranks, rank, phases;       // phases: 1 = push, 2 = wait + merge, 3 = both
};

struct DecodeParams {
    const float* q;   // [B][Hq][D]
    float* out;       // [B][Hq][D]
    float* lse;       // [B][Hq] natural log, nullable
    int n_seqs, hq, hkv, group;
    float scale_log2; // (1/sqrt(D)) * log2(e)
    // split-KV scratch
    float* part_o;    // [items][Hkv][group_pad=8][D] un-normalised partial outputs
    float2* part_ml;  // [items][Hkv][8] (running max in log2 units, partial sum)
    int* tickets;     // [B][Hkv] arrival counters, zero between calls
    // score export: raw scaled logits (log2 units) written at logits[(b*Hq + h)*logit_stride + t]
    float* logits;    // nullable
    int64_t logit_stride;
    float* lse2;      // [B][Hq] log2-domain lse for the finalize kernel (nullable unless logits set)
    int* status;      // set to 1 by a kernel whose bounded wait ran out (nullable)
    // decode step (write the new token's row, then attend): F32 rows [B][Hkv][D] that the CTA owning the last split of a
    // (sequence, KV head) rounds to F16 and stores at position seq_len-1 before it starts reading (nullable)
    const float* k_new;
    const float* v_new;
    PeerExchange xc;  // sequence-sharded decode only
};

// Finalize: p = exp2(logit - lse2) and its reductions over the GQA group.
struct FinalizeParams {
    const float* logits;  // [B][Hq][logit_stride]; may alias `scores`
    int64_t logit_stride;
    const float* lse2;    // [B][Hq]
    float* scores;        // [B][Hq][score_stride] nullable
    float* head_scores;   // [B][Hkv][score_stride] nullable
    float* flat_scores;   // [B][score_stride] nullable
    int64_t score_stride;
    int n_seqs, hq, hkv, group;
    int32_t seq_len[kMaxBatch];
};

// Wait + merge of a sequence-sharded decode as a kernel of its own (exchange_merge.cu): the second half of the
// exchange for callers that ran the decode with phases = 1.
struct ExchangeWaitParams {
    PeerExchange xc;
    float* out;      // [Hq][D]
    int* status;
    int hq, hkv, d, step;
};

}  // namespace argus
