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
// packed part each; the remaining splits cover res_chunk tokens of the residual window each.
struct KiviBatch {
    const uint8_t* qk[kMaxBatch];
    const uint8_t* qv[kMaxBatch];
    const void* res_k[kMaxBatch];   // [Hkv][res_cap][D] F32 or F16
    const void* res_v[kMaxBatch];
    int32_t q_tokens[kMaxBatch];
    int32_t res_tokens[kMaxBatch];
    int32_t chunk_groups[kMaxBatch];
    int32_t n_qsplits[kMaxBatch];
    int32_t item_start[kMaxBatch + 1];
    int32_t res_cap;
    int32_t res_chunk;
    int32_t res_is_f16;
};

// Sequence-sharded decode (one sequence, one KV slice per GPU): the CTA that completes a KV head pushes the head
// group's normalised rows and lse into slot `rank` of every rank's receive buffer, raises the flags, and (phase 2)
// waits for all ranks' flags in its own memory and merges. n_ranks == 0 switches all of it off.
constexpr int kMaxRanks = 16;
struct PeerExchange {
    float* parts[kMaxRanks];        // receive buffer [n_ranks][Hq*D+Hq] of every rank (own entry = local memory)
    int* flags[kMaxRanks];          // flag array [n_ranks][Hq] of every rank
    int* step_ctr;                  // [Hkv] step counters in this rank's memory; the completing CTA of a KV head bumps its own
    float* merged_lse;              // [Hq] natural-log lse of the merged result, nullable
    long long parts_parity_stride;  // floats between the even-step and the odd-step receive buffers
    long long flags_parity_stride;  // ints between the even-step and the odd-step flag arrays
    int n_ranks, rank, phases;      // phases: 1 = push, 2 = wait + merge, 3 = both
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

// Peer exchange + merge of a sequence-sharded decode as a kernel of its own (exchange_merge.cu).
struct ExchangeParams {
    float* peer_parts[kMaxRanks];   // receive buffer [n_ranks][Hq*D+Hq] of every rank (own entry = local memory)
    int* peer_flags[kMaxRanks];     // flag array [n_ranks][Hq] of every rank
    const float* local_part;        // this rank's partial: [Hq][D] outputs, then [Hq] lse
    float* out;                     // [Hq][D]
    float* lse_out;                 // [Hq], nullable
    int* status;
    const int* step_dev;            // nullable: step number in device memory (CUDA-graph replay)
    long long parts_parity_stride;  // floats between the even-step and the odd-step receive buffers
    long long flags_parity_stride;  // ints between the even-step and the odd-step flag arrays
    int n_ranks, rank, step, hq, d, phases;
};

}  // namespace argus
