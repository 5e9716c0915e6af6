// Internal: the object behind argus_b200_ctx and the kernel launchers the entry points call.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/argus_b200.h"
#include "decode_params.h"

namespace argus {

struct Context {
    int device = 0;
    int num_sms = 148;
    uint8_t* ws = nullptr;      // scratch: partials, log-sum-exp, logit scratch
    size_t ws_bytes = 0;
    int* tickets = nullptr;     // arrival counters of the split merge; all zero between calls
    size_t n_tickets = 0;
    uint64_t launches = 0;
    char err[512] = {0};

    void set_error(const char* fmt, ...);
    int cuda_fail(cudaError_t e, const char* what);
    float* scratch(size_t* cursor, size_t bytes);
};

void plan_splits(const int64_t* lens, int n, int hkv, int slots, int waves, int min_chunk, int32_t* chunk,
                 int32_t* nsplit);

// decode_f16.cu
int decode_f16_cta_tokens(int head_dim);
cudaError_t launch_decode_f16(const DecodeParams& p, const DecodeBatch& bt, int head_dim, int n_items, cudaStream_t st);
cudaError_t launch_finalize_scores(const FinalizeParams& f, int max_len, cudaStream_t st);

}  // namespace argus
