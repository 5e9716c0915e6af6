// Merge of (o, lse) partials from the ranks of a sequence-sharded decode.
//
// Same algebra as the reference's chunk merge (engine/src/backend/cpu/neon.rs:1028-1125) in the (o, lse) form:
// M = max over finite lse_r, w_r = exp(lse_r - M), out = sum w_r o_r / sum w_r; ranks with a non-finite lse
// (empty shards) are skipped, and if every rank is empty the output is zero. The reference has no multi-GPU
// path; this kernel runs on every rank after the gather has placed all partials in the rank's own memory.
//
// Layout of one rank's partial: `part_stride` floats = [Hq][D] normalised outputs followed by [Hq] lse values.
#include <cuda_runtime.h>
#include <math.h>

namespace argus {

__global__ void lse_merge_kernel(const float* __restrict__ parts, int n_parts, long long part_stride, int hq, int d,
                                 float* __restrict__ out, float* __restrict__ lse_out) {
    const int h = blockIdx.x;
    float M = -INFINITY;
    for (int r = 0; r < n_parts; ++r) {
        const float l = parts[r * part_stride + (long long)hq * d + h];
        if (isfinite(l) && l > M) M = l;
    }
    float W = 0.f;
    for (int r = 0; r < n_parts; ++r) {
        const float l = parts[r * part_stride + (long long)hq * d + h];
        if (isfinite(l)) W += expf(l - M);
    }
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < n_parts; ++r) {
            const float l = parts[r * part_stride + (long long)hq * d + h];
            if (isfinite(l)) acc += expf(l - M) * parts[r * part_stride + (long long)h * d + c];
        }
        out[(long long)h * d + c] = (W > 0.f) ? acc / W : 0.f;
    }
    if (lse_out != nullptr && threadIdx.x == 0) lse_out[h] = (W > 0.f) ? M + logf(W) : -INFINITY;
}

cudaError_t launch_lse_merge(const float* parts, int n_parts, long long part_stride, int hq, int d, float* out,
                             float* lse_out, cudaStream_t st) {
    lse_merge_kernel<<<hq, d < 128 ? 64 : 128, 0, st>>>(parts, n_parts, part_stride, hq, d, out, lse_out);
    return cudaGetLastError();
}

}  // namespace argus
