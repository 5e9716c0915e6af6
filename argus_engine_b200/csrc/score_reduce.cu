// Attention-score (H2O/D2O) accumulator kernels.
//
// Stand behind CudaScoreReduceBackend::{reduce, reduce_per_layer}
// (crates/argus-extension-api/src/lib.rs:2938-2948; the kernels they replace are
// kernel_score_fused_reduce{,_per_layer}, crates/techniques/attn-score/src/score_reduce.cu:13-91).
// Policy, unchanged: per token, head sum and GQA group mean per layer, MAX across layers (from 0),
// cumulative = cumulative*decay_factor + step. Sums run over heads in ascending order in F32 and the decay is a
// rounded product followed by a rounded sum, exactly as the reference's CPU producer does it (AttnScoreProducer:
// multiply at begin_step, add at end_step; crates/techniques/attn-score/src/lib.rs:175-359), so the result is
// bit-identical to the CPU producer for the same score buffer and the keep-set selection that reads these
// buffers sees the same numbers. The reference's CUDA kernel, built with nvcc's default contraction, fuses the
// product and the sum into one FMA: with a decay factor whose product is inexact (0.9, not 1.0 or 0.5) it can
// differ from the CPU producer, and from this kernel, by one ulp.
//
// One thread per token (loads of a (layer, head) row are coalesced across the warp); the head loop is
// unrolled so that eight row loads are in flight per thread, and there is no 16-KV-head limit because the
// per-head maxima live in shared memory, not in a fixed stack array.
#include <cuda_runtime.h>
#include <stdint.h>

namespace argus {

constexpr int kReduceThreads = 128;

__global__ void __launch_bounds__(kReduceThreads)
score_fused_reduce_kernel(const float* __restrict__ scores, float* __restrict__ importance,
                          float* __restrict__ head_importance, float decay_factor, int n_layers, int hq, int hkv,
                          int T, long long score_stride, long long max_seq) {
    extern __shared__ float step_head[];   // [hkv][kReduceThreads]
    const int t = blockIdx.x * kReduceThreads + threadIdx.x;
    if (t >= T) return;
    const int g = hq / hkv;
    const float inv = 1.0f / (float)g;
    for (int kv = 0; kv < hkv; ++kv) step_head[kv * kReduceThreads + threadIdx.x] = 0.0f;
    float step_flat = 0.0f;
    for (int l = 0; l < n_layers; ++l) {
        const float* base = scores + (long long)l * hq * score_stride + t;
        float flat = 0.0f;
        for (int kv = 0; kv < hkv; ++kv) {
            float gsum = 0.0f;
            int r = 0;
            for (; r + 8 <= g; r += 8) {
                float w[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) w[u] = __ldg(base + (long long)(kv * g + r + u) * score_stride);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    flat += w[u];
                    gsum += w[u];
                }
            }
            for (; r < g; ++r) {
                const float w = __ldg(base + (long long)(kv * g + r) * score_stride);
                flat += w;
                gsum += w;
            }
            float* sh = &step_head[kv * kReduceThreads + threadIdx.x];
            *sh = fmaxf(*sh, gsum * inv);
        }
        step_flat = fmaxf(step_flat, flat);
    }
    importance[t] = __fadd_rn(__fmul_rn(importance[t], decay_factor), step_flat);   // decay, then add: two roundings like the CPU producer
    for (int kv = 0; kv < hkv; ++kv) {
        const long long idx = (long long)kv * max_seq + t;
        head_importance[idx] = __fadd_rn(__fmul_rn(head_importance[idx], decay_factor), step_head[kv * kReduceThreads + threadIdx.x]);
    }
}

__global__ void __launch_bounds__(kReduceThreads)
score_reduce_per_layer_kernel(const float* __restrict__ scores, float* __restrict__ layer_flat, float decay_factor,
                              int n_layers, int hq, int T, long long score_stride, long long max_seq) {
    const int t = blockIdx.x * kReduceThreads + threadIdx.x;
    const int l = blockIdx.y;
    if (t >= T) return;
    const float* base = scores + (long long)l * hq * score_stride + t;
    float s = 0.0f;
    for (int h = 0; h < hq; ++h) s += __ldg(base + (long long)h * score_stride);
    const long long idx = (long long)l * max_seq + t;
    layer_flat[idx] = __fadd_rn(__fmul_rn(layer_flat[idx], decay_factor), s);
}

cudaError_t launch_score_fused_reduce(const float* scores, float* importance, float* head_importance, float decay,
                                      int n_layers, int hq, int hkv, int T, long long stride, long long max_seq,
                                      cudaStream_t st) {
    if (T <= 0) return cudaSuccess;
    const size_t smem = (size_t)hkv * kReduceThreads * sizeof(float);
    score_fused_reduce_kernel<<<(T + kReduceThreads - 1) / kReduceThreads, kReduceThreads, smem, st>>>(
        scores, importance, head_importance, decay, n_layers, hq, hkv, T, stride, max_seq);
    return cudaGetLastError();
}

cudaError_t launch_score_reduce_per_layer(const float* scores, float* layer_flat, float decay, int n_layers, int hq,
                                          int T, long long stride, long long max_seq, cudaStream_t st) {
    if (T <= 0 || n_layers <= 0) return cudaSuccess;
    dim3 grid((T + kReduceThreads - 1) / kReduceThreads, n_layers);
    score_reduce_per_layer_kernel<<<grid, kReduceThreads, 0, st>>>(scores, layer_flat, decay, n_layers, hq, T, stride,
                                                                  max_seq);
    return cudaGetLastError();
}

}  // namespace argus
