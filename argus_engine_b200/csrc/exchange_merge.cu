// Exchange of (o, lse) partials over NVLink peer memory fused with their merge: one kernel per rank replaces
// "all-gather, then merge" of the sequence-sharded decode. The reference has no multi-GPU path; the merge algebra
// is its CPU chunk merge (engine/src/backend/cpu/neon.rs:1028-1125).
//
// Every rank owns a receive buffer `parts` [n_ranks][Hq*D + Hq] and a flag array [n_ranks][Hq] that its peers can
// address (plain peer stores; no multicast, no TMA). CTA h of rank r
//   1. copies row h of the local partial (D outputs + lse) into slot r of every rank's receive buffer, fences at
//      system scope, and stores the step number into flag[r][h] on every rank;
//   2. waits, with an iteration limit, until flag[s][h] >= step for every rank s in its OWN flag array;
//   3. merges the n_ranks rows of head h from its own receive buffer.
// Heads are independent, so no CTA of a launch waits for another CTA of the same launch. Flags only grow (the
// step number), so nothing is reset; callers alternate between two buffer sets on even and odd steps so that a
// fast rank's next push cannot overwrite what a slow rank is still merging. A wait that runs out sets the status
// word and the head's output to zero. `phases` (1 = push, 2 = wait + merge, 3 = both) lets a single-GPU test run
// the ranks one after the other without any kernel ever waiting for a later launch.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "decode_params.h"

namespace argus {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(128) exchange_merge_kernel(const __grid_constant__ ExchangeParams p) {
    const int h = blockIdx.x;
    const int d = p.d, hq = p.hq;
    const long long part_len = (long long)hq * d + hq;
    // The step number comes from the host, or from device memory when the launch is replayed from a CUDA graph
    // (step_increment_kernel bumps it once per step). Its parity selects one of the two buffer sets.
    const int step = p.step_dev != nullptr ? *p.step_dev : p.step;
    const long long poff = (step & 1) ? p.parts_parity_stride : 0, foff = (step & 1) ? p.flags_parity_stride : 0;
    if (p.phases & 1) {
        for (int s = 0; s < p.n_ranks; ++s) {
            float* dst = p.peer_parts[s] + poff + (long long)p.rank * part_len;
            for (int c = threadIdx.x; c < d; c += blockDim.x) dst[(long long)h * d + c] = p.local_part[(long long)h * d + c];
            if (threadIdx.x == 0) dst[(long long)hq * d + h] = p.local_part[(long long)hq * d + h];
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < p.n_ranks) {
            // release in the thread that stores the flag: the rows stored by the other threads were fenced and
            // ordered before this point by the barrier
            __threadfence_system();
            st_release_sys(p.peer_flags[threadIdx.x] + foff + p.rank * hq + h, step);
        }
    }
    if (!(p.phases & 2)) return;
    __shared__ int ok_all;
    if (threadIdx.x == 0) ok_all = 1;
    __syncthreads();
    if (threadIdx.x < p.n_ranks) {
        const int* f = p.peer_flags[p.rank] + foff + threadIdx.x * hq + h;
        bool ok = false;
        for (int it = 0; it < (1 << 21); ++it) {
            if (ld_acquire_sys(f) >= step) { ok = true; break; }
            __nanosleep(64);
        }
        __threadfence_system();   // acquire in the polling thread, before the barrier hands the rows to the others
        if (!ok) {
            ok_all = 0;
            if (p.status != nullptr) atomicExch(p.status, 3);
        }
    }
    __syncthreads();
    __threadfence_system();
    const float* parts = p.peer_parts[p.rank] + poff;
    float M = -INFINITY;
    for (int s = 0; s < p.n_ranks; ++s) {
        const float l = __ldcv(parts + s * part_len + (long long)hq * d + h);
        if (isfinite(l) && l > M) M = l;
    }
    float W = 0.f;
    for (int s = 0; s < p.n_ranks; ++s) {
        const float l = __ldcv(parts + s * part_len + (long long)hq * d + h);
        if (isfinite(l)) W += expf(l - M);
    }
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < p.n_ranks; ++s) {
            const float l = __ldcv(parts + s * part_len + (long long)hq * d + h);
            if (isfinite(l)) acc += expf(l - M) * __ldcv(parts + s * part_len + (long long)h * d + c);
        }
        p.out[(long long)h * d + c] = (ok_all && W > 0.f) ? acc / W : 0.f;
    }
    if (p.lse_out != nullptr && threadIdx.x == 0) p.lse_out[h] = (ok_all && W > 0.f) ? M + logf(W) : -INFINITY;
}

__global__ void step_increment_kernel(int* step) { *step += 1; }

cudaError_t launch_step_increment(int* step, cudaStream_t st) {
    step_increment_kernel<<<1, 1, 0, st>>>(step);
    return cudaGetLastError();
}

cudaError_t launch_exchange_merge(const ExchangeParams& p, cudaStream_t st) {
    exchange_merge_kernel<<<p.hq, 128, 0, st>>>(p);
    return cudaGetLastError();
}

}  // namespace argus
