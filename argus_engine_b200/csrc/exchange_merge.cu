// The receiving half of the sequence-sharded decode's exchange as a kernel of its own: one CTA per KV head waits
// (bounded) for the other ranks' lines of its query heads in this rank's receive buffer and merges them with the
// rank's own rows. The decode kernel does this itself in its epilogue (phases = 3); this kernel exists for callers
// that run the decode with phases = 1 (push only) - single-GPU tests, where all ranks' kernels run one after the other
// and none may wait for a later launch. The reference has no multi-GPU path; the merge algebra is its CPU chunk merge
// (engine/src/backend/cpu/neon.rs:1028-1125).
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "context.h"
#include "decode_epilogue.cuh"
#include "decode_params.h"

namespace argus {

// own_rows: this rank's (o, lse) partial, [Hq][D] outputs then [Hq] lse, as argus_b200_attention_gen writes it.
__global__ void __launch_bounds__(128) exchange_wait_merge_kernel(const __grid_constant__ ExchangeWaitParams p,
                                                                 const float* __restrict__ own_rows) {
    extern __shared__ __align__(16) float xc_rows[];   // [n_ranks][xc_slot_floats]
    __shared__ int ok_flag;
    const int kv = blockIdx.x, g = p.hq / p.hkv, d = p.d, nf = g * (d + 1), nfp = xc_slot_floats(g, d);
    const long long poff = (p.step & 1) ? p.xc.parity_stride_lines : 0;
    for (int e = threadIdx.x; e < nf; e += 128) {
        const int h0 = kv * g;
        xc_rows[p.xc.rank * nfp + e] = (e < g * d) ? own_rows[(long long)h0 * d + e] : own_rows[(long long)p.hq * d + h0 + (e - g * d)];
    }
    const bool ok = xc_wait_merge<128>(p.xc, xc_rows, &ok_flag, kv, p.hq, p.hkv, g, d, p.step, poff, p.out, p.xc.merged_lse);
    if (!ok && threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, 3);
}

cudaError_t launch_exchange_wait_merge(const ExchangeWaitParams& p, const float* own_rows, cudaStream_t st) {
    const int g = p.hq / p.hkv;
    const size_t smem = (size_t)p.xc.n_ranks * xc_slot_floats(g, p.d) * sizeof(float);
    static bool attr_done[kMaxDevices] = {};
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(exchange_wait_merge_kernel), 96 * 1024, attr_done);
    if (e != cudaSuccess) return e;
    if (smem > 96 * 1024) return cudaErrorInvalidValue;
    exchange_wait_merge_kernel<<<p.hkv, 128, smem, st>>>(p, own_rows);
    return cudaGetLastError();
}

}  // namespace argus
