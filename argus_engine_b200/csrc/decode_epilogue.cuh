// Shared tail of the split-KV decode kernels: merge the warps of a CTA, publish the CTA's partial, and let
// the last CTA of a (sequence, KV head) merge all splits. Same algebra as the reference's chunk merge
// (engine/src/backend/cpu/neon.rs:1028-1125): M = max m_c, L = sum exp(m_c-M) l_c, O = sum exp(m_c-M) O_c,
// out = O / L, here in the log2 domain.
#pragma once
#include "decode_params.h"
#include "ptx.cuh"

namespace argus {

template <int D, int WARPS>
struct EpilogueSmem {
    static constexpr int O_OFF = 0;                              // float [WARPS][8][D]
    static constexpr int ML_OFF = WARPS * 8 * D * 4;             // float2 [WARPS][8]
    static constexpr int FLAG_OFF = ML_OFF + WARPS * 8 * 8;      // int
    static constexpr int WARP_MERGE_B = FLAG_OFF + 128;
    static constexpr int SPLIT_MERGE_B = kMaxSplits * 8 * 8 + 8 * 8;   // (m,l) table + totals
    static constexpr int BYTES = WARP_MERGE_B > SPLIT_MERGE_B ? WARP_MERGE_B : SPLIT_MERGE_B;
};

// Flag words of the peer exchange are written and read with release / acquire semantics at system scope.
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Sequence-sharded decode, run by every thread of the CTA that completed KV head `kv` after it has written the head
// group's normalised rows and their natural-log lse into this rank's OWN slot of its receive buffer:
//   push  - copy the g rows + lse into slot `rank` of every other rank's receive buffer with plain peer stores (no
//           multicast, no bulk copy), fence at system scope, then raise flag[rank][head] = step on every rank;
//   merge - wait, with an iteration limit, for flag[s][head] >= step of every rank s in this rank's own flag array
//           and merge the n_ranks rows of each head (same algebra as the split merge above, natural-log lse).
// Only data of this CTA's own heads is waited for, so no CTA of a launch depends on another CTA of the same launch
// and ranks only depend on pushes, which never wait. A wait that runs out zeroes the heads' output and sets the
// status word to 3. Requires Hq % 4 == 0 and parity strides that are multiples of 4 (16-byte rows).
template <int D, int WARPS>
__device__ __forceinline__ void peer_exchange_tail(const DecodeParams& p, int kv, int step, long long poff, long long foff) {
    constexpr int NT = WARPS * 32;
    const PeerExchange& x = p.xc;
    const int hq = p.hq, g = p.group, h0 = kv * g;
    const long long part_len = (long long)hq * D + hq;
    __shared__ int xc_ok;
    if (threadIdx.x == 0) xc_ok = 1;
    __syncthreads();   // the rows and lse written by this CTA are visible to all its threads
    if (x.phases & 1) {
        const float* own = x.parts[x.rank] + poff + x.rank * part_len;
        const int n4 = g * D / 4;
        for (int s = 0; s < x.n_ranks; ++s) {
            if (s == x.rank) continue;
            float* dst = x.parts[s] + poff + x.rank * part_len;
            for (int e = threadIdx.x; e < n4; e += NT)
                reinterpret_cast<float4*>(dst + (long long)h0 * D)[e] = __ldcg(reinterpret_cast<const float4*>(own + (long long)h0 * D) + e);
            if (threadIdx.x < g) dst[(long long)hq * D + h0 + threadIdx.x] = __ldcg(own + (long long)hq * D + h0 + threadIdx.x);
        }
        __threadfence_system();
        __syncthreads();
        for (int i = threadIdx.x; i < x.n_ranks * g; i += NT) {
            __threadfence_system();
            st_release_sys(x.flags[i / g] + foff + x.rank * hq + h0 + (i % g), step);
        }
    }
    if (x.phases & 2) {
        for (int i = threadIdx.x; i < x.n_ranks * g; i += NT) {
            const int* f = x.flags[x.rank] + foff + (i / g) * hq + h0 + (i % g);
            bool ok = false;
            for (int it = 0; it < (1 << 21); ++it) {   // about a second before giving up
                if (ld_acquire_sys(f) >= step) {
                    ok = true;
                    break;
                }
                if (it > 2048) __nanosleep(256);
            }
            __threadfence_system();
            if (!ok) {
                xc_ok = 0;
                if (p.status != nullptr) atomicExch(p.status, 3);
            }
        }
        __syncthreads();
        const bool ok_all = xc_ok != 0;
        const float* parts = x.parts[x.rank] + poff;
        for (int e = threadIdx.x; e < g * D; e += NT) {
            const int h = h0 + e / D, c = e % D;
            float M = -INFINITY;
            for (int s = 0; s < x.n_ranks; ++s) {
                const float l = __ldcv(parts + s * part_len + (long long)hq * D + h);
                if (isfinite(l) && l > M) M = l;
            }
            float W = 0.f, acc = 0.f;
            for (int s = 0; s < x.n_ranks; ++s) {
                const float l = __ldcv(parts + s * part_len + (long long)hq * D + h);
                if (isfinite(l)) {
                    const float w = expf(l - M);
                    W += w;
                    acc += w * __ldcv(parts + s * part_len + (long long)h * D + c);
                }
            }
            p.out[(long long)h * D + c] = (ok_all && W > 0.f) ? acc / W : 0.f;
            if (c == 0 && x.merged_lse != nullptr) x.merged_lse[h] = (ok_all && W > 0.f) ? M + logf(W) : -INFINITY;
        }
    }
    __syncthreads();   // every thread has read the step counter's old value (the caller did) and is done with it
    if (threadIdx.x == 0) x.step_ctr[kv] = step;
}

// Precondition: every warp has stored its un-normalised O tile at smem[O_OFF] as [warp][8][D] and its
// (running max, sum) at smem[ML_OFF] as [warp][8], followed by __syncthreads().
// item  = index of this CTA's partial, item0 = partial of split 0 of the same (sequence, KV head);
// consecutive splits are p.hkv partials apart.
// UNR = split partials each thread keeps in flight per float4 slice in the final merge (registers: 4*UNR per slice).
template <int D, int WARPS, int UNR = 16>
__device__ __forceinline__ void decode_epilogue(uint8_t* smem, const DecodeParams& p, int b, int kv, int64_t item,
                                                int64_t item0, int n_splits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* sm_o = reinterpret_cast<float*>(smem + EpilogueSmem<D, WARPS>::O_OFF);
    float2* sm_ml = reinterpret_cast<float2*>(smem + EpilogueSmem<D, WARPS>::ML_OFF);
    int* sm_flag = reinterpret_cast<int*>(smem + EpilogueSmem<D, WARPS>::FLAG_OFF);
    // Sharded decode: the completing CTA writes the final rows into its own slot of the receive buffer (the buffer set
    // follows the parity of the step number kept in device memory), then pushes and merges (peer_exchange_tail).
    const bool xchg = p.xc.n_ranks > 0;
    float* out_base = p.out;
    float* lse_base = p.lse;
    int xc_step = 0;
    long long xc_poff = 0, xc_foff = 0;
    auto bind_exchange = [&]() {
        xc_step = __ldcg(p.xc.step_ctr + kv) + 1;
        xc_poff = (xc_step & 1) ? p.xc.parts_parity_stride : 0;
        xc_foff = (xc_step & 1) ? p.xc.flags_parity_stride : 0;
        out_base = p.xc.parts[p.xc.rank] + xc_poff + p.xc.rank * ((long long)p.hq * D + p.hq);
        lse_base = out_base + (long long)p.hq * D;
    };
    if (xchg && n_splits == 1) bind_exchange();
    for (int e = threadIdx.x; e < p.group * D; e += WARPS * 32) {
        const int h = e / D, d = e % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_ml[w * 8 + h].x);
        const float Mu = (M == -INFINITY) ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float2 ml = sm_ml[w * 8 + h];
            const float f = fast_exp2(ml.x - Mu);
            L += f * ml.y;
            acc += f * sm_o[(w * 8 + h) * D + d];
        }
        if (n_splits == 1) {
            const int64_t oh = (int64_t)b * p.hq + kv * p.group + h;
            out_base[oh * D + d] = (L > 0.f) ? acc / L : 0.f;
            if (d == 0) {
                const float l2 = (L > 0.f) ? M + log2f(L) : -INFINITY;
                if (lse_base != nullptr) lse_base[oh] = l2 * 0.6931471805599453f;
                if (p.lse2 != nullptr) p.lse2[oh] = l2;
            }
        } else {
            p.part_o[(item * 8 + h) * D + d] = acc;
            if (d == 0) p.part_ml[item * 8 + h] = make_float2(M, L);
        }
    }
    if (n_splits == 1) {
        if (xchg) peer_exchange_tail<D, WARPS>(p, kv, xc_step, xc_poff, xc_foff);
        return;
    }

    // ── ticket: the last split of this (sequence, KV head) merges all of them ──
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(&p.tickets[b * p.hkv + kv], 1);
        *sm_flag = (prev == n_splits - 1);
    }
    __syncthreads();
    if (*sm_flag == 0) return;
    __threadfence();
    if (xchg) bind_exchange();

    // All (max, sum) pairs of this (sequence, KV head) come into shared memory once; everything else
    // is computed from there. The planner keeps n_splits <= kMaxSplits.
    float2* sm_pm = reinterpret_cast<float2*>(smem);                       // [n_splits][8]
    float2* sm_ML = reinterpret_cast<float2*>(smem + kMaxSplits * 8 * 8);  // [8]
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_splits * 8; idx += WARPS * 32) {
        const int s = idx >> 3, h = idx & 7;
        sm_pm[idx] = (h < p.group) ? __ldcg(&p.part_ml[(item0 + (int64_t)s * p.hkv) * 8 + h]) : make_float2(-INFINITY, 0.f);
    }
    __syncthreads();
    for (int h = warp; h < p.group; h += WARPS) {
        float M = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, sm_pm[s * 8 + h].x);
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, sh));
        const float Mu = (M == -INFINITY) ? 0.f : M;
        float L = 0.f;
        for (int s = lane; s < n_splits; s += 32) {
            const float2 ml = sm_pm[s * 8 + h];
            const float f = fast_exp2(ml.x - Mu);
            L += f * ml.y;
            sm_pm[s * 8 + h].x = f;   // the max is no longer needed: keep the rescale factor instead
        }
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) L += __shfl_xor_sync(0xffffffffu, L, sh);
        if (lane == 0) sm_ML[h] = make_float2(M, L);
    }
    __syncthreads();
    // out = sum_s f_s * O_s / L with splits in ascending order (fixed order => run-to-run identical bits).
    // Each thread owns float4 slices of the [group][D] tile and keeps UNR loads per slice in flight: this CTA is the
    // last one of its KV head, so every round trip to L2 here is at the end of the kernel's critical path.
    constexpr int V4 = (8 * D / 4) / (WARPS * 32);   // float4 slices per thread at the full group of 8
    float4 acc[V4];
#pragma unroll
    for (int k = 0; k < V4; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int n_vec = p.group * D / 4;
    const float4* po = reinterpret_cast<const float4*>(p.part_o + item0 * 8 * D);
    const int64_t sstride = (int64_t)p.hkv * 8 * D / 4;
    for (int s0 = 0; s0 < n_splits; s0 += UNR) {
        float4 v[V4][UNR];
#pragma unroll
        for (int k = 0; k < V4; ++k) {
            const int e = threadIdx.x + k * WARPS * 32;
#pragma unroll
            for (int u = 0; u < UNR; ++u)
                v[k][u] = (e < n_vec && s0 + u < n_splits) ? __ldcg(po + (s0 + u) * sstride + e)
                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < V4; ++k) {
            const int e = threadIdx.x + k * WARPS * 32;
            const int h = (e * 4) / D;
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const float f = (e < n_vec && s0 + u < n_splits) ? sm_pm[(s0 + u) * 8 + h].x : 0.f;
                acc[k].x += f * v[k][u].x; acc[k].y += f * v[k][u].y;
                acc[k].z += f * v[k][u].z; acc[k].w += f * v[k][u].w;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < V4; ++k) {
        const int e = threadIdx.x + k * WARPS * 32;
        if (e >= n_vec) continue;
        const int h = (e * 4) / D, d = (e * 4) % D;
        const float2 ML = sm_ML[h];
        const float inv = (ML.y > 0.f) ? 1.0f / ML.y : 0.f;
        const int64_t oh = (int64_t)b * p.hq + kv * p.group + h;
        *reinterpret_cast<float4*>(out_base + oh * D + d) =
            make_float4(acc[k].x * inv, acc[k].y * inv, acc[k].z * inv, acc[k].w * inv);
        if (d == 0) {
            const float l2 = (ML.y > 0.f) ? ML.x + log2f(ML.y) : -INFINITY;
            if (lse_base != nullptr) lse_base[oh] = l2 * 0.6931471805599453f;
            if (p.lse2 != nullptr) p.lse2[oh] = l2;
        }
    }
    if (threadIdx.x == 0) p.tickets[b * p.hkv + kv] = 0;   // ready for the next call
    if (xchg) peer_exchange_tail<D, WARPS>(p, kv, xc_step, xc_poff, xc_foff);
}

}  // namespace argus
