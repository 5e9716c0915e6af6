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

// Optional time stamps of the exchange tail (compiled in with -DARGUS_XC_PROFILE only): g_xc_prof[kv][stage] in ns.
#ifdef ARGUS_XC_PROFILE
__device__ unsigned long long g_xc_prof[64 * 8];
#define XC_STAMP(i) { if (threadIdx.x == 0 && kv < 64) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_xc_prof[kv * 8 + (i)] = t_; } }
#else
#define XC_STAMP(i)
#endif

// ───────── sequence-sharded decode: exchange of the (o, lse) rows of one KV head's query heads ─────────
// Every 128-byte line that crosses NVLink carries its own arrival flag: 30 data words, then the step number twice.
// A line is written by ONE warp-wide store instruction - eight consecutive lanes store 16 bytes each, which the
// load/store unit turns into one aligned 128-byte write that stays whole on NVLink - and read the same way, so a
// reader that finds `step` in both flag words has the 30 data words of the same write (the property NCCL's LL128
// protocol is built on), with no fence on either side and no separate flag traffic. Flags are step numbers, so
// nothing is ever cleared: a line of the buffer set that step n uses last held step n-2.
// The first form used 16-byte lines {float, step, float, step}: correct by the 8-byte store guarantee alone, but at
// eight ranks 28 900 sixteen-byte writes per rank and step made the tail last 14-16 us (4128 writes at two ranks:
// 5-8 us); a 128-byte line moves 15 times the data per write.
//
// The head group's data is the float sequence [g rows of D outputs | g natural-log lse values] = g*(D+1) floats, 30
// per line; a warp store covers four lines, so the line count is rounded up to a multiple of four. Rank r's receive
// buffer holds, per buffer set, [n_ranks][Hkv][lines_per_head] units of 16 bytes (8 per line), 128-byte aligned.
constexpr int kXcLineWords = 30;
__host__ __device__ constexpr int xc_lines128(int g, int d) { return ((g * (d + 1) + kXcLineWords - 1) / kXcLineWords + 3) & ~3; }
__host__ __device__ constexpr int xc_lines_per_head(int g, int d) { return 8 * xc_lines128(g, d); }
// floats between two ranks' slots in the shared-memory region (a multiple of 4: the rows are written as float4)
__host__ __device__ constexpr int xc_slot_floats(int g, int d) { return (g * (d + 1) + 3) & ~3; }

// Push: `stage` holds this CTA's g*(D+1) floats (shared or global memory); they go to slot `rank` of every other rank.
// Work unit = (peer, four lines); the warps of the CTA take the units in turn.
template <int NT>
__device__ __forceinline__ void xc_push(const PeerExchange& x, const float* stage, int kv, int hkv, int g, int d, int step,
                                        long long poff) {
    const int nf = g * (d + 1), lph = xc_lines_per_head(g, d), quads = xc_lines128(g, d) / 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & 7;
    for (int unit = warp; unit < (x.n_ranks - 1) * quads; unit += NT / 32) {
        const int sp = unit / quads, line = (unit - sp * quads) * 4 + (lane >> 3);
        const int s = sp + (sp >= x.rank ? 1 : 0);
        int w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int word = 4 * sub + k, idx = line * kXcLineWords + word;
            w[k] = word >= kXcLineWords ? step : (idx < nf ? __float_as_int(stage[idx]) : 0);
        }
        int4* dst = static_cast<int4*>(x.lines[s]) + poff + ((long long)x.rank * hkv + kv) * lph + line * 8 + sub;
        // volatile: one 16-byte store per lane, not to be split, merged or deferred by the compiler
        asm volatile("st.volatile.global.v4.s32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                     : "memory");
    }
}

// Wait + merge: collects the other ranks' lines of KV head `kv` from this rank's own receive buffer into `rows`
// ([n_ranks][xc_slot_floats] floats of shared memory; slot `rank` is filled by the caller), every wait bounded, then merges:
// M = max finite lse, w = exp(lse - M), out = sum w*o / sum w (engine/src/backend/cpu/neon.rs:1028-1125 in (o, lse)
// form). Returns false, for every thread, when a line never arrived (the caller reports it; the output is zeroed).
template <int NT>
__device__ __forceinline__ bool xc_wait_merge(const PeerExchange& x, float* rows, int* ok_flag, int kv, int hq, int hkv, int g,
                                              int d, int step, long long poff, float* out, float* merged_lse) {
    const int nf = g * (d + 1), nfp = xc_slot_floats(g, d), lph = xc_lines_per_head(g, d), quads = xc_lines128(g, d) / 4;
    const int h0 = kv * g, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & 7;
    if (threadIdx.x == 0) *ok_flag = 1;
    __syncthreads();
    // Work unit = (peer, four lines) = one warp-wide 16-byte load; kXcLoads units in flight per warp, the lines being
    // independent (one dependent round trip per line and per peer made the wait grow with the number of ranks).
    // Four at a time is the measured optimum at eight ranks (106 us per step): sixteen at a time, with or without a
    // joint retry of everything still pending, gave 108-115 us - the first requests go out before the peers' lines
    // can have arrived and each of them pays another round trip.
    constexpr int kXcLoads = 4;
    const int4* base = static_cast<const int4*>(x.lines[x.rank]) + poff + (long long)kv * lph + lane;
    const int total = (x.n_ranks - 1) * quads;
    auto load_line = [](const int4* ptr) {
        int4 v;
        asm volatile("ld.volatile.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
        return v;
    };
    auto arrived = [&](const int4& v) {   // lane 8j+7 holds the two flag words of line j of the quad
        return __all_sync(0xffffffffu, sub != 7 || (v.z == step && v.w == step));
    };
    for (int first = warp; first < total; first += (NT / 32) * kXcLoads) {
        int4 v[kXcLoads];
        const int4* src[kXcLoads];
        int slot[kXcLoads], line[kXcLoads];
#pragma unroll
        for (int u = 0; u < kXcLoads; ++u) {
            const int unit = first + u * (NT / 32);
            const int sp = unit < total ? unit / quads : 0;
            slot[u] = sp + (sp >= x.rank ? 1 : 0);
            line[u] = unit < total ? (unit - sp * quads) * 4 + (lane >> 3) : -1;
            src[u] = base + (long long)slot[u] * hkv * lph + (unit < total ? (unit - sp * quads) * 32 : 0);
            if (line[u] >= 0) v[u] = load_line(src[u]);
        }
#pragma unroll
        for (int u = 0; u < kXcLoads; ++u) {
            if (line[u] < 0) continue;   // uniform across the warp
            bool ok = arrived(v[u]);
            // about a second before giving up; once a line of this head has been given up, the others get one more look
            const int limit = *reinterpret_cast<volatile int*>(ok_flag) != 0 ? (1 << 20) : 1;
            for (int it = 0; !ok && it < limit; ++it) {
                if (it > 256) __nanosleep(it > 4096 ? 1000 : 100);
                v[u] = load_line(src[u]);
                ok = arrived(v[u]);
            }
            if (!ok) *ok_flag = 0;
            const int w4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int word = 4 * sub + k, idx = line[u] * kXcLineWords + word;
                if (word < kXcLineWords && idx < nf) rows[slot[u] * nfp + idx] = __int_as_float(w4[k]);
            }
        }
    }
    __syncthreads();
    const bool ok_all = *ok_flag != 0;
    for (int e = threadIdx.x; e < g * d; e += NT) {
        const int r = e / d;
        float M = -INFINITY;
        for (int s = 0; s < x.n_ranks; ++s) {
            const float l = rows[s * nfp + g * d + r];
            if (isfinite(l) && l > M) M = l;
        }
        float W = 0.f, acc = 0.f;
        for (int s = 0; s < x.n_ranks; ++s) {
            const float l = rows[s * nfp + g * d + r];
            if (isfinite(l)) {
                const float w = expf(l - M);
                W += w;
                acc += w * rows[s * nfp + e];
            }
        }
        out[(long long)h0 * d + e] = (ok_all && W > 0.f) ? acc / W : 0.f;
        if (e % d == 0 && merged_lse != nullptr) merged_lse[h0 + r] = (ok_all && W > 0.f) ? M + logf(W) : -INFINITY;
    }
    return ok_all;
}

// Shared-memory region of the exchange inside a decode CTA: behind the split-merge tables, [n_ranks][xc_slot_floats].
constexpr int kXcSmemOff = kMaxSplits * 8 * 8 + 256;
__host__ __device__ constexpr size_t xc_smem_end(int n_ranks, int g, int d) {
    return (size_t)kXcSmemOff + (size_t)n_ranks * xc_slot_floats(g, d) * sizeof(float);
}

// Run by every thread of the CTA that completed KV head `kv`, after it has written the head group's normalised rows
// and lse into slot `rank` of the shared-memory region. Only data of this CTA's own heads is waited for, so no CTA of a
// launch depends on another CTA of the same launch, and ranks only depend on pushes, which never wait.
template <int D, int WARPS>
__device__ __forceinline__ void peer_exchange_tail(uint8_t* smem, const DecodeParams& p, int kv, int step, long long poff) {
    constexpr int NT = WARPS * 32;
    const PeerExchange& x = p.xc;
    const int g = p.group, nfp = xc_slot_floats(g, D);
    float* rows = reinterpret_cast<float*>(smem + kXcSmemOff);
    __shared__ int xc_ok;
    __syncthreads();   // the rows and lse written by this CTA are visible to all its threads
    XC_STAMP(0)
    if (x.phases & 1) xc_push<NT>(x, rows + x.rank * nfp, kv, p.hkv, g, D, step, poff);
    XC_STAMP(1)
    if (x.phases & 2) {
        const bool ok = xc_wait_merge<NT>(x, rows, &xc_ok, kv, p.hq, p.hkv, g, D, step, poff, p.out, x.merged_lse);
        if (!ok && threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, 3);
    }
    __syncthreads();   // every thread has read the step counter's old value (the caller did) and is done with it
    XC_STAMP(2)
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
    // Sharded decode: the completing CTA writes the final rows and lse into slot `rank` of the exchange region in shared
    // memory (rows [g][D], then [g] lse), then pushes and merges (peer_exchange_tail). The buffer set on the peers
    // follows the parity of the step number kept in device memory.
    const bool xchg = p.xc.n_ranks > 0;
    float* out_base = p.out;
    float* lse_base = p.lse;
    int xc_step = 0;
    long long xc_poff = 0;
    auto bind_exchange = [&]() {
        xc_step = __ldcg(p.xc.step_ctr + kv) + 1;
        xc_poff = (xc_step & 1) ? p.xc.parity_stride_lines : 0;
        float* stage = reinterpret_cast<float*>(smem + kXcSmemOff) + p.xc.rank * xc_slot_floats(p.group, D);
        out_base = stage - (long long)kv * p.group * D;            // indexed below with (kv*g + h)*D + d; b is 0 here
        lse_base = stage + p.group * D - (long long)kv * p.group;   // indexed with kv*g + h
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
        if (xchg) peer_exchange_tail<D, WARPS>(smem, p, kv, xc_step, xc_poff);
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
    if (xchg) peer_exchange_tail<D, WARPS>(smem, p, kv, xc_step, xc_poff);
}

}  // namespace argus
