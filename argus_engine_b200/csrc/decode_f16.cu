// Split-KV GQA decode attention over an F16 KV cache, sm_100a.
//
// Stands behind Backend::attention_gen (engine/src/backend.rs:284-295; the CUDA kernel it replaces is
// attention_gen_f16kv_naive, engine/src/backend/cuda_pc/kernels.cu:471-540). Same math
// (softmax(q·K^T/sqrt(D))·V per query head, optional post-softmax score export), different shape:
//
//  * one CTA per (sequence, KV head, split of the KV sequence) so that every SM streams K/V, and the
//    whole GQA group of a KV head shares one pass over K/V (the reference re-reads K/V once per query head);
//  * each warp owns 16-token tiles of its CTA's split and a private STAGES-deep cp.async ring
//    (128-bit copies, XOR-swizzled rows), so the main loop has no block-wide barrier;
//  * QK^T and PV run on the tensor cores (mma.sync m16n8k16, F32 accumulate). Rows 0..7 of the A
//    operand carry the F16 rounding of q (resp. p), rows 8..15 the rounding residual, so both products
//    keep ~22 bits of q and p although K/V stay F16;
//  * online softmax in the log2 domain per warp, (max, sum, O) merged across warps in shared memory,
//    across splits by the last CTA to arrive at a per-(sequence, KV head) ticket.
//
// Score export writes the scaled logits; finalize_scores_kernel turns them into probabilities once the
// global log-sum-exp is known.
#include "decode_epilogue.cuh"
#include "context.h"
#include "decode_params.h"
#include "ptx.cuh"

namespace argus {

// Optional phase stamps (compiled in with -DARGUS_XC_PROFILE only): min / max over the CTAs of a launch of the
// globaltimer at CTA entry, first tile ready, end of the tile loop and end of the epilogue.
#ifdef ARGUS_XC_PROFILE
__device__ unsigned long long g_phase_prof[8];
#define PH_STAMP(i) { if (threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
    atomicMin(&g_phase_prof[2 * (i)], t_); atomicMax(&g_phase_prof[2 * (i) + 1], t_); } }
#else
#define PH_STAMP(i)
#endif

template <int D, int WARPS, int STAGES>
struct DecodeF16Cfg {
    static constexpr int WT = 16;                 // tokens per warp tile
    static constexpr int ROW_B = D * 2;           // bytes per K/V row
    static constexpr int CH = D / 8;              // 16-byte chunks per row
    static constexpr int TILE_B = WT * ROW_B;     // one K (or V) tile
    static constexpr int STAGE_B = 2 * TILE_B;    // K tile + V tile
    static constexpr int PIPE_B = WARPS * STAGES * STAGE_B;
    static constexpr int EPI_B = EpilogueSmem<D, WARPS>::BYTES;
    static constexpr int SMEM_B = PIPE_B > EPI_B ? PIPE_B : EPI_B;
    static constexpr int CTA_TOK = WARPS * WT;    // tokens consumed per CTA sweep
};

template <int D, int WARPS, int STAGES, bool PAGED = false>
__global__ void __launch_bounds__(WARPS * 32, 2)
decode_f16_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ DecodeBatch bt) {
    using Cfg = DecodeF16Cfg<D, WARPS, STAGES>;
    constexpr int WT = Cfg::WT, ROW_B = Cfg::ROW_B, CH = Cfg::CH, TILE_B = Cfg::TILE_B, STAGE_B = Cfg::STAGE_B;
    constexpr int KS = D / 16;   // k-steps of QK^T
    constexpr int NT = D / 8;    // n-tiles of PV
    extern __shared__ __align__(128) uint8_t smem[];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane >> 2, qlane = lane & 3;
    PH_STAMP(0)

    // ── which item ──
    const int kv = blockIdx.x % p.hkv;
    const int gs = blockIdx.x / p.hkv;
    int b = 0;
    while (b + 1 < p.n_seqs && bt.item_start[b + 1] <= gs) ++b;
    const int split = gs - bt.item_start[b];
    const int n_splits = bt.item_start[b + 1] - bt.item_start[b];
    const int T = bt.seq_len[b];
    const int chunk = bt.chunk[b];
    const int t0 = split * chunk;
    const int t1 = min(t0 + chunk, T);
    const int n_tiles = t1 > t0 ? (t1 - t0 + WT - 1) / WT : 0;
    const int my_tiles = warp < n_tiles ? (n_tiles - warp + WARPS - 1) / WARPS : 0;

    const __half* kbase = static_cast<const __half*>(bt.k[b]) + (int64_t)kv * bt.head_stride[b];
    const __half* vbase = static_cast<const __half*>(bt.v[b]) + (int64_t)kv * bt.head_stride[b];
    const int64_t pos_stride = bt.pos_stride[b];
    const uint32_t wsm = smem_u32(smem) + warp * STAGES * STAGE_B;

    // Paged cache: a warp tile (16 tokens from a multiple of 16) lies inside one page. The page number of a tile is
    // loaded one iteration before the tile is issued, so that the lookup never sits in front of the copies.
    const int32_t* ptab = PAGED ? bt.page_table[b] : nullptr;
    const int P = PAGED ? bt.page_tokens : 1;
    auto page_of = [&](int j) -> int { return __ldg(ptab + (t0 + (warp + j * WARPS) * WT) / P); };
    auto issue = [&](int j, int slot, int page) {
        const int tokb = t0 + (warp + j * WARPS) * WT;
        const uint32_t sb = wsm + slot * STAGE_B;
        const int64_t pbase = PAGED ? (int64_t)page * bt.page_stride - (int64_t)(tokb / P) * P * pos_stride : 0;
#pragma unroll
        for (int i = 0; i < (WT * CH) / 32; ++i) {
            const int id = lane + 32 * i;
            const int row = id / CH, c = id % CH;
            const int tok = tokb + row;
            const bool ok = tok < t1;
            const int64_t off = pbase + (int64_t)(ok ? tok : tokb) * pos_stride + c * 8;
            const uint32_t dst = sb + row * ROW_B + ((c ^ (row & 7)) << 4);
            cp_async16(dst, kbase + off, ok);
            cp_async16(dst + TILE_B, vbase + off, ok);
        }
    };

    // Decode step: the new token is position T-1. Only the last split reads it, so the CTA of that split rounds the
    // F32 row to F16 (nearest even, as the engine's KV write kernel does) and stores it before any of its copies is
    // issued; the barrier orders the store before the other threads' reads of the row.
    if (!PAGED && p.k_new != nullptr && split == n_splits - 1 && T > 0) {
        if (threadIdx.x < D / 2) {
            const int64_t src = ((int64_t)b * p.hkv + kv) * D + 2 * threadIdx.x;
            const int64_t dst = (int64_t)(T - 1) * pos_stride + 2 * threadIdx.x;
            const float2 kx = *reinterpret_cast<const float2*>(p.k_new + src);
            const float2 vx = *reinterpret_cast<const float2*>(p.v_new + src);
            *reinterpret_cast<__half2*>(const_cast<__half*>(kbase) + dst) = __floats2half2_rn(kx.x, kx.y);
            *reinterpret_cast<__half2*>(const_cast<__half*>(vbase) + dst) = __floats2half2_rn(vx.x, vx.y);
        }
        __threadfence();
        __syncthreads();
    }

    // ── prologue: start the ring, then fetch q while the copies fly ──
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < my_tiles) issue(s, s, PAGED ? page_of(s) : 0);
        cp_async_commit();
    }
    int page_next = (PAGED && STAGES - 1 < my_tiles) ? page_of(STAGES - 1) : 0;

    // A-operand fragments of q*scale*log2(e): rows 0..7 = F16 rounding, rows 8..15 = residual.
    const int head = kv * p.group + quad;          // query head of this lane's MMA row
    const bool head_ok = quad < p.group;
    uint32_t qf[KS][4];
    {
        const float* qp = p.q + ((int64_t)b * p.hq + (head_ok ? head : kv * p.group)) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int c0 = ks * 16 + hf * 8 + qlane * 2;
                float2 x = head_ok ? *reinterpret_cast<const float2*>(qp + c0) : make_float2(0.f, 0.f);
                x.x *= p.scale_log2;
                x.y *= p.scale_log2;
                const uint32_t hi = pack_half2(x.x, x.y);
                const float2 hif = unpack_half2(hi);
                qf[ks][hf * 2 + 0] = hi;
                qf[ks][hf * 2 + 1] = pack_half2(x.x - hif.x, x.y - hif.y);
            }
        }
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    float* logit_row = nullptr;
    if (p.logits != nullptr && head_ok) logit_row = p.logits + ((int64_t)b * p.hq + head) * p.logit_stride;

    // ldmatrix lane geometry
    const int lm_mat = lane >> 3, lm_row = lane & 7;
    // K (non-transposed): matrices (tok 0-7,k lo) (tok 0-7,k hi) (tok 8-15,k lo) (tok 8-15,k hi)
    const int k_tok = (lm_mat >> 1) * 8 + lm_row, k_half = lm_mat & 1;
    // V (transposed): matrices (tok 0-7,chunk j) (tok 8-15,chunk j) (tok 0-7,chunk j+1) (tok 8-15,chunk j+1)
    const int v_tok = (lm_mat & 1) * 8 + lm_row, v_half = lm_mat >> 1;

    for (int j = 0; j < my_tiles; ++j) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
#ifdef ARGUS_XC_PROFILE
        if (j == 0) PH_STAMP(1)
#endif
        {
            const int jn = j + STAGES - 1;
            if (jn < my_tiles) issue(jn, jn % STAGES, page_next);
            cp_async_commit();
            if (PAGED && jn + 1 < my_tiles) page_next = page_of(jn + 1);
        }
        const uint32_t sb = wsm + (j % STAGES) * STAGE_B;
        const int tokb = t0 + (warp + j * WARPS) * WT;

        // S = q · K^T for 16 tokens
        float c[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t kb[4];
            ldmatrix_x4(kb, sb + k_tok * ROW_B + ((((ks << 1) | k_half) ^ (k_tok & 7)) << 4));
            mma_f16_16816(c[0], qf[ks], kb[0], kb[1]);
            mma_f16_16816(c[1], qf[ks], kb[2], kb[3]);
        }
        float s[2][2];
        float tile_max = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int tok = tokb + n * 8 + qlane * 2 + i;
                float x = c[n][i] + c[n][i + 2];
                if (tok >= t1 || x != x) x = -INFINITY;   // a NaN logit is skipped, as the CPU backends' guard does
                if (tok < t1 && logit_row != nullptr) logit_row[tok] = x;
                s[n][i] = x;
                tile_max = fmaxf(tile_max, x);
            }
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
        const float m_new = fmaxf(m_run, tile_max);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = fast_exp2(m_run - m_use);   // m_run = -inf -> 0
        m_run = m_new;

        uint32_t pa[4];
        float psum = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const float p0 = fast_exp2(s[n][0] - m_use), p1 = fast_exp2(s[n][1] - m_use);
            psum += p0 + p1;
            const uint32_t hi = pack_half2(p0, p1);
            const float2 hif = unpack_half2(hi);
            pa[n * 2 + 0] = hi;
            pa[n * 2 + 1] = pack_half2(p0 - hif.x, p1 - hif.y);
        }
        l_run = l_run * alpha + psum;
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][0] *= alpha; o[n][1] *= alpha; o[n][2] *= alpha; o[n][3] *= alpha;
            }
        }
        // O += P · V
#pragma unroll
        for (int jn = 0; jn < NT / 2; ++jn) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, sb + TILE_B + v_tok * ROW_B + ((((jn << 1) | v_half) ^ (v_tok & 7)) << 4));
            mma_f16_16816(o[2 * jn], pa, vb[0], vb[1]);
            mma_f16_16816(o[2 * jn + 1], pa, vb[2], vb[3]);
        }
    }
    cp_async_wait<0>();
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();   // every warp is done with its ring: the space becomes the merge buffer

    // ── merge the warps of this CTA ──
    float* sm_o = reinterpret_cast<float*>(smem + EpilogueSmem<D, WARPS>::O_OFF);        // [WARPS][8][D]
    float2* sm_ml = reinterpret_cast<float2*>(smem + EpilogueSmem<D, WARPS>::ML_OFF);    // [WARPS][8]
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        float2 v2 = make_float2(o[n][0] + o[n][2], o[n][1] + o[n][3]);
        *reinterpret_cast<float2*>(sm_o + (warp * 8 + quad) * D + n * 8 + qlane * 2) = v2;
    }
    if (qlane == 0) sm_ml[warp * 8 + quad] = make_float2(m_run, l_run);
    __syncthreads();
    PH_STAMP(2)

    decode_epilogue<D, WARPS>(smem, p, b, kv, (int64_t)gs * p.hkv + kv, (int64_t)bt.item_start[b] * p.hkv + kv, n_splits);
    PH_STAMP(3)
}

// p_t = exp2(logit_t - lse2) per query head, plus the GQA reductions of the score policy
// (crates/techniques/attn-score/src/lib.rs:262-287): flat = sum over heads (h ascending),
// head[kv] = (sum over the group, r ascending) * (1/g). N consecutive tokens of the KV heads [kv0, kv1) per call; all
// loads of a head group are requested before the first is used (the kernel is a stream over the logits, and one load
// in flight per thread leaves it bound by latency).
template <int N>
__device__ __forceinline__ void load_floats(const float* src, float (&x)[N]) {
    if constexpr (N >= 4) {
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            x[i] = v.x; x[i + 1] = v.y; x[i + 2] = v.z; x[i + 3] = v.w;
        }
    } else {
        x[0] = *src;
    }
}
template <int N>
__device__ __forceinline__ void store_floats(float* dst, const float (&x)[N]) {
    if constexpr (N >= 4) {
#pragma unroll
        for (int i = 0; i < N; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    } else {
        *dst = x[0];
    }
}

template <int N>
__device__ __forceinline__ void finalize_tokens(const FinalizeParams& f, int b, int t, int kv0, int kv1, bool want_flat) {
    const float inv_g = 1.0f / (float)f.group;
    float flat[N];
#pragma unroll
    for (int i = 0; i < N; ++i) flat[i] = 0.f;
    for (int kv = kv0; kv < kv1; ++kv) {
        const int64_t h0 = (int64_t)b * f.hq + kv * f.group;
        float gsum[N];
#pragma unroll
        for (int i = 0; i < N; ++i) gsum[i] = 0.f;
        for (int r0 = 0; r0 < f.group; r0 += 4) {   // four heads' loads in flight at a time (registers), r ascending
            float x[4][N], lse4[4];
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {
                const int r = r0 + rr;
                if (r < f.group) {
                    lse4[rr] = f.lse2[h0 + r];
                    load_floats<N>(f.logits + (h0 + r) * f.logit_stride + t, x[rr]);
                }
            }
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {
                const int r = r0 + rr;
                if (r < f.group) {
                    const float lse = lse4[rr];
                    float pr[N];
#pragma unroll
                    for (int i = 0; i < N; ++i) {
                        pr[i] = exp2f(x[rr][i] - lse);
                        gsum[i] += pr[i];
                        if (want_flat) flat[i] += pr[i];
                    }
                    if (f.scores != nullptr) store_floats<N>(f.scores + (h0 + r) * f.score_stride + t, pr);
                }
            }
        }
        if (f.head_scores != nullptr) {
#pragma unroll
            for (int i = 0; i < N; ++i) gsum[i] *= inv_g;
            store_floats<N>(f.head_scores + ((int64_t)b * f.hkv + kv) * f.score_stride + t, gsum);
        }
    }
    if (want_flat) store_floats<N>(f.flat_scores + (int64_t)b * f.score_stride + t, flat);
}

// One thread per (sequence, TPT consecutive tokens) and - when no flat sum over all heads is wanted - per KV head
// (gridDim.z = Hkv). 16-byte accesses where the rows allow them.
template <int TPT>
__global__ void __launch_bounds__(256, 4) finalize_scores_kernel(const __grid_constant__ FinalizeParams f) {
    const int b = blockIdx.y;
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) * TPT;
    const int T = f.seq_len[b];
    if (t >= T) return;
    const bool want_flat = f.flat_scores != nullptr;
    const int kv0 = gridDim.z > 1 ? blockIdx.z : 0, kv1 = gridDim.z > 1 ? kv0 + 1 : f.hkv;
    const bool vec = ((f.logit_stride | f.score_stride) & (TPT - 1)) == 0 && t + TPT <= T &&
                     ((reinterpret_cast<uintptr_t>(f.logits) | reinterpret_cast<uintptr_t>(f.scores) |
                       reinterpret_cast<uintptr_t>(f.head_scores) | reinterpret_cast<uintptr_t>(f.flat_scores)) & 15) == 0;
    if (vec) {
        finalize_tokens<TPT>(f, b, t, kv0, kv1, want_flat);
    } else {
        for (int i = 0; i < TPT && t + i < T; ++i) finalize_tokens<1>(f, b, t + i, kv0, kv1, want_flat);
    }
}

// ── host-side launchers ──
template <int D, int WARPS, int STAGES, bool PAGED = false>
static cudaError_t launch_decode_f16_t(const DecodeParams& p, const DecodeBatch& bt, int n_items, cudaStream_t st) {
    using Cfg = DecodeF16Cfg<D, WARPS, STAGES>;
    static bool attr_done[kMaxDevices] = {};
    auto kern = decode_f16_kernel<D, WARPS, STAGES, PAGED>;
    cudaError_t ea = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::SMEM_B, attr_done);
    if (ea != cudaSuccess) return ea;
    kern<<<n_items * p.hkv, WARPS * 32, Cfg::SMEM_B, st>>>(p, bt);
    return cudaGetLastError();
}

int decode_f16_smem_bytes(int head_dim) { return head_dim == 64 ? DecodeF16Cfg<64, 4, 4>::SMEM_B : DecodeF16Cfg<128, 4, 3>::SMEM_B; }
int decode_f16_cta_tokens(int head_dim) { return head_dim == 64 ? DecodeF16Cfg<64, 4, 4>::CTA_TOK : DecodeF16Cfg<128, 4, 3>::CTA_TOK; }

cudaError_t launch_decode_f16(const DecodeParams& p, const DecodeBatch& bt, int head_dim, int n_items, cudaStream_t st) {
    if (bt.page_tokens > 0) {
        if (head_dim == 128) return launch_decode_f16_t<128, 4, 3, true>(p, bt, n_items, st);
        if (head_dim == 64) return launch_decode_f16_t<64, 4, 4, true>(p, bt, n_items, st);
        return cudaErrorInvalidValue;
    }
    if (head_dim == 128) return launch_decode_f16_t<128, 4, 3>(p, bt, n_items, st);
    if (head_dim == 64) return launch_decode_f16_t<64, 4, 4>(p, bt, n_items, st);
    return cudaErrorInvalidValue;
}

cudaError_t launch_finalize_scores(const FinalizeParams& f, int max_len, cudaStream_t st) {
    if (max_len <= 0) return cudaSuccess;
    // four tokens per thread (eight measured slower: 117 us against 115 us for the KIVI step with the H2O vector)
    dim3 grid(((max_len + 3) / 4 + 255) / 256, f.n_seqs, f.flat_scores == nullptr ? f.hkv : 1);
    finalize_scores_kernel<4><<<grid, 256, 0, st>>>(f);
    return cudaGetLastError();
}

#ifdef ARGUS_XC_PROFILE
extern "C" __attribute__((visibility("default"))) int argus_b200_debug_xc_profile(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_xc_prof, sizeof(g_xc_prof));
}
// reads the phase stamps {min, max} x {entry, first tile, loop end, epilogue end} and re-arms them for the next launch
extern "C" __attribute__((visibility("default"))) int argus_b200_debug_phase_profile(unsigned long long* host_out) {
    cudaError_t e = cudaMemcpyFromSymbol(host_out, g_phase_prof, sizeof(g_phase_prof));
    unsigned long long init[8];
    for (int i = 0; i < 8; ++i) init[i] = (i & 1) ? 0ull : ~0ull;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_phase_prof, init, sizeof(init));
    return (int)e;
}
#endif

}  // namespace argus
