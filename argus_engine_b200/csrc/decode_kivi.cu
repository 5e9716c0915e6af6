// Split-KV GQA decode attention over a KIVI-packed KV cache (Q2/Q4/Q8 blocks + full-precision residual
// window), sm_100a, reading the packed bytes once and never materialising a dequantised value.
//
// Stands behind CudaQuantAttnBackend::attention_gen_quant (crates/argus-extension-api/src/lib.rs:3087-3104;
// the kernels it replaces are kernel_attn_gen_kivi_q{2,4,8}, crates/techniques/kivi/src/kivi_attn.cu:34,220,403).
// Cache layout is the engine's, unchanged (engine/src/kv/quant_window_cache.rs:919-946):
//   K blocks [flush][kv_head][group of 32 tokens][channel]  — one block = 32 TOKENS of one channel
//   V blocks [flush][kv_head][token][channel block of 32]   — one block = 32 CHANNELS of one token
//   block = {f16 d, f16 m, codes}, value = code*d + m        (crates/argus-kv-codec/src/lib.rs:115-202)
//   residual ring F32 (or F16) [kv_head][res_cap][D], token q_tokens + r is row r.
//
// Both the K and the V bytes of one (kv_head, 32-token group) are contiguous (D*block_bytes each), so a
// warp tile is fetched with two bulk async copies (cp.async.bulk + mbarrier) and stays in the packed form
// in shared memory. Lanes pull 4-token (resp. 4-channel) code pieces of the two channels (tokens) that one
// MMA operand register pairs and feed them to mma.sync as they are; the scales d and minima m are folded onto
// the other operand (see "Scale folding" below). Tokens of a group are visited in a permuted order that makes
// those pieces contiguous; softmax does not care and P·V uses the same order. The residual window is a
// separate split handled in plain F32 FMA. Everything after the main loop (warp merge, split merge, score
// finalize) is shared with the F16 kernel.

#include "decode_epilogue.cuh"
#include "context.h"
#include "decode_params.h"
#include "ptx.cuh"

namespace argus {

template <int BITS>
struct KvBlock {
    static constexpr int BYTES = BITS == 2 ? 12 : BITS == 4 ? 20 : 36;
    static constexpr int PIECE = BITS / 2;   // bytes holding 4 consecutive codes
};

// Scale folding. A K block is 32 tokens of ONE channel, a V block 32 channels of ONE token, each with a scale d and a
// minimum m: value = d*c + m. Both scales run along the contraction index of their product, so they move to the other
// operand and the codes go into the tensor cores as they are:
//   s[h][t] = sum_ch (q[h][ch] * d[ch]) * c[t][ch]  +  sum_ch q[h][ch] * m[ch]        (one extra MMA per k-step)
//   o[ch][h] = sum_t c[t][ch] * (p[h][t] * d[t][blk(ch)])  +  sum_t p[h][t] * m[t][blk(ch)]   (one extra MMA per k-step)
// which costs a few multiplications per 32-token group instead of a subtract and a fused multiply-add per code pair.
//
// The codes are used where they sit: a code c in bits [s, s+w) of a 16-bit lane, everything else masked off, is the
// subnormal F16 number c * 2^(s-24), exact, and tensor-core products of F16 inputs are exact in the FP32 accumulator.
// The four codes of a piece therefore carry different powers of two (kCodeUnscale), taken out of the accumulators
// after the MMAs. x = piece(lo element) | piece(hi element) << 16 for 2- and 4-bit codes; for 8-bit codes the two
// pieces (four bytes each) come separately.
template <int BITS>
__device__ __forceinline__ void raw_codes(uint32_t xa, uint32_t xb, uint32_t (&out)[4]) {
    if constexpr (BITS == 4) {
        const uint32_t xs = xa >> 8;
        out[0] = xa & 0x000F000Fu;
        out[1] = xa & 0x00F000F0u;
        out[2] = xs & 0x000F000Fu;
        out[3] = xs & 0x00F000F0u;
    } else if constexpr (BITS == 2) {
        out[0] = xa & 0x00030003u;
        out[1] = xa & 0x000C000Cu;
        out[2] = xa & 0x00300030u;
        out[3] = xa & 0x00C000C0u;
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t t, v;   // byte j of xa and of xb -> low bytes of the two halves, zero above each
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(t) : "r"(xa), "r"(xb), "r"((uint32_t)j | ((uint32_t)(4 + j) << 4)));
            asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(v) : "r"(t), "r"(0u));
            out[j] = v;
        }
    }
}
// 2^24 over the power of two that position j of raw_codes carries
template <int BITS>
__device__ __forceinline__ constexpr float code_unscale(int j) {
    return BITS == 4 ? ((j & 1) ? 1048576.f : 16777216.f)
         : BITS == 2 ? (j == 0 ? 16777216.f : j == 1 ? 4194304.f : j == 2 ? 1048576.f : 262144.f)
                     : 16777216.f;
}

__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
// (hi, lo) halves of the product (a_hi + a_lo) * d: hi = rn(a_hi*d), lo = rn(a_lo*d + (a_hi*d - hi)), the inner term exact
__device__ __forceinline__ void scale_split(uint32_t a_hi, uint32_t a_lo, uint32_t d, uint32_t& hi, uint32_t& lo) {
    const __half2 ah = *reinterpret_cast<const __half2*>(&a_hi), al = *reinterpret_cast<const __half2*>(&a_lo);
    const __half2 dd = *reinterpret_cast<const __half2*>(&d);
    const __half2 h = __hmul2(ah, dd);
    const __half2 l = __hfma2(al, dd, __hfma2(ah, dd, __hneg2(h)));
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// Per-pair header entry of the shared-memory tables: {d,d'} and {m,m'} of the two elements that share an operand register.
__device__ __forceinline__ uint2 make_header(uint32_t h0, uint32_t h1) {
    return make_uint2(__byte_perm(h0, h1, 0x5410), __byte_perm(h0, h1, 0x7632));
}

template <int BITS>
__device__ __forceinline__ uint32_t load_piece(const uint8_t* p) {
    if constexpr (BITS == 2) return *p;
    else if constexpr (BITS == 4) return *reinterpret_cast<const uint16_t*>(p);
    else return *reinterpret_cast<const uint32_t*>(p);
}

// mbarrier / bulk-copy helpers. Every wait is bounded.
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < (1 << 22); ++it) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        __nanosleep(32);   // a spinning warp takes issue slots from the warps that have work
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int D, int BITS, int WARPS, int STAGES>
struct DecodeKiviCfg {
    static constexpr int BB = KvBlock<BITS>::BYTES;
    static constexpr int TILE_B = D * BB;             // K bytes (== V bytes) of one (kv head, 32-token group)
    static constexpr int STAGE_B = 2 * TILE_B;
    static constexpr int RING_B = WARPS * STAGES * STAGE_B;
    static constexpr int KH_N = D / 2;                // {d2, m2} per channel pair
    static constexpr int VH_N = 16 * (D / 32);        // {d2, m2} per (token pair, channel block)
    static constexpr int HDR_B = WARPS * (KH_N + VH_N) * 8;
    static constexpr int BAR_OFF = RING_B + HDR_B;
    static constexpr int PIPE_B = BAR_OFF + WARPS * STAGES * 8;
    static constexpr int EPI_B = EpilogueSmem<D, WARPS>::BYTES;
    static constexpr int SMEM_B = PIPE_B > EPI_B ? PIPE_B : EPI_B;
};

template <int D, int BITS, int WARPS, int STAGES, int MINB>
__global__ void __launch_bounds__(WARPS * 32, MINB)
decode_kivi_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ KiviBatch bt) {
    using Cfg = DecodeKiviCfg<D, BITS, WARPS, STAGES>;
    constexpr int BB = Cfg::BB, TILE_B = Cfg::TILE_B, STAGE_B = Cfg::STAGE_B, PIECE = KvBlock<BITS>::PIECE;
    constexpr int KS = D / 16, NT = D / 8, NB = D / 32;
    extern __shared__ __align__(128) uint8_t smem[];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane >> 2, qlane = lane & 3;

    const int kv = blockIdx.x % p.hkv;
    const int gs = blockIdx.x / p.hkv;   // launch slot: residual splits of all sequences, then the packed splits
    const int n_res = bt.res_start[p.n_seqs];
    int b = 0, split;
    if (gs < n_res) {
        while (b + 1 < p.n_seqs && bt.res_start[b + 1] <= gs) ++b;
        split = bt.n_qsplits[b] + (gs - bt.res_start[b]);
    } else {
        const int gq = gs - n_res;   // packed splits before sequence b: item_start[b] - res_start[b]
        while (b + 1 < p.n_seqs && bt.item_start[b + 1] - bt.res_start[b + 1] <= gq) ++b;
        split = gq - (bt.item_start[b] - bt.res_start[b]);
    }
    const int n_splits = bt.item_start[b + 1] - bt.item_start[b];
    const int n_qsplits = bt.n_qsplits[b];
    const int q_tokens = bt.q_tokens[b];

    float* sm_o = reinterpret_cast<float*>(smem + EpilogueSmem<D, WARPS>::O_OFF);
    float2* sm_ml = reinterpret_cast<float2*>(smem + EpilogueSmem<D, WARPS>::ML_OFF);
    const int64_t item = (int64_t)(bt.item_start[b] + split) * p.hkv + kv;
    const int64_t item0 = (int64_t)bt.item_start[b] * p.hkv + kv;

    if (split >= n_qsplits) {
        // ───────── residual window: plain F32, one token per warp step, lanes split the channels ─────────
        constexpr int EPL = D / 32;   // channels per lane
        const int r0 = (split - n_qsplits) * bt.res_chunk, r1 = min(r0 + bt.res_chunk, bt.res_tokens[b]);
        float qreg[kMaxGroup][EPL], oacc[kMaxGroup][EPL], m_h[kMaxGroup], l_h[kMaxGroup];
#pragma unroll
        for (int h = 0; h < kMaxGroup; ++h) {
            m_h[h] = -INFINITY;
            l_h[h] = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                oacc[h][e] = 0.f;
                qreg[h][e] = (h < p.group) ? p.q[((int64_t)b * p.hq + kv * p.group + h) * D + lane * EPL + e] * p.scale_log2 : 0.f;
            }
        }
        // two tokens per step, both rows requested before either is used: the loop is bound by the latency of its loads
        auto load_row = [&](int r, float (&kr)[EPL], float (&vr)[EPL]) {
            const int64_t off = ((int64_t)kv * bt.res_cap + r) * D + lane * EPL;
            if (bt.res_is_f16) {
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    kr[e] = __half2float(static_cast<const __half*>(bt.res_k[b])[off + e]);
                    vr[e] = __half2float(static_cast<const __half*>(bt.res_v[b])[off + e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    kr[e] = static_cast<const float*>(bt.res_k[b])[off + e];
                    vr[e] = static_cast<const float*>(bt.res_v[b])[off + e];
                }
            }
        };
        auto token = [&](int r, const float (&kr)[EPL], const float (&vr)[EPL]) {
#pragma unroll
            for (int h = 0; h < kMaxGroup; ++h) {
                if (h >= p.group) break;
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) s += qreg[h][e] * kr[e];
#pragma unroll
                for (int sh = 16; sh > 0; sh >>= 1) s += __shfl_xor_sync(0xffffffffu, s, sh);
                if (p.logits != nullptr && lane == 0)
                    p.logits[((int64_t)b * p.hq + kv * p.group + h) * p.logit_stride + q_tokens + r] = s;
                const float m_new = fmaxf(m_h[h], s);
                const float alpha = fast_exp2(m_h[h] - m_new);
                const float pr = fast_exp2(s - m_new);
                m_h[h] = m_new;
                l_h[h] = l_h[h] * alpha + pr;
#pragma unroll
                for (int e = 0; e < EPL; ++e) oacc[h][e] = oacc[h][e] * alpha + pr * vr[e];
            }
        };
        for (int r = r0 + warp; r < r1; r += 2 * WARPS) {
            float ka[EPL], va[EPL], kb[EPL], vb[EPL];
            const bool two = r + WARPS < r1;
            load_row(r, ka, va);
            load_row(two ? r + WARPS : r, kb, vb);
            token(r, ka, va);
            if (two) token(r + WARPS, kb, vb);
        }
#pragma unroll
        for (int h = 0; h < kMaxGroup; ++h) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) sm_o[(warp * 8 + h) * D + lane * EPL + e] = oacc[h][e];
            if (lane == 0) sm_ml[warp * 8 + h] = make_float2(m_h[h], l_h[h]);
        }
        __syncthreads();
        decode_epilogue<D, WARPS>(smem, p, b, kv, item, item0, n_splits);
        return;
    }

    // ───────── packed part: 32-token groups, two bulk copies per warp tile ─────────
    const int gpf = bt.res_cap / 32;                       // groups per flush
    const int g0 = split * bt.chunk_groups[b];
    const int g1 = min(g0 + bt.chunk_groups[b], q_tokens / 32);
    const int n_tiles = g1 > g0 ? g1 - g0 : 0;
    const int my_tiles = warp < n_tiles ? (n_tiles - warp + WARPS - 1) / WARPS : 0;
    const uint8_t* qk = bt.qk[b];
    const uint8_t* qv = bt.qv[b];
    const int32_t* pages = bt.flush_pages[b];

    uint8_t* ring = smem + warp * STAGES * STAGE_B;
    using Header = uint2;
    Header* kh = reinterpret_cast<Header*>(smem + Cfg::RING_B) + warp * (Cfg::KH_N + Cfg::VH_N);
    Header* vh = kh + Cfg::KH_N;
    const uint32_t bar0 = smem_u32(smem + Cfg::BAR_OFF) + warp * STAGES * 8;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    auto issue = [&](int j, int slot) {   // lane 0 only
        const int gidx = g0 + warp + j * WARPS;
        int f = gidx / gpf;
        const int gif = gidx - f * gpf;
        if (pages != nullptr) f = __ldg(pages + f);   // a page holds one flush of all KV heads
        const int64_t kblk = (((int64_t)f * p.hkv + kv) * gpf + gif) * D;
        const int64_t vblk = (((int64_t)f * p.hkv + kv) * bt.res_cap + gif * 32) * NB;
        const uint32_t dst = smem_u32(ring + slot * STAGE_B);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar0 + slot * 8, STAGE_B);
        bulk_g2s(dst, qk + kblk * BB, TILE_B, bar0 + slot * 8);
        bulk_g2s(dst + TILE_B, qv + vblk * BB, TILE_B, bar0 + slot * 8);
    };

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s)
            if (s < my_tiles) issue(s, s);
    }

    const int head = kv * p.group + quad;
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

    // O^T accumulators: m-tile (blk, h) row quad / quad+8 is channel 32*blk + 4*quad + 2*h (+1), columns 2*qlane (+1)
    // are query heads. The transposed product needs half the MMAs and half the registers of O = P·V with 16 head rows.
    constexpr int MT = 2 * NB;
    float o[MT][4];
#pragma unroll
    for (int n = 0; n < MT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float ob[4] = {0.f, 0.f, 0.f, 0.f};   // P·m: row blk (lanes with quad == blk < NB), columns = heads 2*qlane (+1)
    float m_run = -INFINITY, l_run = 0.f;
    float* logit_row = nullptr;
    if (p.logits != nullptr && head_ok) logit_row = p.logits + ((int64_t)b * p.hq + head) * p.logit_stride;
    const bool logit_vec = (reinterpret_cast<uintptr_t>(p.logits) & 15) == 0 && (p.logit_stride & 3) == 0;
    bool timed_out = false;

    for (int j = 0; j < my_tiles; ++j) {
        const int slot = j % STAGES;
        if (!mbar_wait(bar0 + slot * 8, (j / STAGES) & 1)) {
            timed_out = true;
            break;
        }
        __syncwarp();   // everyone is past tile j-1: its slot may be refilled, and the header tables rewritten
        if (lane == 0) {
            const int jn = j + STAGES - 1;
            if (jn < my_tiles) issue(jn, jn % STAGES);
        }
        const uint8_t* kt = ring + slot * STAGE_B;
        const uint8_t* vt = kt + TILE_B;

        // {d,d} / {m,m'} tables of the element pairs that share an MMA operand register
        for (int i = lane; i < Cfg::KH_N; i += 32) {
            const uint32_t h0 = *reinterpret_cast<const uint32_t*>(kt + (2 * i) * BB);
            const uint32_t h1 = *reinterpret_cast<const uint32_t*>(kt + (2 * i + 1) * BB);
            kh[(i & ~7) + (i & 3) * 2 + ((i >> 2) & 1)] = make_header(h0, h1);   // pairs (p, p+4) of a k-step side by side
        }
        for (int i = lane; i < Cfg::VH_N; i += 32) {
            const int blk = i >> 4, t = i & 15;        // pairs (t, t+16)
            const uint32_t h0 = *reinterpret_cast<const uint32_t*>(vt + (t * NB + blk) * BB);
            const uint32_t h1 = *reinterpret_cast<const uint32_t*>(vt + ((t + 16) * NB + blk) * BB);
            vh[i] = make_header(h0, h1);
        }
        __syncwarp();

        // S[head][token]: MMA column `quad` of n-tile jp is token 4*piece + jp of the group, where lane group
        // `quad` reads code piece (quad>>1) + 4*(quad&1). That permutation makes the tokens one lane later pairs
        // for P·V lie 16 apart, so that the four lanes of a quad do not all hit the same shared-memory banks.
        // A = q * d of this group (rows 0-7 the F16 head, rows 8-15 the remainder), B = the codes; cb collects q·m.
        float c[4][4], cb[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
        cb[0] = cb[1] = cb[2] = cb[3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int cha = ks * 16 + 2 * qlane;
            const uint4 hab = *reinterpret_cast<const uint4*>(&kh[ks * 8 + 2 * qlane]);   // {d, m} of (cha, cha+1 | cha+8, cha+9)
            const uint8_t* pk = kt + cha * BB + 4 + PIECE * ((quad >> 1) + 4 * (quad & 1));
            uint32_t xa0 = load_piece<BITS>(pk), xa1 = load_piece<BITS>(pk + BB);
            uint32_t xb0 = load_piece<BITS>(pk + 8 * BB), xb1 = load_piece<BITS>(pk + 9 * BB);
            if constexpr (BITS != 8) {
                xa0 |= xa1 << 16;
                xb0 |= xb1 << 16;
            }
            uint32_t a[4];
            // value and remainder of q*d: dropping the remainder rows was measured (-2 us of 103) and not taken
            scale_split(qf[ks][0], qf[ks][1], hab.x, a[0], a[1]);
            scale_split(qf[ks][2], qf[ks][3], hab.z, a[2], a[3]);
            mma_f16_16816(cb, qf[ks], hab.y, hab.w);
            uint32_t b0[4], b1[4];
            raw_codes<BITS>(xa0, xa1, b0);
            raw_codes<BITS>(xb0, xb1, b1);
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) mma_f16_16816(c[jp], a, b0[jp], b1[jp]);
        }
        const float s_bias = cb[0] + cb[2];   // every column of cb holds the same sum: q·m of this lane's head
        // accumulator column 2*qlane+i of n-tile jp  <->  token 4*qlane + 16*i + jp of the group
        const int tokb = (g0 + warp + j * WARPS) * 32;
        float s[4][2];
        float tile_max = -INFINITY;
#pragma unroll
        for (int jp = 0; jp < 4; ++jp)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float x = fmaf(c[jp][i] + c[jp][i + 2], code_unscale<BITS>(jp), s_bias);
                s[jp][i] = x;
                tile_max = fmaxf(tile_max, x);
            }
        if (logit_row != nullptr) {   // a lane holds tokens 4q + 16i + {0..3}: one 16-byte store per i where rows allow it
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float* dst = logit_row + tokb + 4 * qlane + 16 * i;
                if (logit_vec) *reinterpret_cast<float4*>(dst) = make_float4(s[0][i], s[1][i], s[2][i], s[3][i]);
                else { dst[0] = s[0][i]; dst[1] = s[1][i]; dst[2] = s[2][i]; dst[3] = s[3][i]; }
            }
        }
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
        const float m_new = fmaxf(m_run, tile_max);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = fast_exp2(m_run - m_use);
        m_run = m_new;
        float psum = 0.f;
#pragma unroll
        for (int jp = 0; jp < 4; ++jp)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[jp][i] = fast_exp2(s[jp][i] - m_use);
                psum += s[jp][i];
            }
        l_run = l_run * alpha + psum;
        if (__any_sync(0xffffffffu, alpha != 1.f)) {   // this lane's columns are heads 2*qlane and 2*qlane+1
            const float a0 = __shfl_sync(0xffffffffu, alpha, 8 * qlane), a1 = __shfl_sync(0xffffffffu, alpha, 8 * qlane + 4);
#pragma unroll
            for (int n = 0; n < MT; ++n) {
                o[n][0] *= a0; o[n][1] *= a1; o[n][2] *= a0; o[n][3] *= a1;
            }
            ob[0] *= a0;
            ob[1] *= a1;
        }
        // O^T[channel][head] += V^T · P^T. k-step u: A columns (2q, 2q+1 | 2q+8, 2q+9) and B rows alike are tokens
        // (4q+2u, 4q+16+2u | 4q+2u+1, 4q+17+2u); B column `quad` is this lane's own head, so P goes from the S
        // accumulators into the B registers without leaving the lane. A = the codes, B = P * d of (token, channel
        // block); ob collects P·m, its row `blk` (lanes with quad == blk) against the same unscaled P.
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const uint32_t pb0 = pack_half2(s[2 * u][0], s[2 * u][1]);
            const uint32_t pb1 = pack_half2(s[2 * u + 1][0], s[2 * u + 1][1]);
            const int ta = 4 * qlane + 2 * u;
            {
                const int bq = quad < NB ? quad : 0;
                const uint4 mm = *reinterpret_cast<const uint4*>(&vh[bq * 16 + qlane * 4 + 2 * u]);
                const uint32_t am[4] = {quad < NB ? mm.y : 0u, 0u, quad < NB ? mm.w : 0u, 0u};
                mma_f16_16816(ob, am, pb0, pb1);
            }
#pragma unroll
            for (int blk = 0; blk < NB; ++blk) {
                const uint4 dd = *reinterpret_cast<const uint4*>(&vh[blk * 16 + qlane * 4 + 2 * u]);
                const uint32_t pd0 = hmul2_u(pb0, dd.x), pd1 = hmul2_u(pb1, dd.z);
                const uint8_t* pv = vt + (ta * NB + blk) * BB + 4 + PIECE * quad;
                uint32_t xa0 = load_piece<BITS>(pv), xa1 = load_piece<BITS>(pv + 16 * NB * BB);
                uint32_t xb0 = load_piece<BITS>(pv + NB * BB), xb1 = load_piece<BITS>(pv + 17 * NB * BB);
                if constexpr (BITS != 8) {
                    xa0 |= xa1 << 16;
                    xb0 |= xb1 << 16;
                }
                uint32_t va[4], vb[4];
                raw_codes<BITS>(xa0, xa1, va);
                raw_codes<BITS>(xb0, xb1, vb);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t a[4] = {va[2 * h], va[2 * h + 1], vb[2 * h], vb[2 * h + 1]};
                    mma_f16_16816(o[blk * 2 + h], a, pd0, pd1);
                }
            }
        }
    }
    if (timed_out) {
        // A copy never landed. Give every outstanding copy one more bounded chance to finish so that none is
        // in flight when shared memory is reused, report through the status word, and contribute nothing.
        for (int s = 0; s < STAGES; ++s) (void)mbar_wait(bar0 + s * 8, 0);
        if (p.status != nullptr) atomicExch(p.status, 1);
#pragma unroll
        for (int n = 0; n < MT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        ob[0] = ob[1] = 0.f;
        m_run = -INFINITY;
        l_run = 0.f;
    }
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();

    // accumulator (m-tile blk*2+h, register 2*r+i) is channel 32*blk + 4*quad + 2*h + r of head 2*qlane + i, still
    // carrying the power of two of code position 2*h + r; the P·m sum of (blk, head) sits in the lane with quad == blk
#pragma unroll
    for (int blk = 0; blk < NB; ++blk)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float bias = __shfl_sync(0xffffffffu, ob[i], blk * 4 + qlane);
            const float4 v4 = make_float4(fmaf(o[blk * 2][i], code_unscale<BITS>(0), bias),
                                          fmaf(o[blk * 2][2 + i], code_unscale<BITS>(1), bias),
                                          fmaf(o[blk * 2 + 1][i], code_unscale<BITS>(2), bias),
                                          fmaf(o[blk * 2 + 1][2 + i], code_unscale<BITS>(3), bias));
            *reinterpret_cast<float4*>(&sm_o[(warp * 8 + 2 * qlane + i) * D + 32 * blk + 4 * quad]) = v4;
        }
    if (qlane == 0) sm_ml[warp * 8 + quad] = make_float2(m_run, l_run);
    __syncthreads();
    decode_epilogue<D, WARPS>(smem, p, b, kv, item, item0, n_splits);
}

template <int D, int BITS, int WARPS, int STAGES, int MINB = 2>
static cudaError_t launch_kivi_t(const DecodeParams& p, const KiviBatch& bt, int n_items, cudaStream_t st) {
    using Cfg = DecodeKiviCfg<D, BITS, WARPS, STAGES>;
    static bool attr_done[kMaxDevices] = {};
    auto kern = decode_kivi_kernel<D, BITS, WARPS, STAGES, MINB>;
    cudaError_t ea = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::SMEM_B, attr_done);
    if (ea != cudaSuccess) return ea;
    kern<<<n_items * p.hkv, WARPS * 32, Cfg::SMEM_B, st>>>(p, bt);
    return cudaGetLastError();
}

// CTAs of the selected instantiation that are resident per SM: the split planner fills exactly one such wave.
int decode_kivi_ctas_per_sm(int head_dim, int bits) { return (head_dim == 128 && bits == 4) ? 3 : 2; }

// CTA slots per SM the split planner fills: one resident wave where three CTAs fit (B=8 x 32K tokens, Q4: 3 -> 102 us,
// 4 -> 111, 5 -> 113, 6 -> 107, 7 -> 106, 9 -> 111), two waves where two fit (Q8: 2 -> 124, 3 -> 149, 4 -> 120, 5 -> 137,
// 6 -> 127; Q2: 2 -> 113, 3 -> 139, 4 -> 110, 5 -> 128, 6 -> 117).
int decode_kivi_plan_slots_per_sm(int head_dim, int bits) { return decode_kivi_ctas_per_sm(head_dim, bits) == 3 ? 3 : 4; }

cudaError_t launch_decode_kivi(const DecodeParams& p, const KiviBatch& bt, int head_dim, int bits, int n_items,
                               cudaStream_t st) {
    if (head_dim == 128) {
        if (bits == 4) return launch_kivi_t<128, 4, 4, 3, 3>(p, bt, n_items, st);   // 3 CTAs per SM
        if (bits == 8) return launch_kivi_t<128, 8, 4, 3>(p, bt, n_items, st);
        if (bits == 2) return launch_kivi_t<128, 2, 4, 4>(p, bt, n_items, st);
    } else if (head_dim == 64) {
        if (bits == 4) return launch_kivi_t<64, 4, 4, 4>(p, bt, n_items, st);
        if (bits == 8) return launch_kivi_t<64, 8, 4, 4>(p, bt, n_items, st);
        if (bits == 2) return launch_kivi_t<64, 2, 4, 4>(p, bt, n_items, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace argus
