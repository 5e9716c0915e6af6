// KIVI Q4 decode as TRANSPOSED attention on the 5th-generation tensor cores (tcgen05 + TMEM), head_dim 128.
//
// Same contract and cache layout as decode_kivi.cu (CudaQuantAttnBackend::attention_gen_quant,
// crates/argus-extension-api/src/lib.rs:3087-3104; reference kernel kernel_attn_gen_kivi_q4,
// crates/techniques/kivi/src/kivi_attn.cu:220-390). The mma.sync kernel spends ~1100 instructions per 32-token
// group shuffling codes into MMA fragment order. Here the packed layouts are used the way they lie in memory:
//
//   S^T[token][head] = K_d[token][channel] · q[head][channel]^T     A = K_d, MN-major (tokens contiguous):
//       one dequantised code word (8 tokens of one channel) is exactly one 16-byte row of a UMMA core matrix
//   O^T[channel][head] += V_d[token][channel]^T · P^T[token][head]   A = V_d, MN-major (channels contiguous):
//       one dequantised word (8 channels of one token) is again one core-matrix row; B = P^T, one 16-byte row
//       of 8 heads per token
//
// so dequantisation is a plain vector loop (LOP3 + HSUB2 + HFMA2 on whole words, 16-byte shared-memory stores)
// and the tensor core reads the tiles through shared-memory descriptors. One CTA = (sequence, KV head, split);
// a tile is 4 groups = 128 tokens. Roles: warp 0 bulk-copies packed K/V groups, warp 1 issues the S^T MMAs and
// warp 2 the P·V MMAs (two issuers on two schedulers: next to 16 busy ALU warps one thread cannot issue fast
// enough), warps 4..7 own one token each for the softmax (TMEM lane = token for S^T, = channel for O^T),
// warps 8..23 dequantise. q and p each travel as an F16 value plus its rounding residual (8 + 8 columns), so both keep
// ~22 bits. The residual window and the split merge are the code paths of decode_kivi.cu / decode_epilogue.cuh.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "decode_epilogue.cuh"
#include "context.h"
#include "decode_params.h"
#include "ptx.cuh"

namespace argus {
namespace ktc {

constexpr int D = 128, BB = 20, TILE_TOK = 128, GROUPS = 4;
constexpr int GRP_B = D * BB;                    // 2560: packed K (== V) bytes of one group
constexpr int PK_STAGE_B = 2 * GROUPS * GRP_B;   // 20480: packed K + V of one tile
constexpr int PK_STAGES = 2;                    // a stage is released as soon as its codes are in registers
constexpr int P_BUFS = 3;                       // p(T) is held until P·V(T) has completed
constexpr int VD_BUFS = 3;                      // V_d(T) is held until P·V(T), two handoffs after K_d(T) is used
constexpr int KD_B = TILE_TOK * D * 2;           // 32 KB dequantised K (or V) tile
constexpr int Q_B = 16 * 2 * 128;                // q tile: 16 k-blocks x 2 n-blocks (value, residual) x 128 B
constexpr int P_B = 16 * 2 * 128;                // p tile: 16 k-blocks (tokens) x 2 n-blocks x 128 B
constexpr int OFF_PK = 0;
constexpr int OFF_KD = OFF_PK + PK_STAGES * PK_STAGE_B;
constexpr int OFF_VD = OFF_KD + 2 * KD_B;
constexpr int OFF_Q = OFF_VD + VD_BUFS * KD_B;
constexpr int OFF_P = OFF_Q + Q_B;
constexpr int OFF_RED = OFF_P + P_BUFS * P_B;         // float [3][4 warps][8 heads] softmax exchange
constexpr int OFF_BAR = OFF_RED + 3 * 32 * 4;   // two tile-max buffers + one for the final sums
constexpr int N_BAR = 2 * PK_STAGES + 4 + 2 * VD_BUFS + 2 + P_BUFS + 2;
constexpr int SMEM_B = OFF_BAR + N_BAR * 8 + 64 + 128;
constexpr int DEQ_WARPS = 16;
constexpr int FIRST_DEQ_WARP = 8;
constexpr int THREADS = (FIRST_DEQ_WARP + DEQ_WARPS) * 32;   // 768
constexpr int N_DEQ = DEQ_WARPS * 32;         // one K block and one V block per thread and tile
constexpr int N_WARPS = THREADS / 32;
constexpr uint32_t TMEM_COLS = 64;               // S^T: 2 x 16 columns at 0, O^T: 16 columns at 32
constexpr uint32_t O_COL = 32;
// mbarrier indices
constexpr int B_PK_FULL = 0, B_PK_EMPTY = PK_STAGES, B_KD_FULL = 2 * PK_STAGES, B_KD_EMPTY = B_KD_FULL + 2,
              B_VD_FULL = B_KD_FULL + 4, B_VD_EMPTY = B_VD_FULL + VD_BUFS, B_S_FULL = B_VD_EMPTY + VD_BUFS,
              B_P_FULL = B_S_FULL + 2, B_DONE = B_P_FULL + P_BUFS;   // B_DONE + {0, 1}: all MMAs of an issuer have completed
constexpr float LAZY = 8.0f;


__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < (1 << 23); ++it) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
        __nanosleep(32);   // a spinning warp takes issue slots from the warps it is waiting for
    }
    return false;
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Descriptors travel as two 32-bit halves: only the 14-bit start-address field of the low word changes from one
// MMA to the next, so stepping through a tile is one 32-bit add per operand.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                       uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{ .reg .b64 a, b; .reg .pred p; mov.b64 a, {%1, %2}; mov.b64 b, {%3, %4}; setp.ne.b32 p, %6, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, p; }" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tc_mma64(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
                 "l"(a), "l"(b), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) { return (uint64_t)lo | ((uint64_t)hi << 32); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor without swizzle (sm_100: version 1 at bit 46, layout type 0). A core matrix is
// 8 rows of 16 bytes, stored contiguously (128 B). For an MN-major operand the 16 bytes run along M/N and the
// rows along K; for a K-major operand the other way round. In both cases LBO is the byte distance between core
// matrices that are neighbours along K and SBO between neighbours along M/N. Offsets are in 16-byte units.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo_bytes) { return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14); }
// kind::f16 instruction descriptor: F32 accumulate, F16 operands, operand majors (1 = MN-major), N, M.
__host__ __device__ constexpr uint32_t idesc_f16(int a_mn, int b_mn, int M, int N) {
    return (1u << 4) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}

// One packed block (32 4-bit codes + f16 {d, m}) -> four 16-byte vectors of 8 F16 values. The two codes that share
// a 32-bit lane of a vector are 4 positions apart: vector w holds elements 8w + {0,4,1,5,2,6,3,7}.
__device__ __forceinline__ void dequant_block_q4(const uint8_t* blk, uint4 (&out)[4]) {
    const uint32_t hdr = *reinterpret_cast<const uint32_t*>(blk);
    const uint32_t d2u = __byte_perm(hdr, hdr, 0x1010), m2u = __byte_perm(hdr, hdr, 0x3232);
    const __half2 d2 = *reinterpret_cast<const __half2*>(&d2u), m2 = *reinterpret_cast<const __half2*>(&m2u);
    const __half2 d16 = __hmul2(d2, __float2half2_rn(0.0625f));
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t x = *reinterpret_cast<const uint32_t*>(blk + 4 + 4 * w);
        const uint32_t y = x >> 8;
        uint32_t v0 = (x & 0x000F000Fu) | 0x64006400u;   // 1024 + {n0, n4}
        uint32_t v1 = (x & 0x00F000F0u) | 0x64006400u;   // 1024 + 16*{n1, n5}
        uint32_t v2 = (y & 0x000F000Fu) | 0x64006400u;   // 1024 + {n2, n6}
        uint32_t v3 = (y & 0x00F000F0u) | 0x64006400u;   // 1024 + 16*{n3, n7}
        __half2 h0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&v0), k1024), d2, m2);
        __half2 h1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&v1), k1024), d16, m2);
        __half2 h2 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&v2), k1024), d2, m2);
        __half2 h3 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&v3), k1024), d16, m2);
        out[w] = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                            *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
    }
}

// position inside a 16-byte row -> element (0,4,1,5,2,6,3,7) and its inverse (0,2,4,6,1,3,5,7), as arithmetic
__device__ __forceinline__ int perm8(int r) { return (r >> 1) + 4 * (r & 1); }
__device__ __forceinline__ int invperm8(int e) { return ((e & 3) << 1) | (e >> 2); }

// Bounded wait that gives up at once when another thread of the CTA has already given up.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (*abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    *abort_flag = 1;
    return false;
}

// The same for a whole warp, with one answer for all lanes (the lanes meet again at __syncwarp later on).
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag));
}

// float <-> unsigned key whose unsigned order is the float order (for redux.sync.max)
__device__ __forceinline__ uint32_t f2key(float x) {
    const uint32_t u = __float_as_uint(x);
    return u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
    return __uint_as_float(k ^ ((k >> 31) ? 0x80000000u : 0xFFFFFFFFu));
}

// One arrival per warp: 512 arrivals on one mbarrier word serialise (they are shared-memory atomics on one address),
// so the lanes meet at __syncwarp (which orders their earlier shared-memory accesses) and lane 0 arrives for them.
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

// barrier ids: 0 = __syncthreads; 1 = the 128 softmax threads
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// the same barrier, returning the OR of `flag` over the 128 threads (one answer for all of them)
__device__ __forceinline__ bool softmax_bar_or(bool flag) {
    uint32_t out;
    asm volatile("{ .reg .pred p, q; setp.ne.b32 q, %1, 0; bar.red.or.pred p, 1, 128, q; selp.u32 %0, 1, 0, p; }"
                 : "=r"(out)
                 : "r"((uint32_t)flag)
                 : "memory");
    return out != 0;
}


// Residual-window split (all warps): plain F32 FMA. Warp w owns heads 4*(w&1).. and the tokens r0 + (w>>1) + (N_WARPS/2)*i,
// two at a time; lanes split the channels. The per-warp results are merged into warp slot 0 of the shared
// epilogue layout. Rows must be 16-byte (F32) / 8-byte (F16) aligned, which the host checks.
constexpr int RES_SLOT_OFF = 36 * 1024;   // above the epilogue's own shared memory
__device__ __forceinline__ void load_row4(const void* base, int64_t off, bool f16, float (&x)[4]) {
    if (f16) {
        const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __half*>(base) + off);
        const float2 a = unpack_half2(u.x), b = unpack_half2(u.y);
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    } else {
        const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + off);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
}
__device__ __forceinline__ void residual_split(uint8_t* smem, const DecodeParams& p, const KiviBatch& bt, int b, int kv,
                                               int split, int q_tokens) {
    constexpr int TS = N_WARPS / 2;   // token slots
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hset = warp & 1, tslot = warp >> 1;
    float* slot_o = reinterpret_cast<float*>(smem + RES_SLOT_OFF);                           // [N_WARPS][4][D]
    float2* slot_ml = reinterpret_cast<float2*>(smem + RES_SLOT_OFF + N_WARPS * 4 * D * 4);   // [N_WARPS][4]
    const int r0 = (split - bt.n_qsplits[b]) * bt.res_chunk, r1 = min(r0 + bt.res_chunk, bt.res_tokens[b]);
    const bool f16 = bt.res_is_f16 != 0;
    float q[4][4], o[4][4], m_h[4], l_h[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        m_h[h] = -INFINITY;
        l_h[h] = 0.f;
        const int hh = 4 * hset + h;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            o[h][e] = 0.f;
            q[h][e] = (hh < p.group) ? p.q[((int64_t)b * p.hq + kv * p.group + hh) * D + lane * 4 + e] * p.scale_log2 : 0.f;
        }
    }
    for (int r = r0 + tslot; r < r1; r += 2 * TS) {
        float kr[2][4], vr[2][4];
        const bool two = r + TS < r1;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int64_t off = ((int64_t)kv * bt.res_cap + (u == 0 || two ? r + u * TS : r)) * D + lane * 4;
            load_row4(bt.res_k[b], off, f16, kr[u]);
            load_row4(bt.res_v[b], off, f16, vr[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (u == 1 && !two) break;
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const int hh = 4 * hset + h;
                if (hh >= p.group) break;
                float sc = q[h][0] * kr[u][0] + q[h][1] * kr[u][1] + q[h][2] * kr[u][2] + q[h][3] * kr[u][3];
#pragma unroll
                for (int sh = 16; sh > 0; sh >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, sh);
                if (p.logits != nullptr && lane == 0)
                    p.logits[((int64_t)b * p.hq + kv * p.group + hh) * p.logit_stride + q_tokens + r + u * TS] = sc;
                const float m_new = fmaxf(m_h[h], sc);
                const float alpha = fast_exp2(m_h[h] - m_new);
                const float pr = fast_exp2(sc - m_new);
                m_h[h] = m_new;
                l_h[h] = l_h[h] * alpha + pr;
#pragma unroll
                for (int e = 0; e < 4; ++e) o[h][e] = o[h][e] * alpha + pr * vr[u][e];
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        *reinterpret_cast<float4*>(slot_o + (warp * 4 + h) * D + lane * 4) = make_float4(o[h][0], o[h][1], o[h][2], o[h][3]);
        if (lane == 0) slot_ml[warp * 4 + h] = make_float2(m_h[h], l_h[h]);
    }
    __syncthreads();
    float* sm_o = reinterpret_cast<float*>(smem + EpilogueSmem<D, 4>::O_OFF);
    float2* sm_ml = reinterpret_cast<float2*>(smem + EpilogueSmem<D, 4>::ML_OFF);
    for (int e = threadIdx.x; e < 4 * 8 * D; e += THREADS) {
        const int w = e / (8 * D), h = (e / D) & 7, d = e & (D - 1);
        float acc = 0.f, M = -INFINITY, L = 0.f;
        if (w == 0) {
            const int hs = h >> 2, hh = h & 3;
#pragma unroll
            for (int t = 0; t < TS; ++t) M = fmaxf(M, slot_ml[(2 * t + hs) * 4 + hh].x);
            const float Mu = (M == -INFINITY) ? 0.f : M;
#pragma unroll
            for (int t = 0; t < TS; ++t) {
                const float2 ml = slot_ml[(2 * t + hs) * 4 + hh];
                const float f = fast_exp2(ml.x - Mu);
                L += f * ml.y;
                acc += f * slot_o[((2 * t + hs) * 4 + hh) * D + d];
            }
        }
        sm_o[e] = acc;
        if (d == 0) sm_ml[w * 8 + h] = make_float2(M, L);
    }
}


__global__ void __launch_bounds__(THREADS, 1)
decode_kivi_tc_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ KiviBatch bt) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // The grid lists every packed split first and every residual split after them: the packed CTAs (one per SM,
    // long) start at once and the short residual CTAs fill the SMs that are left over.
    const int kv = blockIdx.x % p.hkv;
    const int gs = blockIdx.x / p.hkv;
    const int n_packed = bt.q_start[p.n_seqs];
    int b = 0, split;
    if (gs < n_packed) {
        while (b + 1 < p.n_seqs && bt.q_start[b + 1] <= gs) ++b;
        split = gs - bt.q_start[b];
    } else {
        const int r = gs - n_packed;
        while (b + 1 < p.n_seqs && bt.item_start[b + 1] - bt.q_start[b + 1] <= r) ++b;
        split = bt.n_qsplits[b] + r - (bt.item_start[b] - bt.q_start[b]);
    }
    const int n_splits = bt.item_start[b + 1] - bt.item_start[b];
    const int q_tokens = bt.q_tokens[b];
    const int64_t item = (int64_t)(bt.item_start[b] + split) * p.hkv + kv;
    const int64_t item0 = (int64_t)bt.item_start[b] * p.hkv + kv;

    if (gs >= n_packed) {   // CTA-uniform
        residual_split(smem, p, bt, b, kv, split, q_tokens);
        __syncthreads();
        if (threadIdx.x >= 128) return;
        decode_epilogue<D, 4>(smem, p, b, kv, item, item0, n_splits);
        return;
    }

    const int gpf = bt.res_cap / 32;   // groups per flush
    const int g0 = split * bt.chunk_groups[b];
    const int g1 = min(g0 + bt.chunk_groups[b], q_tokens / 32);
    const int n_groups = g1 > g0 ? g1 - g0 : 0;
    const int n_tiles = (n_groups + GROUPS - 1) / GROUPS;

    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + OFF_BAR;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + N_BAR * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_BAR + N_BAR * 8 + 4);

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < PK_STAGES; ++s) {
            mbar_init(bar0 + 8 * (B_PK_FULL + s), 1);
            mbar_init(bar0 + 8 * (B_PK_EMPTY + s), DEQ_WARPS);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar0 + 8 * (B_KD_FULL + i), DEQ_WARPS);
            mbar_init(bar0 + 8 * (B_KD_EMPTY + i), 1);
            mbar_init(bar0 + 8 * (B_S_FULL + i), 1);
        }
#pragma unroll
        for (int i = 0; i < P_BUFS; ++i) mbar_init(bar0 + 8 * (B_P_FULL + i), 4);
#pragma unroll
        for (int i = 0; i < VD_BUFS; ++i) {
            mbar_init(bar0 + 8 * (B_VD_FULL + i), DEQ_WARPS);
            mbar_init(bar0 + 8 * (B_VD_EMPTY + i), 1);
        }
        mbar_init(bar0 + 8 * B_DONE, 1);
        mbar_init(bar0 + 8 * (B_DONE + 1), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    // q tile (B operand of S^T, K-major): core matrix (k-block kb, n-block nb) at (kb*2 + nb)*128, row = head,
    // 16 bytes = 8 channels; n-block 0 holds F16(q*scale), n-block 1 the rounding residual.
    for (int e = threadIdx.x; e < 8 * D; e += THREADS) {
        const int h = e >> 7, ch = e & (D - 1);
        const float x = (h < p.group) ? p.q[((int64_t)b * p.hq + kv * p.group + h) * D + ch] * p.scale_log2 : 0.f;
        const __half hi = __float2half_rn(x);
        const __half lo = __float2half_rn(x - __half2float(hi));
        uint8_t* at = smem + OFF_Q + (ch >> 3) * 256 + h * 16 + (ch & 7) * 2;
        *reinterpret_cast<__half*>(at) = hi;
        *reinterpret_cast<__half*>(at + 128) = lo;
    }
    // p tiles: n-block 0 is rewritten every tile, n-block 1 stays zero (the MMA needs N = 16)
    for (int e = threadIdx.x; e < P_BUFS * P_B / 16; e += THREADS) reinterpret_cast<uint4*>(smem + OFF_P)[e] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    float o_fin[8], m_ref[8], l_run[8];
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        o_fin[h] = 0.f;
        m_ref[h] = -INFINITY;
        l_run[h] = 0.f;
    }

    if (warp == 0) {
        // ───────── packed K/V groups -> shared memory (one thread) ─────────
        if (lane == 0) {
            // Groups of one flush are contiguous for K and for V, so a tile is fetched in runs (one run of 4 groups
            // when a flush holds a multiple of 4 groups); the position advances without divisions.
            int f = g0 / gpf, gif = g0 - f * gpf;
            int T = 0;   // tiles issued so far
            for (; T < n_tiles; ++T) {
                const int s = T % PK_STAGES;
                if (T >= PK_STAGES && !wait_or_abort(bar0 + 8 * (B_PK_EMPTY + s), ((T / PK_STAGES) - 1) & 1, abort_flag)) break;
                const int ng = min(GROUPS, n_groups - GROUPS * T);
                const uint32_t full = bar0 + 8 * (B_PK_FULL + s);
                const uint32_t dst = sbase + OFF_PK + s * PK_STAGE_B;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(full, (uint32_t)ng * 2 * GRP_B);
                for (int gi = 0; gi < ng;) {
                    const int run = min(ng - gi, gpf - gif);
                    const int64_t kblk = (((int64_t)f * p.hkv + kv) * gpf + gif) * D;
                    const int64_t vblk = (((int64_t)f * p.hkv + kv) * bt.res_cap + gif * 32) * (D / 32);
                    bulk_g2s(dst + gi * GRP_B, bt.qk[b] + kblk * BB, (uint32_t)run * GRP_B, full);
                    bulk_g2s(dst + (GROUPS + gi) * GRP_B, bt.qv[b] + vblk * BB, (uint32_t)run * GRP_B, full);
                    gi += run;
                    gif += run;
                    if (gif == gpf) {
                        gif = 0;
                        ++f;
                    }
                }
            }
            if (*abort_flag)   // gave up: let the copies still in flight land before shared memory is reused
                for (int Ti = max(0, T - PK_STAGES); Ti < T; ++Ti)
                    (void)mbar_wait(bar0 + 8 * (B_PK_FULL + Ti % PK_STAGES), (Ti / PK_STAGES) & 1);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ───────── S^T = K_d · q^T issue (one thread) ─────────
        // Next to 16 ALU-bound warps this thread gets few issue slots, so all descriptors are built before the loop
        // and a batch is nothing but eight tcgen05.mma.
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_f16(1, 0, 128, 16);   // A = K_d MN-major, B = q K-major
            constexpr uint32_t hi = desc_hi(128);                    // every operand: SBO 128
            uint64_t ad[2][8], bd[8];
#pragma unroll
            for (uint32_t ks = 0; ks < 8; ++ks) {
                ad[0][ks] = desc64(desc_lo(sbase + OFF_KD + ks * 4096, 2048), hi);
                ad[1][ks] = desc64(desc_lo(sbase + OFF_KD + KD_B + ks * 4096, 2048), hi);
                bd[ks] = desc64(desc_lo(sbase + OFF_Q + ks * 512, 256), hi);
            }
            for (int T = 0; T < n_tiles; ++T) {
                const uint32_t bf = T & 1;
                if (!wait_or_abort(bar0 + 8 * (B_KD_FULL + bf), (T >> 1) & 1, abort_flag)) break;
                // softmax(T-2) has read this S buffer once p(T-2) is complete
                if (T >= 2 && !wait_or_abort(bar0 + 8 * (B_P_FULL + (T - 2) % P_BUFS), ((T - 2) / P_BUFS) & 1, abort_flag)) break;
                tc_fence_after();
                if (bf == 0) {
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks) tc_mma64(tmem, ad[0][ks], bd[ks], idesc_s, ks > 0 ? 1u : 0u);
                } else {
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks) tc_mma64(tmem + 16, ad[1][ks], bd[ks], idesc_s, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar0 + 8 * (B_S_FULL + bf));
                tc_commit(bar0 + 8 * (B_KD_EMPTY + bf));
            }
            // nothing of this thread is in flight when tensor memory is released, whatever happened above
            tc_commit(bar0 + 8 * B_DONE);
            if (!mbar_wait(bar0 + 8 * B_DONE, 0)) *abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 2) {
        // ───────── O^T += V_d^T · p issue (one thread) ─────────
        if (lane == 0) {
            constexpr uint32_t idesc_o = idesc_f16(1, 1, 128, 16);   // A = V_d MN-major, B = p MN-major
            constexpr uint32_t hi = desc_hi(128);
            for (int T = 0; T < n_tiles; ++T) {
                const uint32_t vb = T % VD_BUFS, pb = T % P_BUFS;
                uint64_t ad[8], bd[8];   // built while there is nothing to issue
#pragma unroll
                for (uint32_t t = 0; t < 8; ++t) {
                    ad[t] = desc64(desc_lo(sbase + OFF_VD + vb * KD_B + t * 4096, 2048), hi);
                    bd[t] = desc64(desc_lo(sbase + OFF_P + pb * P_B + t * 512, 256), hi);
                }
                if (!wait_or_abort(bar0 + 8 * (B_VD_FULL + vb), (T / VD_BUFS) & 1, abort_flag)) break;
                if (!wait_or_abort(bar0 + 8 * (B_P_FULL + pb), (T / P_BUFS) & 1, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (uint32_t t = 0; t < 8; ++t) tc_mma64(tmem + O_COL, ad[t], bd[t], idesc_o, (T > 0 || t > 0) ? 1u : 0u);
                tc_commit(bar0 + 8 * (B_VD_EMPTY + vb));
            }
            tc_commit(bar0 + 8 * (B_DONE + 1));
            if (!mbar_wait(bar0 + 8 * (B_DONE + 1), 0)) *abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 3) {
        // spare warp: keeps the softmax warps on TMEM lane quarters 0..3 and the epilogue on threads 0..127
    } else if (warp >= FIRST_DEQ_WARP) {
        // ───────── dequantise: packed groups -> F16 operand tiles (one K block and one V block per thread) ─────────
        const int dt = threadIdx.x - FIRST_DEQ_WARP * 32;
        // K block (group kgi, channel kch): word w = tokens 8w.. of the group -> core matrix (token block 4kgi+w,
        // channel block kch/8) at (kch/8)*2048 + (4kgi+w)*128, row kch%8.
        const int kgi = dt >> 7, kch = dt & 127;
        const int k_src = kgi * GRP_B + kch * BB;
        const int k_dst = (kch >> 3) * 2048 + (4 * kgi) * 128 + (kch & 7) * 16;
        // V block (token vtt, channel block vblk): word w = channels 32vblk+8w.. -> core matrix (channel block
        // 4vblk+w, token block vtt/8) at (vtt/8)*2048 + (4vblk+w)*128, row = position of the token in its block.
        // Eight consecutive lanes take the eight tokens of one block, so that their rows fill one core matrix.
        const int va = dt & 7, vblk = (dt >> 3) & 3, vtt = (dt >> 5) * 8 + va, vgi = vtt >> 5;
        const int v_src = vgi * GRP_B + ((vtt & 31) * 4 + vblk) * BB;
        const int v_dst = (vtt >> 3) * 2048 + (4 * vblk) * 128 + invperm8(va) * 16;
        for (int T = 0; T < n_tiles; ++T) {
            const int s = T % PK_STAGES, bf = T & 1, vb = T % VD_BUFS;
            const int ng = min(GROUPS, n_groups - GROUPS * T);
            if (!warp_wait(bar0 + 8 * (B_PK_FULL + s), (T / PK_STAGES) & 1, abort_flag)) break;
            const uint8_t* pk_k = smem + OFF_PK + s * PK_STAGE_B;
            const uint8_t* pk_v = pk_k + GROUPS * GRP_B;
            uint4 kvec[4], vvec[4];
            if (kgi < ng) dequant_block_q4(pk_k + k_src, kvec);
            else kvec[0] = kvec[1] = kvec[2] = kvec[3] = make_uint4(0u, 0u, 0u, 0u);
            if (vgi < ng) dequant_block_q4(pk_v + v_src, vvec);
            else vvec[0] = vvec[1] = vvec[2] = vvec[3] = make_uint4(0u, 0u, 0u, 0u);
            // the codes are in registers (the values above depend on every load): the packed stage may be refilled
            warp_arrive(bar0 + 8 * (B_PK_EMPTY + s), lane);
            if (T >= 2 && !warp_wait(bar0 + 8 * (B_KD_EMPTY + bf), ((T >> 1) - 1) & 1, abort_flag)) break;
            uint8_t* kd = smem + OFF_KD + bf * KD_B + k_dst;
#pragma unroll
            for (int w = 0; w < 4; ++w) *reinterpret_cast<uint4*>(kd + w * 128) = kvec[w];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            warp_arrive(bar0 + 8 * (B_KD_FULL + bf), lane);
            if (T >= VD_BUFS && !warp_wait(bar0 + 8 * (B_VD_EMPTY + vb), ((T / VD_BUFS) - 1) & 1, abort_flag)) break;
            uint8_t* vd = smem + OFF_VD + vb * KD_B + v_dst;
#pragma unroll
            for (int w = 0; w < 4; ++w) *reinterpret_cast<uint4*>(vd + w * 128) = vvec[w];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            warp_arrive(bar0 + 8 * (B_VD_FULL + vb), lane);
        }
    } else {
        // ───────── softmax: thread = TMEM lane L = token position of S^T, channel position of O^T ─────────
        const int L = 32 * (warp & 3) + lane;
        const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
        const int tok_in_tile = (L & ~7) + perm8(L & 7);
        int* red = reinterpret_cast<int*>(smem + OFF_RED);
        bool gave_up = false;
        // The reference point m_ref of exp2(s - m_ref) only has to be near the running maximum (it is raised when a
        // tile exceeds it by more than LAZY), so the tile maximum is taken on the bits of s + MAX_OFS as signed
        // integers: non-negative floats order like their bits, one redux.sync per head. Logits (log2 units) below
        // -MAX_OFS, masked positions included, are clamped there: exp2 of them against any sane maximum is zero.
        constexpr float MAX_OFS = 16384.f;   // resolution of the maximum: 2^-9 near zero, one ulp for huge logits
        for (int T = 0; T < n_tiles; ++T) {
            const int bf = T & 1;
            const int ng = min(GROUPS, n_groups - GROUPS * T);
            const bool s_ok = wait_or_abort(bar0 + 8 * (B_S_FULL + bf), (T >> 1) & 1, abort_flag);
            tc_fence_after();
            uint32_t r[16];
            tmem_ld16(tmem + lane_off + 16 * bf, r);
            tmem_wait_ld();
            const bool valid = L < 32 * ng;
            float s[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) s[h] = valid ? __uint_as_float(r[h]) + __uint_as_float(r[8 + h]) : -INFINITY;
            int* rd = red + (T & 1) * 32;
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                const int k = __reduce_max_sync(0xffffffffu, __float_as_int(fmaxf(s[h], -MAX_OFS) + MAX_OFS));
                if (lane == 0) rd[(warp & 3) * 8 + h] = k;
            }
            // the tile-maximum exchange doubles as the give-up vote: the 128 threads leave the loop together
            if (softmax_bar_or(!s_ok || *abort_flag != 0)) {
                gave_up = true;
                break;
            }
            if (p.logits != nullptr && valid) {
                const int64_t tok = (int64_t)(g0 + GROUPS * T) * 32 + tok_in_tile;
#pragma unroll
                for (int h = 0; h < 8; ++h)
                    if (h < p.group) p.logits[((int64_t)b * p.hq + kv * p.group + h) * p.logit_stride + tok] = s[h];
            }
            float tmax[8];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                int4 x = *reinterpret_cast<const int4*>(rd + hh * 4);
#pragma unroll
                for (int w = 1; w < 4; ++w) {
                    const int4 y = *reinterpret_cast<const int4*>(rd + w * 8 + hh * 4);
                    x.x = max(x.x, y.x); x.y = max(x.y, y.y); x.z = max(x.z, y.z); x.w = max(x.w, y.w);
                }
                tmax[hh * 4 + 0] = __int_as_float(x.x) - MAX_OFS; tmax[hh * 4 + 1] = __int_as_float(x.y) - MAX_OFS;
                tmax[hh * 4 + 2] = __int_as_float(x.z) - MAX_OFS; tmax[hh * 4 + 3] = __int_as_float(x.w) - MAX_OFS;
            }
            bool need = false;
#pragma unroll
            for (int h = 0; h < 8; ++h) need |= tmax[h] > m_ref[h] + LAZY;
            if (need) {   // uniform over the 128 threads: they all see the same maxima
                float alpha[8];
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    const bool up = tmax[h] > m_ref[h] + LAZY;
                    alpha[h] = up ? fast_exp2(m_ref[h] - tmax[h]) : 1.f;
                    if (up) m_ref[h] = tmax[h];
                    l_run[h] *= alpha[h];
                }
                if (T > 0) {
                    (void)wait_or_abort(bar0 + 8 * (B_VD_EMPTY + (T - 1) % VD_BUFS), ((T - 1) / VD_BUFS) & 1, abort_flag);
                    tc_fence_after();
                    uint32_t o[16];
                    tmem_ld16(tmem + lane_off + O_COL, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int h = 0; h < 8; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
                    tmem_st16(tmem + lane_off + O_COL, o);
                    tmem_wait_st();
                }
            }
            float pr[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                pr[h] = fast_exp2(s[h] - ((m_ref[h] == -INFINITY) ? 0.f : m_ref[h]));
                l_run[h] += pr[h];
            }
            // P·V(T-3) read this p buffer: it has to be complete before the buffer is rewritten. (It also keeps
            // p_full from running two phases ahead of the P·V issuer, which waits on its parity.)
            if (T >= P_BUFS)
                (void)wait_or_abort(bar0 + 8 * (B_VD_EMPTY + (T - P_BUFS) % VD_BUFS), ((T - P_BUFS) / VD_BUFS) & 1, abort_flag);
            // p as F16 (<= 2^LAZY, relative error 2^-11): one 16-byte row of 8 heads
            uint8_t* pt = smem + OFF_P + (T % P_BUFS) * P_B + (L >> 3) * 256 + (L & 7) * 16;
            *reinterpret_cast<uint4*>(pt) = make_uint4(pack_half2(pr[0], pr[1]), pack_half2(pr[2], pr[3]),
                                                       pack_half2(pr[4], pr[5]), pack_half2(pr[6], pr[7]));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            warp_arrive(bar0 + 8 * (B_P_FULL + T % P_BUFS), lane);
        }
        if (n_tiles > 0 && !gave_up) {
            const int Tl = n_tiles - 1;   // the last P·V
            if (!mbar_wait(bar0 + 8 * (B_VD_EMPTY + Tl % VD_BUFS), (Tl / VD_BUFS) & 1)) *abort_flag = 1;
            tc_fence_after();
            uint32_t o[16];
            tmem_ld16(tmem + lane_off + O_COL, o);
            tmem_wait_ld();
#pragma unroll
            for (int h = 0; h < 8; ++h) o_fin[h] = __uint_as_float(o[h]);
        }
        float* rs = reinterpret_cast<float*>(red + 64);
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            float x = l_run[h];
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) x += __shfl_xor_sync(0xffffffffu, x, sh);
            if (lane == 0) rs[(warp & 3) * 8 + h] = x;
        }
        softmax_bar();
#pragma unroll
        for (int h = 0; h < 8; ++h) l_run[h] = rs[h] + rs[8 + h] + rs[16 + h] + rs[24 + h];
    }

    tc_fence_before();
    __syncthreads();   // every copy has landed and every MMA has completed: the pipeline memory is free
    const bool aborted = *abort_flag != 0;
    float* sm_o = reinterpret_cast<float*>(smem + EpilogueSmem<D, 4>::O_OFF);
    float2* sm_ml = reinterpret_cast<float2*>(smem + EpilogueSmem<D, 4>::ML_OFF);
    // the epilogue merges four warp slots: slot 0 is this CTA's result, slots 1..3 are neutral
    for (int e = threadIdx.x; e < 3 * 8 * D; e += THREADS) sm_o[8 * D + e] = 0.f;
    if (threadIdx.x < 24) sm_ml[8 + threadIdx.x] = make_float2(-INFINITY, 0.f);
    if (warp >= 4 && warp < 8) {
        const int L = 32 * (warp & 3) + lane;
        const int ch = (L & ~7) + perm8(L & 7);
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            sm_o[h * D + ch] = aborted ? 0.f : o_fin[h];
            if (L == h) sm_ml[h] = aborted ? make_float2(-INFINITY, 0.f) : make_float2(m_ref[h], l_run[h]);
        }
    }
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
        if (aborted && lane == 0 && p.status != nullptr) atomicExch(p.status, 1);
    }
    if (threadIdx.x >= 128) return;
    decode_epilogue<D, 4>(smem, p, b, kv, item, item0, n_splits);
}

}  // namespace ktc

// Packed-part splits of this kernel are planned in whole tiles of 4 groups; one CTA per SM.
cudaError_t launch_decode_kivi_tc(const DecodeParams& p, const KiviBatch& bt, int n_items, cudaStream_t st) {
    static bool attr_done[kMaxDevices] = {};
    cudaError_t ea = ensure_dynamic_smem(reinterpret_cast<const void*>(ktc::decode_kivi_tc_kernel), ktc::SMEM_B, attr_done);
    if (ea != cudaSuccess) return ea;
    ktc::decode_kivi_tc_kernel<<<n_items * p.hkv, ktc::THREADS, ktc::SMEM_B, st>>>(p, bt);
    return cudaGetLastError();
}

}  // namespace argus
