// Causal GQA flash-attention prefill on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a.
//
// Stands behind Backend::flash_attention_prefill (engine/src/backend.rs:1011-1027; CUDA implementation
// engine/src/backend/cuda_pc.rs:830-926 with flash_attn_prefill_f16kv_dk128, engine/src/backend/cuda_pc/
// kernels.cu:691-816). Same contract: Q/O [B][S][Hq][D], K/V HeadMajor [B][Hkv][cap][D], query row r sees
// keys <= cache_seq_len - seq_len + r, rows without a visible key produce zeros. The reference runs one
// thread per query row with scalar FMAs; here one CTA owns two 128-row query tiles of one head, TMA feeds
// 128B-swizzled Q/K/V tiles, one thread issues tcgen05.mma for S = Q·K^T and O += P·V with the accumulators
// (and P) in tensor memory, and eight softmax warps own one query row per thread. The kernel comment below
// gives the roles and the TMEM map. Every mbarrier wait is bounded; a wait that runs out raises the status
// word, makes every role leave its loop, and the CTA still frees its TMEM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace argus {

struct PrefillParams {
    void* out;          // [B][S][Hq][D] 16-bit (same type as Q) or F32
    int B, S, T, hq, hkv, group;
    int n_qtiles;
    float scale_log2;
    int* status;
};

namespace pf {

constexpr int BM = 128, BN = 128, D = 128;
constexpr int TILE_B = BM * D * 2;          // 32 KB: one Q/K/V/P tile of 16-bit elements
constexpr int HALF_B = TILE_B / 2;          // one 64-column (128-byte wide) swizzled block of a tile
constexpr int K_STAGES = 3, V_STAGES = 2;      // K is needed one tile ahead of V (S_{j+1} is issued before P_j·V_j)
constexpr int OFF_Q = 0;                       // two query tiles
constexpr int OFF_K = OFF_Q + 2 * TILE_B;
constexpr int OFF_V = OFF_K + K_STAGES * TILE_B;
constexpr int OFF_BAR = OFF_V + V_STAGES * TILE_B;   // 224 KB
constexpr int N_BAR = 1 + 2 * K_STAGES + 3 * V_STAGES + 6;
constexpr int SMEM_B = OFF_BAR + N_BAR * 8 + 16 + 1024;   // + TMEM base slot + alignment slack
constexpr uint32_t TMEM_COLS = 512;
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
// Bounded wait: returns false when the phase did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < (1 << 24); ++it) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,"
        "%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
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

// Shared-memory matrix descriptor (sm_100 format: version 1 at bit 46, layout type SWIZZLE_128B = 2 at bit 61).
// Offsets are in 16-byte units.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: F32 accumulate, A/B format (0 = F16, 1 = BF16), B major, N, M.
__host__ __device__ constexpr uint32_t instr_desc(int fmt, int b_mn_major, int M, int N) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
    if constexpr (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    } else {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
}

}  // namespace pf

// tcgen05.mma with the A operand in tensor memory (16-bit elements, two per 32-bit column, K-major).
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// Packed F32 pairs (sm_100): one issue slot for two FMAs / adds.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// One CTA = two 128-row query tiles (X = 0, 1) of one head, FlashAttention-4 style:
//   warp 0        TMA producer (Q0, Q1 once; K_j, V_j stages)
//   warp 1        MMA issuer: S_X = Q_X·K_j^T into TMEM, O_X += P_X·V_j with P_X read from TMEM
//   warps 2..3    idle (they only exist so that the register budget can move between whole warpgroups)
//   warps 4..7    softmax of tile 0, warps 8..11 softmax of tile 1 (one query row per thread)
// TMEM: S_0 [0,128) S_1 [128,256) O_0 [256,384) O_1 [384,512). P_X overwrites S_X in place as 16-bit
// pairs (columns [0,64) of the region; with PSPLIT the rounding residual goes to [64,128) and P·V runs
// twice, which keeps ~16 bits of P when the cache type is BF16). The tensor pipe executes one thread's
// MMAs in issue order, so S_X(j+1) may be issued right behind P_X(j)·V_j although it reuses the region.
// While one tile's softmax runs, the tensor pipe works on the other tile.
template <bool BF16, bool OUT_F32, bool PSPLIT, bool VCONV>
__global__ void __launch_bounds__(384, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ PrefillParams p) {
    using namespace pf;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;   // 128B-swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (smem0 - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t bar = smem0 + OFF_BAR;
    const uint32_t b_qfull = bar;
    auto b_kfull = [&](int s) { return bar + 8 * (1 + s); };
    auto b_kempty = [&](int s) { return bar + 8 * (1 + K_STAGES + s); };
    auto b_vfull = [&](int s) { return bar + 8 * (1 + 2 * K_STAGES + s); };
    auto b_vempty = [&](int s) { return bar + 8 * (1 + 2 * K_STAGES + V_STAGES + s); };
    auto b_vconv = [&](int s) { return bar + 8 * (1 + 2 * K_STAGES + 2 * V_STAGES + s); };   // V tile converted to F16 (VCONV)
    const uint32_t bar2 = bar + 8 * (1 + 2 * K_STAGES + 3 * V_STAGES);
    auto b_sfull = [&](int x) { return bar2 + 8 * x; };
    auto b_pfull = [&](int x) { return bar2 + 8 * (2 + x); };
    auto b_ofull = [&](int x) { return bar2 + 8 * (4 + x); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + N_BAR * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_BAR + N_BAR * 8 + 8);

    // work item: long query tiles first (they see the most keys); heads of one KV group are adjacent CTAs
    const int qt = p.n_qtiles - 1 - (int)(blockIdx.x / (p.hq * p.B));
    const int hb = blockIdx.x % (p.hq * p.B);
    const int h = hb % p.hq, b = hb / p.hq;
    const int kvh = h / p.group;
    const int r0 = qt * (2 * BM);
    const int q_start = p.T - p.S;                                   // global position of query row 0
    // keys [0, kv_end_x) can be visible to tile x; a tile that starts past the last query row does nothing
    int n_x[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int kv_end = (r0 + x * BM < p.S) ? min(p.T, q_start + r0 + x * BM + BM) : 0;
        n_x[x] = (kv_end + BN - 1) / BN;
    }
    const int n_tiles = max(n_x[0], n_x[1]);

    if (threadIdx.x == 0) {
        mbar_init(b_qfull, 1);
        for (int s = 0; s < K_STAGES; ++s) {
            mbar_init(b_kfull(s), 1);
            mbar_init(b_kempty(s), 1);
        }
        for (int s = 0; s < V_STAGES; ++s) {
            mbar_init(b_vfull(s), 1);
            mbar_init(b_vconv(s), 64);
            mbar_init(b_vempty(s), 1);
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(b_sfull(x), 1);
            mbar_init(b_pfull(x), 128);
            mbar_init(b_ofull(x), 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem0 + OFF_BAR + N_BAR * 8),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    auto fail = [&]() {
        *abort_flag = 1;
        if (p.status != nullptr) atomicExch(p.status, 2);
    };

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 128;");
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
    }
    if (warp == 0) {
        // ───────── TMA producer ─────────
        if (lane == 0) {
            mbar_expect_tx(b_qfull, 2 * TILE_B);
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                tma_load_4d(smem0 + OFF_Q + x * TILE_B, &tm_q, b_qfull, 0, r0 + x * BM, h, b);
                tma_load_4d(smem0 + OFF_Q + x * TILE_B + HALF_B, &tm_q, b_qfull, 64, r0 + x * BM, h, b);
            }
            for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
                const int s = j % K_STAGES, sv = j % V_STAGES;
                if (j >= K_STAGES && !mbar_wait(b_kempty(s), ((j / K_STAGES) & 1) ^ 1)) { fail(); break; }
                mbar_expect_tx(b_kfull(s), TILE_B);
                tma_load_4d(smem0 + OFF_K + s * TILE_B, &tm_k, b_kfull(s), 0, j * BN, kvh, b);
                tma_load_4d(smem0 + OFF_K + s * TILE_B + HALF_B, &tm_k, b_kfull(s), 64, j * BN, kvh, b);
                if (j >= V_STAGES && !mbar_wait(b_vempty(sv), ((j / V_STAGES) & 1) ^ 1)) { fail(); break; }
                mbar_expect_tx(b_vfull(sv), TILE_B);
                tma_load_4d(smem0 + OFF_V + sv * TILE_B, &tm_v, b_vfull(sv), 0, j * BN, kvh, b);
                tma_load_4d(smem0 + OFF_V + sv * TILE_B + HALF_B, &tm_v, b_vfull(sv), 64, j * BN, kvh, b);
            }
        }
    } else if (warp == 1) {
        // ───────── MMA issuer ─────────
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(BF16 ? 1 : 0, 0, BM, BN);   // K tile is K-major
            // With VCONV the V tile has been rewritten as F16 in shared memory and P is packed as F16 too.
            constexpr uint32_t idesc_o = instr_desc((BF16 && !VCONV) ? 1 : 0, 1, BM, D);    // V tile is MN-major
            bool ok = mbar_wait(b_qfull, 0);
            auto issue_s = [&](int x, int j) {
                const int s = j % K_STAGES;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t qa = smem0 + OFF_Q + x * TILE_B + (k >> 2) * HALF_B + (k & 3) * 32;
                    const uint32_t ka = smem0 + OFF_K + s * TILE_B + (k >> 2) * HALF_B + (k & 3) * 32;
                    tc_mma(tmem + x * 128, smem_desc(qa, 16, 1024), smem_desc(ka, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
                }
                tc_commit(b_sfull(x));
            };
            auto issue_pv = [&](int x, int j) {
                const int s = j % V_STAGES;
#pragma unroll
                for (int pass = 0; pass < (PSPLIT ? 2 : 1); ++pass)
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k) {
                        // A = P from TMEM: 16 keys = 8 columns per k-step. B = V: MN-major, d along the 128-byte
                        // rows (two 64-d blocks LBO = 16 KB apart), 8 keys per 1024-byte group (SBO), 16 keys = 2 KB.
                        const uint32_t va = smem0 + OFF_V + s * TILE_B + k * 2048;
                        tc_mma_ts(tmem + 256 + x * 128, tmem + x * 128 + pass * 64 + k * 8, smem_desc(va, HALF_B, 1024),
                                  idesc_o, (j > 0 || k > 0 || pass > 0) ? 1u : 0u);
                    }
            };
            if (ok && n_tiles > 0) {
                ok = mbar_wait(b_kfull(0), 0);
                if (ok) {
                    tc_fence_after();
                    if (n_x[0] > 0) issue_s(0, 0);
                    if (n_x[1] > 0) issue_s(1, 0);
                    tc_commit(b_kempty(0));
                }
            }
            for (int j = 0; j < n_tiles && ok && !*abort_flag; ++j) {
                const int s = j % V_STAGES;
                const bool more = (j + 1 < n_tiles);
                bool v_ready = false, k_ready = false;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (j < n_x[x]) {
                        ok = mbar_wait(b_pfull(x), j & 1);
                        if (ok && !v_ready) { ok = mbar_wait(VCONV ? b_vconv(s) : b_vfull(s), (j / V_STAGES) & 1); v_ready = true; }
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv(x, j);
                        if (j + 1 >= n_x[x]) tc_commit(b_ofull(x));
                    }
                    if (j + 1 < n_x[x]) {
                        if (!k_ready) { ok = mbar_wait(b_kfull((j + 1) % K_STAGES), ((j + 1) / K_STAGES) & 1); k_ready = true; }
                        if (!ok) break;
                        tc_fence_after();
                        issue_s(x, j + 1);
                    }
                }
                if (!ok) break;
                tc_commit(b_vempty(s));
                if (more) tc_commit(b_kempty((j + 1) % K_STAGES));
            }
            if (!ok) fail();
        }
    } else if (warp < 4) {
        // ───────── warps 2..3: V tile BF16 -> F16 in place (VCONV only), otherwise idle ─────────
        if constexpr (VCONV) {
            const int t64 = threadIdx.x - 64;   // 0..63
            bool clamped = false;   // a finite BF16 value beyond the F16 range met the saturating conversion
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % V_STAGES;
                if (*abort_flag || !mbar_wait(b_vfull(s), (j / V_STAGES) & 1)) { fail(); break; }
                uint4* tile = reinterpret_cast<uint4*>(smem + OFF_V + s * TILE_B);
#pragma unroll 4
                for (int i = 0; i < TILE_B / 16 / 64; ++i) {
                    uint4 w = tile[t64 + 64 * i];
                    uint32_t* e = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float lo = __uint_as_float(e[k] << 16), hi = __uint_as_float(e[k] & 0xffff0000u);
                        uint32_t r;
                        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
                        clamped |= fmaxf(fabsf(lo), fabsf(hi)) > 65504.0f;   // false for NaN; the BF16 infinities count too
                        e[k] = r;
                    }
                    tile[t64 + 64 * i] = w;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(b_vconv(s));
            }
            // informational status 4, never over an error code already there
            if (clamped && p.status != nullptr) atomicCAS(p.status, 0, 4);
        }
    } else {
        // ───────── softmax / correction / epilogue: one query row per thread ─────────
        const int x = (warp - 4) >> 2;                      // which query tile
        const int quarter = warp & 3;                       // TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;
        const uint32_t t_s = tmem + ((uint32_t)(quarter * 32) << 16) + x * 128;
        const uint32_t t_o = tmem + ((uint32_t)(quarter * 32) << 16) + 256 + x * 128;
        const int rq = r0 + x * BM + row;                   // query row inside the sequence
        const int qi = q_start + rq;                        // its global position
        const int n_mine = n_x[x];
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_mine; ++j) {
            if (*abort_flag || !mbar_wait(b_sfull(x), j & 1)) { ok = false; break; }
            tc_fence_after();
            // pass 1: row maximum (the S row is read twice from tensor memory rather than held in 128 registers)
            const bool diag = (j * BN + BN - 1 > q_start + r0 + x * BM);   // some key of this tile may be masked
            float mx = -INFINITY;
            {
                // four independent max chains
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    uint32_t sv[2][32];
                    tmem_ld32(t_s + hf * 64, sv[0]);
                    tmem_ld32(t_s + hf * 64 + 32, sv[1]);
                    tmem_wait_ld();
                    if (diag) {
#pragma unroll
                        for (int c = 0; c < 2; ++c)
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (j * BN + hf * 64 + c * 32 + i <= qi)
                                    m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sv[c][i]));
                    } else {
#pragma unroll
                        for (int c = 0; c < 2; ++c)
#pragma unroll
                            for (int i = 0; i < 32; i += 2)
                                m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
                    }
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            const float m_tile = mx * p.scale_log2;
            float alpha = 1.f;
            if (m_tile > m_ref + LAZY) {                    // also the first tile (m_ref = -inf)
                alpha = fast_exp2(m_ref - m_tile);
                m_ref = m_tile;
            }
            // O rescale (rare after the first tiles). s_full(j) was committed behind P·V of tile j-1, so O is quiescent.
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t ov[32];
                    tmem_ld32(t_o + c * 32, ov);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                    tmem_st32(t_o + c * 32, ov);
                }
            }
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
            uint64_t psum2 = pack_f32x2(0.f, 0.f), psum2b = pack_f32x2(0.f, 0.f);
            const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), negm2 = pack_f32x2(neg_m, neg_m);
            if constexpr (!PSPLIT) {
                // pass 2, pipelined by 32-key chunks: chunk c+1 is in flight while chunk c is turned into P.
                // P chunk c (16 packed columns at 16c) lands inside S chunk c/2, which has been read by then.
                uint32_t sbuf[2][32];
                tmem_ld32(t_s, sbuf[0]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (c + 1 < 4) tmem_ld32(t_s + (c + 1) * 32, sbuf[(c + 1) & 1]);
                    uint32_t hi16[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float s0 = __uint_as_float(sbuf[c & 1][2 * e]), s1 = __uint_as_float(sbuf[c & 1][2 * e + 1]);
                        if (diag) {
                            const int kc = j * BN + c * 32 + 2 * e;
                            if (kc > qi) s0 = -INFINITY;
                            if (kc + 1 > qi) s1 = -INFINITY;
                        }
                        float x0, x1;
                        unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), scale2, negm2), x0, x1);
                        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                        if (e & 1) psum2b = add_f32x2(psum2b, pack_f32x2(p0, p1));
                        else psum2 = add_f32x2(psum2, pack_f32x2(p0, p1));
                        hi16[e] = pack16<BF16 && !VCONV>(p0, p1);
                    }
                    if (c + 1 < 4) tmem_wait_ld();
                    tmem_st16(t_s + c * 16, hi16);
                }
            } else {
            // pass 2: p = exp2(s*scale - m), packed to 16 bits. P overwrites S in place: the first half's results
            // are stored only after the second half of S has been read.
            uint32_t hi[2][32], lo[PSPLIT ? 2 : 1][PSPLIT ? 32 : 1];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint32_t sv[2][32];
                tmem_ld32(t_s + hf * 64, sv[0]);
                tmem_ld32(t_s + hf * 64 + 32, sv[1]);
                tmem_wait_ld();
                if (hf == 1) {
                    tmem_st32(t_s, hi[0]);
                    if constexpr (PSPLIT) tmem_st32(t_s + 64, lo[0]);
                }
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float s0 = __uint_as_float(sv[c][2 * e]), s1 = __uint_as_float(sv[c][2 * e + 1]);
                        if (diag) {
                            const int kc = j * BN + hf * 64 + c * 32 + 2 * e;
                            if (kc > qi) s0 = -INFINITY;
                            if (kc + 1 > qi) s1 = -INFINITY;
                        }
                        float x0, x1;
                        unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), scale2, negm2), x0, x1);
                        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                        psum2 = add_f32x2(psum2, pack_f32x2(p0, p1));
                        const uint32_t w = pack16<BF16 && !VCONV>(p0, p1);
                        hi[hf][c * 16 + e] = w;
                        if constexpr (PSPLIT) {
                            float h0, h1;
                            if constexpr (BF16) {
                                h0 = __uint_as_float(w << 16);
                                h1 = __uint_as_float(w & 0xffff0000u);
                            } else {
                                const float2 hf2 = unpack_half2(w);
                                h0 = hf2.x;
                                h1 = hf2.y;
                            }
                            lo[hf][c * 16 + e] = pack16<BF16>(p0 - h0, p1 - h1);
                        }
                    }
            }
            tmem_st32(t_s + 32, hi[1]);
            if constexpr (PSPLIT) tmem_st32(t_s + 96, lo[1]);
            }
            psum2 = add_f32x2(psum2, psum2b);
            float psum0, psum1;
            unpack_f32x2(psum2, psum0, psum1);
            l = l * alpha + (psum0 + psum1);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(b_pfull(x));
        }
        // epilogue
        if (ok && n_mine > 0 && !*abort_flag) ok = mbar_wait(b_ofull(x), 0);
        if (!ok) fail();
        tc_fence_after();
        const bool row_ok = rq < p.S;
        const float inv_l = (ok && l > 0.f) ? 1.0f / l : 0.f;
        const int64_t obase = (((int64_t)b * p.S + rq) * p.hq + h) * D;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t ov[32];
            if (ok && n_mine > 0) {
                tmem_ld32(t_o + c * 32, ov);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) ov[i] = 0;
            }
            if (row_ok) {
                if constexpr (OUT_F32) {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + obase + c * 32);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        dst[i] = make_float4(__uint_as_float(ov[4 * i]) * inv_l, __uint_as_float(ov[4 * i + 1]) * inv_l,
                                             __uint_as_float(ov[4 * i + 2]) * inv_l, __uint_as_float(ov[4 * i + 3]) * inv_l);
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + obase + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            w[e] = pack16<BF16>(__uint_as_float(ov[8 * i + 2 * e]) * inv_l,
                                                __uint_as_float(ov[8 * i + 2 * e + 1]) * inv_l);
                        dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

// F32 -> F16 copy of Q for the engine's F32-Q entry.
__global__ void __launch_bounds__(256) cast_f32_to_f16_kernel(const float* __restrict__ src, __half* __restrict__ dst,
                                                              long long n) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        *reinterpret_cast<__half2*>(dst + i) = __floats2half2_rn(v.x, v.y);
        *reinterpret_cast<__half2*>(dst + i + 2) = __floats2half2_rn(v.z, v.w);
    } else {
        for (long long k = i; k < n; ++k) dst[k] = __float2half_rn(src[k]);
    }
}

// ── host side ──
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 4-D view {D, rows, heads, batch} of a 16-bit tensor with a {64, 128, 1, 1} box, 128-byte swizzle, zero fill.
static bool make_map(CUtensorMap* m, bool bf16, const void* base, uint64_t rows, uint64_t heads, uint64_t batch,
                     uint64_t row_stride_e, uint64_t head_stride_e, uint64_t batch_stride_e) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return false;
    cuuint64_t dims[4] = {128, rows, heads, batch};
    cuuint64_t strides[3] = {row_stride_e * 2, head_stride_e * 2, batch_stride_e * 2};
    cuuint32_t box[4] = {64, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base),
               dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// q16/k/v: 16-bit tensors (BF16 or F16). K/V element (b, kvh, t, c) at b*kv_batch_stride + kvh*kv_head_stride +
// t*kv_pos_stride + c (elements). Returns cudaErrorNotSupported when the driver entry point is missing.
cudaError_t launch_prefill_tc(const void* q16, const void* k, const void* v, void* out, bool bf16, bool out_f32, int B,
                              int S, int T, int hq, int hkv, int64_t cap_rows, int64_t kv_pos_stride,
                              int64_t kv_head_stride, int64_t kv_batch_stride, int p_mode, int* status, cudaStream_t st) {
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, bf16, q16, (uint64_t)S, (uint64_t)hq, (uint64_t)B, (uint64_t)hq * 128, 128, (uint64_t)S * hq * 128) ||
        !make_map(&mk, bf16, k, (uint64_t)cap_rows, (uint64_t)hkv, (uint64_t)B, (uint64_t)kv_pos_stride,
                  (uint64_t)kv_head_stride, (uint64_t)kv_batch_stride) ||
        !make_map(&mv, bf16, v, (uint64_t)cap_rows, (uint64_t)hkv, (uint64_t)B, (uint64_t)kv_pos_stride,
                  (uint64_t)kv_head_stride, (uint64_t)kv_batch_stride))
        return cudaErrorNotSupported;
    PrefillParams p;
    p.out = out;
    p.B = B;
    p.S = S;
    p.T = T;
    p.hq = hq;
    p.hkv = hkv;
    p.group = hq / hkv;
    p.n_qtiles = (S + 2 * pf::BM - 1) / (2 * pf::BM);
    p.scale_log2 = (1.0f / sqrtf(128.0f)) * 1.4426950408889634f;
    p.status = status;
    const int grid = p.n_qtiles * hq * B;
    auto launch = [&](auto kern) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pf::SMEM_B);
        if (e != cudaSuccess) return e;
        kern<<<grid, 384, pf::SMEM_B, st>>>(mq, mk, mv, p);
        return cudaGetLastError();
    };
    // BF16 keeps 8 significant bits of P per MMA operand, which does not hold the 2e-3 absolute tolerance.
    // p_mode 2 (default for BF16): the V tile is rewritten as F16 in shared memory by two otherwise idle warps
    // (exact for |v| < 65504, saturating beyond) and P is F16 (11 bits). p_mode 1: P = BF16 rounding + residual,
    // two P.V passes, exact for any V. p_mode 0: single BF16 P (fastest, outside the tolerance on rare elements).
    if (bf16) {
        if (p_mode == 2) return out_f32 ? launch(prefill_tc_kernel<true, true, false, true>) : launch(prefill_tc_kernel<true, false, false, true>);
        if (p_mode == 1) return out_f32 ? launch(prefill_tc_kernel<true, true, true, false>) : launch(prefill_tc_kernel<true, false, true, false>);
        return out_f32 ? launch(prefill_tc_kernel<true, true, false, false>) : launch(prefill_tc_kernel<true, false, false, false>);
    }
    return out_f32 ? launch(prefill_tc_kernel<false, true, false, false>) : launch(prefill_tc_kernel<false, false, false, false>);
}

cudaError_t launch_cast_f32_to_f16(const float* src, void* dst, long long n, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    const long long threads = (n + 3) / 4;
    cast_f32_to_f16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(src, static_cast<__half*>(dst), n);
    return cudaGetLastError();
}

}  // namespace argus
