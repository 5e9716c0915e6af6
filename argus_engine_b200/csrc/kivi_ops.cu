// KIVI container kernels: bit-exact block pack (flush), block unpack into the F16 view, residual ring
// write and residual scatter.
//
// Reference interfaces: CudaQuantAttnBackend::{gather_update_quant, dequant_flush, scatter_residual}
// (crates/argus-extension-api/src/lib.rs:3094-3103; kernels crates/techniques/kivi/src/kivi_q2.cu:19-138),
// and the CPU flush the engine runs before uploading blocks (QuantizedRecentWindowCache::flush_residual,
// engine/src/kv/quant_window_cache.rs:844-965) with the codecs of crates/argus-kv-codec/src/lib.rs:36-202.
//
// Bit-exactness of the pack: every step uses the explicitly rounded intrinsics (__fsub_rn, __fmul_rn,
// __fdiv_rn) so that nvcc cannot contract or approximate, roundf is half-away-from-zero like Rust's
// f32::round, fminf/fmaxf skip NaN like f32::min/max, NaN codes become 0 like Rust's `as u8`, and the f16
// parameters are stored round-to-nearest-even like half::f16::from_f32. min/max are order-independent.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace argus {

__device__ __forceinline__ int block_bytes_dev(int bits) { return bits == 2 ? 12 : bits == 4 ? 20 : 36; }

// One warp packs one block: lane i holds element i. Writes block_bytes(bits) bytes at dst.
__device__ __forceinline__ void pack_block_warp(float x, int bits, uint8_t* dst) {
    const int lane = threadIdx.x & 31;
    float mn = x, mx = x;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, sh));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    }
    const float L = bits == 2 ? 3.0f : bits == 4 ? 15.0f : 255.0f;
    const float d = __fdiv_rn(__fsub_rn(mx, mn), L);
    const float id = (d == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d);
    float r = roundf(__fmul_rn(__fsub_rn(x, mn), id));
    r = (r != r) ? 0.0f : fminf(fmaxf(r, 0.0f), L);
    const uint32_t code = (uint32_t)r;
    if (lane == 0) {
        reinterpret_cast<__half*>(dst)[0] = __float2half_rn(d);
        reinterpret_cast<__half*>(dst)[1] = __float2half_rn(mn);
    }
    if (bits == 8) {
        dst[4 + lane] = (uint8_t)code;
    } else if (bits == 4) {
        const uint32_t hi = __shfl_down_sync(0xffffffffu, code, 1);
        if ((lane & 1) == 0) dst[4 + (lane >> 1)] = (uint8_t)(code | (hi << 4));
    } else {
        const uint32_t c1 = __shfl_down_sync(0xffffffffu, code, 1);
        const uint32_t c2 = __shfl_down_sync(0xffffffffu, code, 2);
        const uint32_t c3 = __shfl_down_sync(0xffffffffu, code, 3);
        if ((lane & 3) == 0) dst[4 + (lane >> 2)] = (uint8_t)(code | (c1 << 2) | (c2 << 4) | (c3 << 6));
    }
}

// Flush of n_groups*32 ring tokens. K: grid (D/32, n_groups, Hkv), 1024 threads: a 32x32 (token x channel)
// tile goes through shared memory so that global reads run along channels and each warp then owns one
// channel's 32 tokens. Blocks land at qk + (k_block_start + (h*n_groups + g)*D + ch) * bytes, i.e. the
// reference push order `for h, for group, for ch`.
__global__ void __launch_bounds__(1024) kivi_pack_k_kernel(const float* __restrict__ res_k, uint8_t* __restrict__ qk,
                                                           int hkv, int d, int res_cap, int n_groups, int bits,
                                                           long long k_block_start) {
    __shared__ float tile[32][33];
    const int ct = blockIdx.x, g = blockIdx.y, h = blockIdx.z;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    tile[w][lane] = res_k[((long long)h * res_cap + g * 32 + w) * d + ct * 32 + lane];   // token w, channel lane
    __syncthreads();
    const float x = tile[lane][w];                                                       // channel w, token lane
    const long long blk = k_block_start + ((long long)h * n_groups + g) * d + ct * 32 + w;
    pack_block_warp(x, bits, qk + blk * block_bytes_dev(bits));
}

// V: one warp per block of 32 channels of one token; order `for h, for tok, for blk`.
__global__ void __launch_bounds__(256) kivi_pack_v_kernel(const float* __restrict__ res_v, uint8_t* __restrict__ qv,
                                                          int hkv, int d, int res_cap, int flush_tokens, int bits,
                                                          long long v_block_start) {
    const int nb = d / 32;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long total = (long long)hkv * flush_tokens * nb;
    if (wid >= total) return;
    const int lane = threadIdx.x & 31;
    const int b = (int)(wid % nb);
    const long long tmp = wid / nb;
    const int t = (int)(tmp % flush_tokens), h = (int)(tmp / flush_tokens);
    const float x = res_v[((long long)h * res_cap + t) * d + b * 32 + lane];
    pack_block_warp(x, bits, qv + (v_block_start + wid) * block_bytes_dev(bits));
}

__device__ __forceinline__ float block_value(const uint8_t* blk, int bits, int i) {
    const float d = __half2float(reinterpret_cast<const __half*>(blk)[0]);
    const float m = __half2float(reinterpret_cast<const __half*>(blk)[1]);
    const uint32_t c = bits == 8 ? blk[4 + i] : bits == 4 ? ((blk[4 + (i >> 1)] >> ((i & 1) * 4)) & 0xF)
                                                          : ((blk[4 + (i >> 2)] >> ((i & 3) * 2)) & 0x3);
    return __fadd_rn(__fmul_rn((float)c, d), m);   // multiply, then add: two roundings like the CPU codec
}

// Unpack of one flush into the F16 SeqMajor view [max_seq][Hkv][D] (reference: Q2 only,
// kivi_dequantize_{key,value}_q2_f16; here any bit width). One thread per (block, element).
__global__ void __launch_bounds__(256) kivi_dequant_flush_kernel(const uint8_t* __restrict__ q, __half* __restrict__ attn,
                                                                 int hkv, int d, int n, int tok_base,
                                                                 long long block_start, int bits, int is_key) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n_blocks = is_key ? (long long)hkv * n * d : (long long)hkv * n * (d / 32);
    if (idx >= n_blocks * 32) return;
    const long long bid = idx >> 5;
    const int i = (int)(idx & 31);
    const float v = block_value(q + (block_start + bid) * block_bytes_dev(bits), bits, i);
    long long dst;
    if (is_key) {   // bid = (h*groups + g)*D + ch ; element i = token g*32+i
        const int ch = (int)(bid % d);
        const long long tmp = bid / d;
        const int g = (int)(tmp % n), h = (int)(tmp / n);
        dst = ((long long)(tok_base + g * 32 + i) * hkv + h) * d + ch;
    } else {        // bid = (h*tokens + t)*(D/32) + b ; element i = channel b*32+i
        const int nb = d / 32;
        const int b = (int)(bid % nb);
        const long long tmp = bid / nb;
        const int t = (int)(tmp % n), h = (int)(tmp / n);
        dst = ((long long)(tok_base + t) * hkv + h) * d + b * 32 + i;
    }
    attn[dst] = __float2half_rn(v);
}

// F32 ring rows [0,res_pos) -> F16 SeqMajor view rows tok_base.. (kivi_scatter_residual_f16).
__global__ void __launch_bounds__(256) kivi_scatter_residual_kernel(const float* __restrict__ res, __half* __restrict__ attn,
                                                                    int hkv, int res_cap, int d, int res_pos, int tok_base) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)hkv * res_pos * d) return;
    const int c = (int)(idx % d);
    const long long tmp = idx / d;
    const int t = (int)(tmp % res_pos), h = (int)(tmp / res_pos);
    attn[((long long)(tok_base + t) * hkv + h) * d + c] = __float2half_rn(res[((long long)h * res_cap + t) * d + c]);
}

// New rows [seq_len][Hkv][D] F32 -> ring rows res_pos.. of [Hkv][res_cap][D] (kivi_gather_update).
__global__ void __launch_bounds__(256) kivi_gather_update_kernel(const float* __restrict__ in, float* __restrict__ res,
                                                                 int hkv, int res_cap, int d, int seq_len, int res_pos) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)seq_len * hkv * d) return;
    const int c = (int)(idx % d);
    const long long tmp = idx / d;
    const int h = (int)(tmp % hkv), s = (int)(tmp / hkv);
    res[((long long)h * res_cap + res_pos + s) * d + c] = in[idx];
}

static inline unsigned blocks_for(long long n, int bs) { return (unsigned)((n + bs - 1) / bs); }

cudaError_t launch_kivi_pack(const float* res_k, const float* res_v, uint8_t* qk, uint8_t* qv, int hkv, int d,
                             int res_cap, int n_groups, int bits, long long k_block_start, long long v_block_start,
                             cudaStream_t st) {
    if (n_groups <= 0) return cudaSuccess;
    dim3 gk(d / 32, n_groups, hkv);
    kivi_pack_k_kernel<<<gk, 1024, 0, st>>>(res_k, qk, hkv, d, res_cap, n_groups, bits, k_block_start);
    const long long warps = (long long)hkv * n_groups * 32 * (d / 32);
    kivi_pack_v_kernel<<<blocks_for(warps, 8), 256, 0, st>>>(res_v, qv, hkv, d, res_cap, n_groups * 32, bits, v_block_start);
    return cudaGetLastError();
}

cudaError_t launch_kivi_dequant_flush(const uint8_t* q, __half* attn, int hkv, int d, int n, int tok_base,
                                      long long block_start, int bits, int is_key, cudaStream_t st) {
    const long long n_blocks = is_key ? (long long)hkv * n * d : (long long)hkv * n * (d / 32);
    if (n_blocks <= 0) return cudaSuccess;
    kivi_dequant_flush_kernel<<<blocks_for(n_blocks * 32, 256), 256, 0, st>>>(q, attn, hkv, d, n, tok_base, block_start,
                                                                            bits, is_key);
    return cudaGetLastError();
}

cudaError_t launch_kivi_scatter_residual(const float* res, __half* attn, int hkv, int res_cap, int d, int res_pos,
                                         int tok_base, cudaStream_t st) {
    const long long n = (long long)hkv * res_pos * d;
    if (n <= 0) return cudaSuccess;
    kivi_scatter_residual_kernel<<<blocks_for(n, 256), 256, 0, st>>>(res, attn, hkv, res_cap, d, res_pos, tok_base);
    return cudaGetLastError();
}

cudaError_t launch_kivi_gather_update(const float* in, float* res, int hkv, int res_cap, int d, int seq_len, int res_pos,
                                      cudaStream_t st) {
    const long long n = (long long)seq_len * hkv * d;
    if (n <= 0) return cudaSuccess;
    kivi_gather_update_kernel<<<blocks_for(n, 256), 256, 0, st>>>(in, res, hkv, res_cap, d, seq_len, res_pos);
    return cudaGetLastError();
}

}  // namespace argus
