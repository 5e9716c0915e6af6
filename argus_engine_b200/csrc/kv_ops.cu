// KV-cache write and eviction executors on a device-resident F16/F32 cache: the callers either side of the
// attention kernels. All three are byte movers bounded by HBM (16-byte vector accesses, one row = head_dim
// elements), and all are bit-exact with the reference's arithmetic.
//
//   kv_scatter        kv_scatter_f32_to_f16 / _batch / f32_to_f32_batch (engine/src/backend/cuda_pc/kernels.cu:305-360):
//                     new K/V rows [seq][Hkv][D] F32 -> cache rows write_pos.. (F16: round to nearest even)
//   kv_compact        KVCache::compact_keep_positions[_for_head] (engine/src/kv/kv_cache.rs:1266-1352):
//                     row write_start+i <- row keep[i], keep ascending
//   pfa_reduce        the accumulation half of prefill_attention_scores (engine/src/kv/standard_format.rs:1480-1508)
//   kv_weighted_merge apply_weighted_merges, F32/F16 arms (engine/src/kv/standard_format.rs:754-893):
//                     into <- into_w*into + sum_j w_j*from_j, every product and sum rounded on its own, list order
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace argus {

// ───────── KV write ─────────
template <bool DST_F16>
__global__ void __launch_bounds__(256) kv_scatter_kernel(const float* __restrict__ k_src, const float* __restrict__ v_src,
                                                         void* __restrict__ k_dst, void* __restrict__ v_dst, int hkv, int d,
                                                         long long head_stride, long long pos_stride, long long write_pos,
                                                         long long seq_len) {
    // CTA = one source row block [Hkv][D] (position s); thread = (head, four channels)
    const int vec_per_row = d / 4;
    const long long s = blockIdx.x;
    if (s >= seq_len) return;
    for (int t = threadIdx.x; t < hkv * vec_per_row; t += blockDim.x) {
        const int h = t / vec_per_row, c = (t - h * vec_per_row) * 4;
        const long long so = (s * hkv + h) * d + c;
        const long long dof = h * head_stride + (write_pos + s) * pos_stride + c;
        const float4 kx = *reinterpret_cast<const float4*>(k_src + so);
        const float4 vx = *reinterpret_cast<const float4*>(v_src + so);
        if constexpr (DST_F16) {
            __half2 ka = __floats2half2_rn(kx.x, kx.y), kb = __floats2half2_rn(kx.z, kx.w);
            __half2 va = __floats2half2_rn(vx.x, vx.y), vb = __floats2half2_rn(vx.z, vx.w);
            *reinterpret_cast<uint2*>(static_cast<__half*>(k_dst) + dof) =
                make_uint2(*reinterpret_cast<uint32_t*>(&ka), *reinterpret_cast<uint32_t*>(&kb));
            *reinterpret_cast<uint2*>(static_cast<__half*>(v_dst) + dof) =
                make_uint2(*reinterpret_cast<uint32_t*>(&va), *reinterpret_cast<uint32_t*>(&vb));
        } else {
            *reinterpret_cast<float4*>(static_cast<float*>(k_dst) + dof) = kx;
            *reinterpret_cast<float4*>(static_cast<float*>(v_dst) + dof) = vx;
        }
    }
}

cudaError_t launch_kv_scatter(const float* k_src, const float* v_src, void* k_dst, void* v_dst, bool dst_f16, int hkv,
                              int d, long long head_stride, long long pos_stride, long long write_pos, long long seq_len,
                              cudaStream_t st) {
    if (seq_len <= 0 || hkv <= 0 || d < 4) return cudaSuccess;
    if (seq_len > 0x7fffffffLL) return cudaErrorInvalidValue;
    const unsigned grid = (unsigned)seq_len;
    if (dst_f16)
        kv_scatter_kernel<true><<<grid, 256, 0, st>>>(k_src, v_src, k_dst, v_dst, hkv, d, head_stride, pos_stride, write_pos, seq_len);
    else
        kv_scatter_kernel<false><<<grid, 256, 0, st>>>(k_src, v_src, k_dst, v_dst, hkv, d, head_stride, pos_stride, write_pos, seq_len);
    return cudaGetLastError();
}

// One new row for each of n sequences in ONE launch (a batched decode step): sequence b's row [Hkv][D] goes to
// position write_pos[b] of its own cache. The descriptor table travels as a kernel parameter.
struct KvRowBatch {
    void* k[64];
    void* v[64];
    long long head_stride[64];
    long long pos_stride[64];
    long long write_pos[64];
};
template <bool DST_F16>
__global__ void __launch_bounds__(256) kv_scatter_rows_kernel(const float* __restrict__ k_src, const float* __restrict__ v_src,
                                                              const __grid_constant__ KvRowBatch bt, int n, int hkv, int d) {
    const int vec_per_row = d / 4;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * hkv * vec_per_row) return;
    const int c = (idx % vec_per_row) * 4;
    const int h = (idx / vec_per_row) % hkv, b = idx / (vec_per_row * hkv);
    const long long so = ((long long)b * hkv + h) * d + c;
    const long long dof = h * bt.head_stride[b] + bt.write_pos[b] * bt.pos_stride[b] + c;
    const float4 kx = *reinterpret_cast<const float4*>(k_src + so);
    const float4 vx = *reinterpret_cast<const float4*>(v_src + so);
    if constexpr (DST_F16) {
        __half2 ka = __floats2half2_rn(kx.x, kx.y), kb = __floats2half2_rn(kx.z, kx.w);
        __half2 va = __floats2half2_rn(vx.x, vx.y), vb = __floats2half2_rn(vx.z, vx.w);
        *reinterpret_cast<uint2*>(static_cast<__half*>(bt.k[b]) + dof) =
            make_uint2(*reinterpret_cast<uint32_t*>(&ka), *reinterpret_cast<uint32_t*>(&kb));
        *reinterpret_cast<uint2*>(static_cast<__half*>(bt.v[b]) + dof) =
            make_uint2(*reinterpret_cast<uint32_t*>(&va), *reinterpret_cast<uint32_t*>(&vb));
    } else {
        *reinterpret_cast<float4*>(static_cast<float*>(bt.k[b]) + dof) = kx;
        *reinterpret_cast<float4*>(static_cast<float*>(bt.v[b]) + dof) = vx;
    }
}

cudaError_t launch_kv_scatter_rows(const float* k_src, const float* v_src, void* const* k_dst, void* const* v_dst,
                                   const long long* head_stride, const long long* pos_stride, const long long* write_pos,
                                   int n, bool dst_f16, int hkv, int d, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    KvRowBatch bt;
    for (int i = 0; i < n; ++i) {
        bt.k[i] = k_dst[i];
        bt.v[i] = v_dst[i];
        bt.head_stride[i] = head_stride[i];
        bt.pos_stride[i] = pos_stride[i];
        bt.write_pos[i] = write_pos[i];
    }
    const int total = n * hkv * (d / 4);
    if (dst_f16) kv_scatter_rows_kernel<true><<<(total + 255) / 256, 256, 0, st>>>(k_src, v_src, bt, n, hkv, d);
    else kv_scatter_rows_kernel<false><<<(total + 255) / 256, 256, 0, st>>>(k_src, v_src, bt, n, hkv, d);
    return cudaGetLastError();
}

// ───────── prefix snapshot payload: strided cache rows <-> packed [Hkv][token_count][D] bytes ─────────
// to_packed = 1: packed[(h*n_tok + t)*row_vecs + v] = cache[h*head_stride + t*pos_stride + v]; 0: the other way round.
// Used where the rows of a head are not contiguous in the cache (SeqMajor); the HeadMajor case is a pitched copy.
__global__ void __launch_bounds__(256) kv_prefix_rows_kernel(uint4* __restrict__ cache, uint4* __restrict__ packed,
                                                             long long n_tok, int hkv, int row_vecs,
                                                             long long head_stride_v, long long pos_stride_v, int to_packed) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tok * hkv * row_vecs) return;
    const int v = (int)(idx % row_vecs);
    const long long t = (idx / row_vecs) % n_tok;
    const int h = (int)(idx / (row_vecs * n_tok));
    uint4* c = cache + h * head_stride_v + t * pos_stride_v + v;
    if (to_packed) packed[idx] = *c;
    else *c = packed[idx];
}

cudaError_t launch_kv_prefix_rows(void* cache, void* packed, long long n_tok, int hkv, int row_bytes,
                                  long long head_stride_bytes, long long pos_stride_bytes, int to_packed, cudaStream_t st) {
    const long long total = n_tok * hkv * (row_bytes / 16);
    if (total <= 0) return cudaSuccess;
    kv_prefix_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(static_cast<uint4*>(cache), static_cast<uint4*>(packed),
                                                                         n_tok, hkv, row_bytes / 16, head_stride_bytes / 16,
                                                                         pos_stride_bytes / 16, to_packed);
    return cudaGetLastError();
}

// ───────── keep-set compaction ─────────
// The move is in place and to the left (keep[i] >= write_start + i), and the distance keep[i] - (write_start + i)
// never shrinks along an ascending list. Rows are moved chunk after chunk in ascending order, so that a later
// chunk's sources lie to the right of everything written before. Inside a chunk [i0, i0 + n):
//   * if its first row moves by at least n positions, every source of the chunk lies right of every destination of
//     the chunk: the first launch copies the rows directly and the second one returns at once;
//   * otherwise a destination may be another row's source: the first launch gathers the rows into scratch, the
//     second writes them (all reads precede all writes).
// Rows already in place are skipped. An entry that is not above its predecessor or that would move a row to the
// right, or that lies at or beyond `capacity`, is skipped and sets *status = 2; the contents of the cache are then unspecified.
// first = 1: direct copy or cache -> scratch; 0: scratch -> cache. Scratch layout [heads][rows of the chunk][row_vecs].
__global__ void __launch_bounds__(256) kv_compact_kernel(uint4* __restrict__ cache, uint4* __restrict__ scratch,
                                                         const int* __restrict__ keep, long long i0, long long n_rows,
                                                         long long write_start, int head0, int n_heads, int row_vecs,
                                                         long long head_stride_v, long long pos_stride_v, int first,
                                                         long long capacity, int* status) {
    const bool direct = (long long)keep[i0] - (write_start + i0) >= n_rows;   // the same answer in every thread
    if (direct && !first) return;
    // blockIdx.y = head of the pass; a chunk has at most 32768 rows, so 32-bit index arithmetic is enough
    const unsigned t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (unsigned)n_rows * (unsigned)row_vecs) return;
    const unsigned r = t / (unsigned)row_vecs;
    const int v = (int)(t - r * (unsigned)row_vecs);
    const int hh = (int)blockIdx.y;
    const long long i = i0 + r;
    const long long src = keep[i], dst = write_start + i;
    if (src == dst) return;
    if (src < dst || src >= capacity || (i > 0 && keep[i - 1] >= src)) {   // the reference's slice index would panic
        if (status != nullptr && v == 0 && hh == 0) atomicExch(status, 2);
        return;
    }
    const long long base = (long long)(head0 + hh) * head_stride_v;
    uint4* s = scratch + ((long long)hh * n_rows + r) * row_vecs + v;
    if (direct) cache[base + dst * pos_stride_v + v] = cache[base + src * pos_stride_v + v];
    else if (first) *s = cache[base + src * pos_stride_v + v];
    else cache[base + dst * pos_stride_v + v] = *s;
}

cudaError_t launch_kv_compact_pass(void* cache, void* scratch, const int* keep, long long i0, long long n_rows,
                                   long long write_start, int head0, int n_heads, int row_bytes, long long head_stride_bytes,
                                   long long pos_stride_bytes, int first, long long capacity, int* status,
                                   cudaStream_t st) {
    const int row_vecs = row_bytes / 16;
    const long long per_head = n_rows * row_vecs;
    if (per_head <= 0 || n_heads <= 0) return cudaSuccess;
    if (per_head > 0x7fffffffLL || n_heads > 65535) return cudaErrorInvalidValue;
    kv_compact_kernel<<<dim3((unsigned)((per_head + 255) / 256), (unsigned)n_heads), 256, 0, st>>>(
        static_cast<uint4*>(cache), static_cast<uint4*>(scratch), keep, i0, n_rows, write_start, head0, n_heads, row_vecs,
        head_stride_bytes / 16, pos_stride_bytes / 16, first, capacity, status);
    return cudaGetLastError();
}

// ───────── prefill attention scores: accumulate the per-row probabilities ─────────
// rows [n_rows][Hq][prefix_len] are the probabilities of n_rows consecutive query rows; row r sits at absolute position
// p = row0_pos + r and sees keys lo..=p (lo = 0, or max(0, p - (window-1)) with a sliding window). Only those entries are
// read - the reference adds keys lo..=p and nothing else - so whatever a reused or uninitialised per-row buffer holds
// outside a row's range never reaches the sums. sum_out[h][t] += sum over rows in ascending row order;
// mean_out[row][t] += rows[row][h][t] * (1/Hq) in ascending head order: the reference's loop orders, element by element.
__global__ void __launch_bounds__(256) pfa_reduce_kernel(const float* __restrict__ rows, float* __restrict__ sum_out,
                                                         float* __restrict__ mean_out, int n_rows, int hq,
                                                         long long prefix_len, float inv_heads, long long row0_pos,
                                                         int window) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n_sum = sum_out ? (long long)hq * prefix_len : 0;
    if (idx < n_sum) {
        const long long t = idx % prefix_len;
        float acc = sum_out[idx];
        for (int r = 0; r < n_rows; ++r) {
            const long long p = row0_pos + r, lo = window > 0 ? max(0LL, p - (window - 1)) : 0LL;
            if (t >= lo && t <= p) acc = __fadd_rn(acc, rows[(long long)r * hq * prefix_len + idx]);
        }
        sum_out[idx] = acc;
        return;
    }
    const long long j = idx - n_sum;
    if (mean_out == nullptr || j >= (long long)n_rows * prefix_len) return;
    const long long r = j / prefix_len, t = j % prefix_len;
    const long long p = row0_pos + r, lo = window > 0 ? max(0LL, p - (window - 1)) : 0LL;
    if (t < lo || t > p) return;
    float acc = mean_out[j];
    for (int h = 0; h < hq; ++h) acc = __fadd_rn(acc, __fmul_rn(rows[(r * hq + h) * prefix_len + t], inv_heads));
    mean_out[j] = acc;
}

cudaError_t launch_pfa_reduce(const float* rows, float* sum_out, float* mean_out, int n_rows, int hq, long long prefix_len,
                              long long row0_pos, int window, cudaStream_t st) {
    const long long total = (sum_out ? (long long)hq * prefix_len : 0) + (mean_out ? (long long)n_rows * prefix_len : 0);
    if (total <= 0 || n_rows <= 0) return cudaSuccess;
    pfa_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(rows, sum_out, mean_out, n_rows, hq, prefix_len,
                                                                       1.0f / (float)hq, row0_pos, window);
    return cudaGetLastError();
}

// ───────── weighted merge (D2O) ─────────
// Merges are disjoint (a `from` row is evicted, an `into` row is retained, neither occurs twice), so they run in
// parallel: CTA = (merge, kv head), thread = channel. from_start is a CSR offset array [n_merges + 1].
template <typename T>
__device__ __forceinline__ float load_f32(const T* p);
template <>
__device__ __forceinline__ float load_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_f32<__half>(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void store_f32(float* p, float x) { *p = x; }
__device__ __forceinline__ void store_f32(__half* p, float x) { *p = __float2half_rn(x); }

template <typename T>
__global__ void __launch_bounds__(128) kv_weighted_merge_kernel(T* __restrict__ k, T* __restrict__ v, int d,
                                                                long long head_stride, long long pos_stride,
                                                                const int* __restrict__ into_pos,
                                                                const float* __restrict__ into_w,
                                                                const int* __restrict__ from_start,
                                                                const int* __restrict__ from_pos,
                                                                const float* __restrict__ from_w, int do_k, int do_v) {
    const int m = blockIdx.x, h = blockIdx.y;
    const int f0 = from_start[m], f1 = from_start[m + 1];
    if (f1 <= f0) return;   // an empty `from` list leaves the row untouched
    const long long base = (long long)h * head_stride;
    const long long io = base + (long long)into_pos[m] * pos_stride;
    const float iw = into_w[m];
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        if (do_k) {
            float acc = __fmul_rn(iw, load_f32(k + io + c));
            for (int j = f0; j < f1; ++j)
                acc = __fadd_rn(acc, __fmul_rn(from_w[j], load_f32(k + base + (long long)from_pos[j] * pos_stride + c)));
            store_f32(k + io + c, acc);
        }
        if (do_v) {
            float acc = __fmul_rn(iw, load_f32(v + io + c));
            for (int j = f0; j < f1; ++j)
                acc = __fadd_rn(acc, __fmul_rn(from_w[j], load_f32(v + base + (long long)from_pos[j] * pos_stride + c)));
            store_f32(v + io + c, acc);
        }
    }
}

// The same merge with four channels per thread and all KV heads of a merge in one CTA (thread = (head, 4 channels)):
// the list of a merge is read once per CTA and rows move as 8- or 16-byte vectors. Per element the products and
// sums are the ones above, in the same order. Needs d, the strides and the base addresses to be multiples of 4
// elements.
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
    __device__ __forceinline__ void get(float (&x)[4]) const { x[0] = raw.x; x[1] = raw.y; x[2] = raw.z; x[3] = raw.w; }
    __device__ __forceinline__ void set(const float (&x)[4]) { raw = make_float4(x[0], x[1], x[2], x[3]); }
};
template <>
struct Vec4<__half> {
    uint2 raw;
    __device__ __forceinline__ void load(const __half* p) { raw = *reinterpret_cast<const uint2*>(p); }
    __device__ __forceinline__ void store(__half* p) const { *reinterpret_cast<uint2*>(p) = raw; }
    __device__ __forceinline__ void get(float (&x)[4]) const {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    }
    __device__ __forceinline__ void set(const float (&x)[4]) {
        const __half2 a = __halves2half2(__float2half_rn(x[0]), __float2half_rn(x[1]));
        const __half2 b = __halves2half2(__float2half_rn(x[2]), __float2half_rn(x[3]));
        raw.x = *reinterpret_cast<const uint32_t*>(&a);
        raw.y = *reinterpret_cast<const uint32_t*>(&b);
    }
};

template <typename T>
__global__ void __launch_bounds__(256) kv_weighted_merge_vec_kernel(T* __restrict__ k, T* __restrict__ v, int d, int hkv,
                                                                    long long head_stride, long long pos_stride,
                                                                    const int* __restrict__ into_pos,
                                                                    const float* __restrict__ into_w,
                                                                    const int* __restrict__ from_start,
                                                                    const int* __restrict__ from_pos,
                                                                    const float* __restrict__ from_w, int do_k, int do_v) {
    const int m = blockIdx.x;
    const int f0 = from_start[m], f1 = from_start[m + 1];
    if (f1 <= f0) return;   // an empty `from` list leaves the row untouched
    const long long ipos = into_pos[m];
    const float iw = into_w[m];
    const int vecs = d >> 2;
    for (int t = threadIdx.x; t < hkv * vecs; t += blockDim.x) {
        const int h = t / vecs, c = (t - h * vecs) << 2;
        const long long base = (long long)h * head_stride + c;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            if (which == 0 ? !do_k : !do_v) continue;
            T* buf = which == 0 ? k : v;
            Vec4<T> x;
            float acc[4], val[4];
            x.load(buf + base + ipos * pos_stride);
            x.get(val);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = __fmul_rn(iw, val[e]);
            for (int j = f0; j < f1; ++j) {
                const float w = from_w[j];
                x.load(buf + base + (long long)from_pos[j] * pos_stride);
                x.get(val);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] = __fadd_rn(acc[e], __fmul_rn(w, val[e]));
            }
            x.set(acc);
            x.store(buf + base + ipos * pos_stride);
        }
    }
}

cudaError_t launch_kv_weighted_merge(void* k, void* v, bool f16, int hkv, int d, long long head_stride,
                                     long long pos_stride, const int* into_pos, const float* into_w, const int* from_start,
                                     const int* from_pos, const float* from_w, int n_merges, int do_k, int do_v,
                                     cudaStream_t st) {
    if (n_merges <= 0) return cudaSuccess;
    const size_t vec_bytes = f16 ? 8 : 16;
    const bool vec_ok = (d % 4 == 0) && (head_stride % 4 == 0) && (pos_stride % 4 == 0) &&
                        (!do_k || reinterpret_cast<uintptr_t>(k) % vec_bytes == 0) &&
                        (!do_v || reinterpret_cast<uintptr_t>(v) % vec_bytes == 0);
    if (vec_ok) {
        if (f16)
            kv_weighted_merge_vec_kernel<__half><<<(unsigned)n_merges, 256, 0, st>>>(
                static_cast<__half*>(k), static_cast<__half*>(v), d, hkv, head_stride, pos_stride, into_pos, into_w, from_start,
                from_pos, from_w, do_k, do_v);
        else
            kv_weighted_merge_vec_kernel<float><<<(unsigned)n_merges, 256, 0, st>>>(
                static_cast<float*>(k), static_cast<float*>(v), d, hkv, head_stride, pos_stride, into_pos, into_w, from_start,
                from_pos, from_w, do_k, do_v);
        return cudaGetLastError();
    }
    const dim3 grid((unsigned)n_merges, (unsigned)hkv);
    if (f16)
        kv_weighted_merge_kernel<__half><<<grid, 128, 0, st>>>(static_cast<__half*>(k), static_cast<__half*>(v), d,
                                                              head_stride, pos_stride, into_pos, into_w, from_start,
                                                              from_pos, from_w, do_k, do_v);
    else
        kv_weighted_merge_kernel<float><<<grid, 128, 0, st>>>(static_cast<float*>(k), static_cast<float*>(v), d,
                                                             head_stride, pos_stride, into_pos, into_w, from_start,
                                                             from_pos, from_w, do_k, do_v);
    return cudaGetLastError();
}

}  // namespace argus

namespace argus {

// ───────── D2O nearest retained token (Eq. 8) ─────────
// find_nearest_layer_wide_via + cosine_similarity (crates/techniques/d2o/src/lib.rs:187-255): for every evicted
// position, the retained position whose head-concatenated K row has the largest cosine similarity, the first one in
// list order on ties, never the evicted position itself. The reference accumulates dot and the two squared norms
// over the Hkv*D channels in order, one rounding per product and per sum; the kernels below do exactly that (so the
// similarities and therefore the selected indices are bit-identical): the norms once per listed row, the dot
// products in 64 x 64 tiles of (evicted, retained) pairs, 4 x 4 pairs per thread, channels in ascending order.
template <typename T>
__global__ void __launch_bounds__(128) d2o_norms_kernel(const T* __restrict__ k, long long head_stride, long long pos_stride,
                                                        int hkv, int d, const int* __restrict__ evict, int n_evict,
                                                        const int* __restrict__ retain, int n_retain,
                                                        float* __restrict__ norms) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_evict + n_retain) return;
    const long long pos = i < n_evict ? evict[i] : retain[i - n_evict];
    float acc = 0.f;
    for (int h = 0; h < hkv; ++h) {
        const T* row = k + h * head_stride + pos * pos_stride;
        for (int c = 0; c < d; ++c) {
            const float x = load_f32(row + c);
            acc = __fadd_rn(acc, __fmul_rn(x, x));
        }
    }
    norms[i] = acc;
}

__device__ __forceinline__ unsigned long long d2o_key(float sim, int list_index) {
    sim = sim + 0.0f;   // -0 -> +0: the reference's `>` does not tell them apart
    const uint32_t u = __float_as_uint(sim);
    const uint32_t ord = u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u);
    return ((unsigned long long)ord << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)list_index);
}

template <typename T>
__global__ void __launch_bounds__(256) d2o_pairs_kernel(const T* __restrict__ k, long long head_stride, long long pos_stride,
                                                        int hkv, int d, const int* __restrict__ evict, int n_evict,
                                                        const int* __restrict__ retain, int n_retain,
                                                        const float* __restrict__ norms, unsigned long long* __restrict__ best) {
    // 64 x 64 pairs per CTA, 4 x 4 per thread; a 32-channel chunk of the 128 rows sits in shared memory channel-major,
    // so a thread fetches its four rows of either side with one 16-byte load per channel.
    constexpr int TP = 64, LD = TP + 4;
    __shared__ __align__(16) float sa[32][LD], sb[32][LD];
    __shared__ int pa[TP], pb[TP];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int e0 = blockIdx.y * TP, r0 = blockIdx.x * TP;
    if (threadIdx.x < TP) pa[threadIdx.x] = e0 + threadIdx.x < n_evict ? evict[e0 + threadIdx.x] : -1;
    else if (threadIdx.x < 2 * TP) pb[threadIdx.x - TP] = r0 + threadIdx.x - TP < n_retain ? retain[r0 + threadIdx.x - TP] : -1;
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int dim = hkv * d;
    for (int g0 = 0; g0 < dim; g0 += 32) {
        // 128 rows x 32 channels of this chunk -> shared memory as F32 (d is a multiple of 32: a chunk stays in one head)
        const int h = g0 / d, c0 = g0 % d;
        for (int e = threadIdx.x; e < 2 * TP * 32; e += 256) {
            const int r = e >> 5, c = e & 31;
            const int pos = r < TP ? pa[r] : pb[r - TP];
            const float x = pos >= 0 ? load_f32(k + h * head_stride + (long long)pos * pos_stride + c0 + c) : 0.f;
            if (r < TP) sa[c][r] = x;
            else sb[c][r - TP] = x;
        }
        __syncthreads();
#pragma unroll 4
        for (int c = 0; c < 32; ++c) {
            const float4 a4 = *reinterpret_cast<const float4*>(&sa[c][4 * ty]);
            const float4 b4 = *reinterpret_cast<const float4*>(&sb[c][4 * tx]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int ei = e0 + 4 * ty + i;
        unsigned long long key = 0;   // 0 = no candidate
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ri = r0 + 4 * tx + j;
            if (ei < n_evict && ri < n_retain && pb[4 * tx + j] != pa[4 * ty + i]) {
                const float denom = __fsqrt_rn(__fmul_rn(norms[ei], norms[n_evict + ri]));
                const float sim = denom < 1e-10f ? 0.f : __fdiv_rn(acc[i][j], denom);
                if (sim == sim && sim != -INFINITY) {   // NaN and -inf never beat the reference's initial -inf
                    const unsigned long long kk = d2o_key(sim, ri);
                    key = kk > key ? kk : key;
                }
            }
        }
        // the 16 threads with this ty share the evicted rows: reduce over tx, one atomic per row and block
#pragma unroll
        for (int sh = 8; sh > 0; sh >>= 1) {
            const unsigned long long o = __shfl_xor_sync(0xffffffffu, key, sh);
            key = o > key ? o : key;
        }
        if (tx == 0 && key != 0 && ei < n_evict) atomicMax(best + ei, key);
    }
}

__global__ void __launch_bounds__(256) d2o_finalize_kernel(const unsigned long long* __restrict__ best,
                                                           const int* __restrict__ evict, int n_evict,
                                                           const int* __restrict__ retain, int n_retain,
                                                           int* __restrict__ nearest, float* __restrict__ sim_out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_evict) return;
    const unsigned long long key = best[i];
    if (key == 0) {   // no valid target: the first retained position (or the evicted one), similarity 0
        nearest[i] = n_retain > 0 ? retain[0] : evict[i];
        sim_out[i] = 0.f;
        return;
    }
    const uint32_t ord = (uint32_t)(key >> 32);
    nearest[i] = retain[0xFFFFFFFFu - (uint32_t)key];
    sim_out[i] = __uint_as_float(ord ^ ((ord >> 31) ? 0x80000000u : 0xFFFFFFFFu));
}

cudaError_t launch_d2o_nearest(const void* k, bool f16, long long head_stride, long long pos_stride, int hkv, int d,
                               const int* evict, int n_evict, const int* retain, int n_retain, float* norms,
                               unsigned long long* best, int* nearest, float* sim_out, cudaStream_t st) {
    if (n_evict <= 0) return cudaSuccess;
    cudaError_t e = cudaMemsetAsync(best, 0, (size_t)n_evict * sizeof(unsigned long long), st);
    if (e != cudaSuccess) return e;
    const int rows = n_evict + n_retain;
    const dim3 grid((unsigned)((n_retain + 63) / 64), (unsigned)((n_evict + 63) / 64));
    if (f16) {
        d2o_norms_kernel<__half><<<(rows + 127) / 128, 128, 0, st>>>(static_cast<const __half*>(k), head_stride, pos_stride, hkv,
                                                                     d, evict, n_evict, retain, n_retain, norms);
        if (n_retain > 0)
            d2o_pairs_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(k), head_stride, pos_stride, hkv, d, evict,
                                                            n_evict, retain, n_retain, norms, best);
    } else {
        d2o_norms_kernel<float><<<(rows + 127) / 128, 128, 0, st>>>(static_cast<const float*>(k), head_stride, pos_stride, hkv, d,
                                                                    evict, n_evict, retain, n_retain, norms);
        if (n_retain > 0)
            d2o_pairs_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(k), head_stride, pos_stride, hkv, d, evict,
                                                           n_evict, retain, n_retain, norms, best);
    }
    d2o_finalize_kernel<<<(n_evict + 255) / 256, 256, 0, st>>>(best, evict, n_evict, retain, n_retain, nearest, sim_out);
    return cudaGetLastError();
}

}  // namespace argus
