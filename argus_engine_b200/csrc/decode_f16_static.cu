// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: code that runs inside a CUDA-graph capture or
// a latency-critical serving loop where an allocation would synchronise the device, and embedders whose
// memory is handed out once by their own pool (the engine's `panic = "abort"` build treats a failed
// allocation in the middle of a token as fatal). argus_b200_attention_gen_static is the F16 split-KV decode
// kernel with its scratch (split partials, per-head log-sum-exp, arrival tickets) placed in a fixed array
// that lives in the library image instead of in a context-owned allocation. No context object is needed.
//
// The array is one per device that loads the library and is held until the process exits. Every call on a
// device shares it and finds the previous call's bytes in it, so the ticket words are cleared on the
// caller's stream at the start of each call, and two calls whose kernels can overlap on the GPU (different
// streams, or different host threads) race on it: serialise them. Problems whose plan needs more than the
// array holds are rejected with ARGUS_B200_E_WORKSPACE; nothing is ever allocated as a fallback.
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "context.h"

namespace argus {

constexpr size_t kStaticScratchBytes = size_t(4) << 20;   // 4 MiB per device
constexpr int kStaticTickets = 256;                        // one per KV head

// Host code must never pass this name to a kernel: on the host it is only a stand-in for the symbol.
// The device address is looked up once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticDeviceState {
    bool ready = false;
    unsigned char* base = nullptr;   // device address of g_static_scratch on this device
    int num_sms = 0;
};
static StaticDeviceState g_dev[kMaxDevices];
static std::mutex g_dev_mutex;
static thread_local char g_static_err[256] = {0};

static int static_fail(int code, const char* msg) {
    snprintf(g_static_err, sizeof(g_static_err), "%s", msg);
    return code;
}

// First call on a device: resolve the array's device address and read the SM count. Runs with that device
// current. Not capturable work (symbol lookup, attribute queries), hence "first call before any capture".
static int static_setup(int device, StaticDeviceState** out) {
    if (device < 0 || device >= kMaxDevices) return static_fail(ARGUS_B200_E_INVALID, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    StaticDeviceState& s = g_dev[device];
    if (!s.ready) {
        int major = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e != cudaSuccess) return static_fail(ARGUS_B200_E_CUDA, cudaGetErrorString(e));
        if (major != 10) return static_fail(ARGUS_B200_E_UNSUPPORTED, "not an sm_100 device");
        e = cudaDeviceGetAttribute(&s.num_sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return static_fail(ARGUS_B200_E_CUDA, cudaGetErrorString(e));
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return static_fail(ARGUS_B200_E_CUDA, e != cudaSuccess ? cudaGetErrorString(e) : "null symbol address");
        s.base = static_cast<unsigned char*>(ptr);
        s.ready = true;
    }
    *out = &s;
    return ARGUS_B200_OK;
}

}  // namespace argus

extern "C" {

size_t argus_b200_static_scratch_bytes(void) { return argus::kStaticScratchBytes; }
const char* argus_b200_static_last_error(void) { return argus::g_static_err; }

int argus_b200_attention_gen_static(void* stream, const float* q, const void* k_cache, const void* v_cache, float* out,
                                    float* lse, int num_heads_q, int num_heads_kv, int head_dim, int64_t cache_seq_len,
                                    int kv_dtype, int64_t head_stride, int64_t pos_stride) {
    using namespace argus;
    g_static_err[0] = 0;
    if (!q || !out || num_heads_q <= 0 || num_heads_kv <= 0 || num_heads_q % num_heads_kv != 0 || cache_seq_len < 0 ||
        cache_seq_len > 0x7fffffff - 4096)
        return static_fail(ARGUS_B200_E_INVALID, "null pointer, bad head counts or bad length");
    const int g = num_heads_q / num_heads_kv;
    if (kv_dtype != ARGUS_B200_KV_F16 || (head_dim != 64 && head_dim != 128) || g > kMaxGroup)
        return static_fail(ARGUS_B200_E_UNSUPPORTED, "unsupported kv dtype, head_dim or group size");
    if (cache_seq_len > 0 &&
        (!k_cache || !v_cache || (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15) ||
         (head_stride & 7) || (pos_stride & 7) || pos_stride < head_dim))
        return static_fail(ARGUS_B200_E_INVALID, "K/V must be 16-byte aligned with strides that are multiples of 8 elements");
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return static_fail(ARGUS_B200_E_INVALID, "q/out must be 16-byte aligned");
    if (num_heads_kv > kStaticTickets) return static_fail(ARGUS_B200_E_WORKSPACE, "more KV heads than ticket slots (256)");

    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_fail(ARGUS_B200_E_CUDA, cudaGetErrorString(e));
    StaticDeviceState* dev = nullptr;
    int rc = static_setup(device, &dev);
    if (rc != ARGUS_B200_OK) return rc;

    DecodeBatch bt;
    memset(&bt, 0, sizeof(bt));
    bt.k[0] = k_cache;
    bt.v[0] = v_cache;
    bt.head_stride[0] = head_stride;
    bt.pos_stride[0] = pos_stride;
    bt.seq_len[0] = (int32_t)cache_seq_len;
    int32_t nsplit = 1;
    const int64_t len = cache_seq_len;
    plan_splits(&len, 1, num_heads_kv, dev->num_sms * 2, 1, 2 * decode_f16_cta_tokens(head_dim), bt.chunk, &nsplit);
    bt.item_start[0] = 0;
    bt.item_start[1] = nsplit;

    // carve the fixed array: [tickets | lse2 | (m,l) partials | O partials]
    auto align256 = [](size_t x) { return (x + 255) & ~size_t(255); };
    const size_t off_lse2 = align256(kStaticTickets * sizeof(int));
    const size_t off_ml = align256(off_lse2 + (size_t)num_heads_q * sizeof(float));
    const size_t off_o = align256(off_ml + (size_t)nsplit * num_heads_kv * 8 * sizeof(float2));
    const size_t need = off_o + (size_t)nsplit * num_heads_kv * 8 * head_dim * sizeof(float);
    if (need > kStaticScratchBytes) {
        snprintf(g_static_err, sizeof(g_static_err),
                 "this call needs %zu bytes of scratch, the fixed array holds %zu", need, kStaticScratchBytes);
        return ARGUS_B200_E_WORKSPACE;
    }

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the last call (finished or not) left in it; the tickets must start at zero.
    e = cudaMemsetAsync(dev->base, 0, kStaticTickets * sizeof(int), st);
    if (e != cudaSuccess) return static_fail(ARGUS_B200_E_CUDA, cudaGetErrorString(e));

    DecodeParams p;
    memset(&p, 0, sizeof(p));
    p.q = q;
    p.out = out;
    p.lse = lse;
    p.n_seqs = 1;
    p.hq = num_heads_q;
    p.hkv = num_heads_kv;
    p.group = g;
    p.scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    p.tickets = reinterpret_cast<int*>(dev->base);
    p.lse2 = reinterpret_cast<float*>(dev->base + off_lse2);
    p.part_ml = reinterpret_cast<float2*>(dev->base + off_ml);
    p.part_o = reinterpret_cast<float*>(dev->base + off_o);
    e = launch_decode_f16(p, bt, head_dim, nsplit, st);
    if (e != cudaSuccess) return static_fail(ARGUS_B200_E_CUDA, cudaGetErrorString(e));
    return ARGUS_B200_OK;
}

}  // extern "C"
