// F32 K/V cache -> packed F16 HeadMajor copy [Hkv][T][D] in scratch, for Backend::attention_gen calls whose
// cache dtype is F32 (engine/src/backend.rs:305-313 accepts both; the engine's default is F16). The decode
// kernel then runs on the copy. Values are rounded to nearest even like half::f16::from_f32.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace argus {

// Block = (d/4 threads along a row) x (rows); blockIdx.y = KV head: no index division.
__global__ void __launch_bounds__(256) kv_f32_to_f16_kernel(const float* __restrict__ src, __half* __restrict__ dst,
                                                            long long T, int d, long long head_stride,
                                                            long long pos_stride) {
    const long long t = (long long)blockIdx.x * blockDim.y + threadIdx.y;
    if (t >= T) return;
    const int c = threadIdx.x * 4;   // 4 channels per thread
    const long long h = blockIdx.y;
    const float4 v = *reinterpret_cast<const float4*>(src + h * head_stride + t * pos_stride + c);
    __half2* o = reinterpret_cast<__half2*>(dst + (h * T + t) * d + c);
    o[0] = __floats2half2_rn(v.x, v.y);
    o[1] = __floats2half2_rn(v.z, v.w);
}

cudaError_t launch_kv_f32_to_f16(const float* src, void* dst, int hkv, long long T, int d, long long head_stride,
                                 long long pos_stride, cudaStream_t st) {
    if (hkv <= 0 || T <= 0 || d <= 0) return cudaSuccess;
    const int vpr = d / 4;
    if (d % 4 != 0 || vpr > 256 || hkv > 65535) return cudaErrorInvalidValue;
    const int rows = 256 / vpr;
    const long long blocks = (T + rows - 1) / rows;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    kv_f32_to_f16_kernel<<<dim3((unsigned)blocks, (unsigned)hkv), dim3((unsigned)vpr, (unsigned)rows), 0, st>>>(
        src, static_cast<__half*>(dst), T, d, head_stride, pos_stride);
    return cudaGetLastError();
}

}  // namespace argus
