// F32 K/V cache -> packed F16 HeadMajor copy [Hkv][T][D] in scratch, for Backend::attention_gen calls whose
// cache dtype is F32 (engine/src/backend.rs:305-313 accepts both; the engine's default is F16). The decode
// kernel then runs on the copy. Values are rounded to nearest even like half::f16::from_f32.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace argus {

__global__ void __launch_bounds__(256) kv_f32_to_f16_kernel(const float* __restrict__ src, __half* __restrict__ dst,
                                                            int hkv, long long T, int d, long long head_stride,
                                                            long long pos_stride) {
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;   // 4 channels per thread
    const long long total = (long long)hkv * T * d;
    if (idx >= total) return;
    const int c = (int)(idx % d);
    const long long row = idx / d;
    const long long t = row % T, h = row / T;
    const float4 v = *reinterpret_cast<const float4*>(src + h * head_stride + t * pos_stride + c);
    __half2* o = reinterpret_cast<__half2*>(dst + idx);
    o[0] = __floats2half2_rn(v.x, v.y);
    o[1] = __floats2half2_rn(v.z, v.w);
}

cudaError_t launch_kv_f32_to_f16(const float* src, void* dst, int hkv, long long T, int d, long long head_stride,
                                 long long pos_stride, cudaStream_t st) {
    const long long total = (long long)hkv * T * d;
    if (total <= 0) return cudaSuccess;
    const long long threads = total / 4;
    kv_f32_to_f16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(src, static_cast<__half*>(dst), hkv, T, d,
                                                                          head_stride, pos_stride);
    return cudaGetLastError();
}

}  // namespace argus
