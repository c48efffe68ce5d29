// Shared helpers for the libmbema kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mbema.h"

namespace mbema {

void set_last_cuda_error(cudaError_t e);

inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        return MBEMA_ERR_CUDA;
    }
    return MBEMA_OK;
}

#define MBEMA_CUDA_TRY(expr)                 \
    do {                                     \
        cudaError_t e__ = (expr);            \
        if (e__ != cudaSuccess) {            \
            mbema::set_last_cuda_error(e__); \
            return MBEMA_ERR_CUDA;           \
        }                                    \
    } while (0)

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// element load with dtype conversion to fp32
template <int DT>
__device__ __forceinline__ float ld_as_f32(const void* p, size_t i) {
    if (DT == MBEMA_F32)
        return reinterpret_cast<const float*>(p)[i];
    else
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float ld_dyn_f32(const void* p, int dt, size_t i) {
    return dt == MBEMA_F32 ? reinterpret_cast<const float*>(p)[i]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// four consecutive elements starting at index i (i % 4 == 0, base 16-byte aligned)
__device__ __forceinline__ float4 ld4_dyn_f32(const void* p, int dt, size_t i) {
    if (dt == MBEMA_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
}

__device__ __forceinline__ void st4_dyn(void* p, int dt, size_t i, float4 v) {
    if (dt == MBEMA_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
        __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = raw;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

}  // namespace mbema
