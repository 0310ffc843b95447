// Scalar load / store with conversion to and from fp32, for kernels that are instantiated for half, bf16 AND float storage
// (models whose residual stream, norms and softmax run in 32-bit while projections run in 16-bit, or entirely in 32-bit).
#pragma once

#include "common.cuh"

namespace sllm {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// block-wide sum (every thread gets the total, added in the same order); red: >= 32 floats of shared memory
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();                       // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; w++) total += red[w];
    return total;
}

// dispatch on the dtype tag, float included
#define SLLM_DISPATCH_DTYPE_F32(dtype, ...)                                 \
    do {                                                                    \
        if ((dtype) == SLLM_F16) { using T = __half; __VA_ARGS__; }         \
        else if ((dtype) == SLLM_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else if ((dtype) == SLLM_F32) { using T = float; __VA_ARGS__; }     \
        else { ::sllm::set_error("unknown dtype tag %d", (int)(dtype)); return 1; } \
    } while (0)

}  // namespace sllm
