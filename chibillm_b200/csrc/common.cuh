// Shared helpers of the sm_100a kernels: element types, loads and stores in
// 32-bit arithmetic, warp and block reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Element type codes used by every C entry point.
#define CHIBI_F32 0
#define CHIBI_BF16 1

// Return codes of the C entry points (0 = ok, >0 = cudaError_t, <0 = ours).
#define CHIBI_OK 0
#define CHIBI_ERR_ARGUMENT (-1)
#define CHIBI_ERR_UNSUPPORTED (-2)
#define CHIBI_ERR_DEVICE_CHECK (-3)

#define CHIBI_API extern "C" __attribute__((visibility("default")))

namespace chibi {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v)
{
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds at least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0)
        scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0)
            scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0)
        scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0)
            scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

inline int launch_status()
{
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? CHIBI_OK : static_cast<int>(e);
}

} // namespace chibi

// Calls `body` with `T` bound to the element type that `code` names.
#define CHIBI_DISPATCH_TYPE(code, T, ...)                                                          \
    do {                                                                                           \
        if ((code) == CHIBI_F32) {                                                                 \
            using T = float;                                                                       \
            __VA_ARGS__;                                                                           \
        } else if ((code) == CHIBI_BF16) {                                                         \
            using T = __nv_bfloat16;                                                               \
            __VA_ARGS__;                                                                           \
        } else {                                                                                   \
            return CHIBI_ERR_ARGUMENT;                                                             \
        }                                                                                          \
    } while (0)
