// Shared helpers of the sm_100a kernels: element types, 32-bit conversions, reductions and
// the error channel of the C launchers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLM_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum : int { LLM_F32 = 0, LLM_BF16 = 1 };

// launch status codes (0 and CUDA's own error numbers aside)
enum : int { LLM_OK = 0, LLM_REFUSED = -1 };

// Records a human-readable reason for the last refusal; read back with llm_last_error().
void llm_set_error(const char* format, ...);
int llm_check_launch(const char* what);

template <typename T>
struct Num;

template <>
struct Num<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};

template <>
struct Num<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float total = (threadIdx.x < warps) ? scratch[threadIdx.x] : 0.0f;
    if (warp == 0) {
        total = warp_sum(total);
        if (lane == 0) scratch[32] = total;
    }
    __syncthreads();
    return scratch[32];
}

#define LLM_DISPATCH_DTYPE(dtype, ...)                                   \
    do {                                                                 \
        if ((dtype) == LLM_F32) {                                        \
            using T = float;                                             \
            __VA_ARGS__;                                                 \
        } else if ((dtype) == LLM_BF16) {                                \
            using T = __nv_bfloat16;                                     \
            __VA_ARGS__;                                                 \
        } else {                                                         \
            llm_set_error("unknown dtype code %d", (int)(dtype));        \
            return LLM_REFUSED;                                          \
        }                                                                \
    } while (0)

// Activation type T with a weight type W: W is T, or float for a small tensor that the checkpoint
// stores in 32-bit (such tensors are not narrowed).
#define LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, ...)                                     \
    do {                                                                                        \
        if ((dtype) == LLM_F32 && (weight_dtype) == LLM_F32) {                                  \
            using T = float;                                                                    \
            using W = float;                                                                    \
            __VA_ARGS__;                                                                        \
        } else if ((dtype) == LLM_BF16 && (weight_dtype) == LLM_BF16) {                         \
            using T = __nv_bfloat16;                                                            \
            using W = __nv_bfloat16;                                                            \
            __VA_ARGS__;                                                                        \
        } else if ((dtype) == LLM_BF16 && (weight_dtype) == LLM_F32) {                          \
            using T = __nv_bfloat16;                                                            \
            using W = float;                                                                    \
            __VA_ARGS__;                                                                        \
        } else {                                                                                \
            llm_set_error("unsupported dtype pair: activations %d, weights %d", (int)(dtype),   \
                          (int)(weight_dtype));                                                 \
            return LLM_REFUSED;                                                                 \
        }                                                                                       \
    } while (0)
