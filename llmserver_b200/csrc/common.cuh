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

// Programmatic dependent launch: a kernel launched with the attribute below may start while the kernel
// before it in the stream is still running; it calls pdl_wait() before it touches anything that kernel
// wrote (or anything it will overwrite), and pdl_trigger() as early as possible so that its own successor
// can start.  Without the attribute both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool llm_pdl_enabled();

// Raises a kernel's dynamic shared-memory limit to `bytes` on the current device, once per (kernel, device); with
// `max_carveout` the kernel also asks for the largest shared-memory carve-out.  Returns LLM_OK or a CUDA error (with
// the message recorded).
int llm_raise_shared_limit(const void* kernel, size_t bytes, const char* what, bool max_carveout = false);

// Launches `kernel` on `stream` with programmatic stream serialization (unless switched off with
// LLMSERVER_B200_PDL=0).  Every kernel launched this way begins with pdl_trigger(); pdl_wait();
template <typename... Params, typename... Args>
inline void llm_launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared, cudaStream_t stream,
                       Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = llm_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);   // errors surface in llm_check_launch
}

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

// 16-byte vector access: VEC = 16 / sizeof(T) elements (8 bfloat16 or 4 float) to and from 32-bit values.
template <typename T>
struct Vec16;

template <>
struct Vec16<float> {
    static constexpr int kCount = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 raw = *reinterpret_cast<const float4*>(p);
        v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};

template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int kCount = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 pair = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[i]));
            v[2 * i] = pair.x;
            v[2 * i + 1] = pair.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint32_t words[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            words[i] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(words[0], words[1], words[2], words[3]);
    }
};

// Eight consecutive elements of either type to and from 32-bit values (pointers 16-byte aligned).
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
    if constexpr (sizeof(T) == 2) {
        Vec16<T>::load(p, v);
    } else {
        float low[4], high[4];
        Vec16<float>::load(reinterpret_cast<const float*>(p), low);
        Vec16<float>::load(reinterpret_cast<const float*>(p) + 4, high);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[j] = low[j];
            v[4 + j] = high[j];
        }
    }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
    if constexpr (sizeof(T) == 2) {
        Vec16<T>::store(p, v);
    } else {
        float low[4], high[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            low[j] = v[j];
            high[j] = v[4 + j];
        }
        Vec16<float>::store(reinterpret_cast<float*>(p), low);
        Vec16<float>::store(reinterpret_cast<float*>(p) + 4, high);
    }
}

__host__ __device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

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
