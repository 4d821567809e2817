// SwiGLU gate: out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i], gate half first
// (utils/layers.py:205-217).  The sigmoid and the product are 32-bit and the result is rounded once;
// the reference's fused kernel rounds silu(gate) to the activation type before the product
// (utils/fused_ops.py:80-88).
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int intermediate) {
    const size_t row = blockIdx.y;
    const T* src = gate_up + row * 2 * (size_t)intermediate;
    T* dst = out + row * (size_t)intermediate;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < intermediate; i += gridDim.x * blockDim.x) {
        const float gate = Num<T>::load(src + i);
        const float up = Num<T>::load(src + intermediate + i);
        Num<T>::store(dst + i, gate / (1.0f + expf(-gate)) * up);
    }
}

LLM_EXPORT int llm_silu_mul(const void* gate_up, void* out, int n_rows, int intermediate, int dtype,
                            cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    if (n_rows > 65535 * 1) {
        // grid.y is limited to 65535 rows per launch; split the launch
        int status = llm_silu_mul(gate_up, out, 65535, intermediate, dtype, stream);
        if (status != LLM_OK) return status;
        const size_t element = dtype == LLM_F32 ? 4 : 2;
        return llm_silu_mul((const char*)gate_up + (size_t)65535 * 2 * intermediate * element,
                            (char*)out + (size_t)65535 * intermediate * element, n_rows - 65535, intermediate, dtype,
                            stream);
    }
    const int threads = 256;
    int blocks_x = (intermediate + threads - 1) / threads;
    if (blocks_x > 64) blocks_x = 64;
    dim3 grid(blocks_x, n_rows);
    LLM_DISPATCH_DTYPE(dtype, (silu_mul_kernel<T><<<grid, threads, 0, stream>>>((const T*)gate_up, (T*)out,
                                                                                intermediate)));
    return llm_check_launch("silu_mul");
}
