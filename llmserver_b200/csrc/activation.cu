// SwiGLU gate: out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i], gate half first
// (utils/layers.py:205-217).  The sigmoid and the product are 32-bit and the result is rounded once;
// the reference's fused kernel rounds silu(gate) to the activation type before the product
// (utils/fused_ops.py:80-88).  16-byte accesses when the intermediate size allows, else element-wise.
#include "common.cuh"

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int intermediate,
                                    size_t total_vectors) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    constexpr int kCount = Vec16<T>::kCount;
    const int vectors_per_row = intermediate / kCount;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < total_vectors; v += (size_t)gridDim.x * blockDim.x) {
        const size_t row = v / vectors_per_row;
        const int column = (int)(v % vectors_per_row) * kCount;
        const T* src = gate_up + row * 2 * (size_t)intermediate + column;
        float gate[kCount], up[kCount], result[kCount];
        Vec16<T>::load(src, gate);
        Vec16<T>::load(src + intermediate, up);
#pragma unroll
        for (int i = 0; i < kCount; ++i) result[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
        Vec16<T>::store(out + row * (size_t)intermediate + column, result);
    }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int intermediate, size_t total) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t row = e / intermediate;
        const int column = (int)(e % intermediate);
        const T* src = gate_up + row * 2 * (size_t)intermediate + column;
        const float gate = Num<T>::load(src);
        const float up = Num<T>::load(src + intermediate);
        Num<T>::store(out + e, gate / (1.0f + expf(-gate)) * up);
    }
}

LLM_EXPORT int llm_silu_mul(const void* gate_up, void* out, int n_rows, int intermediate, int dtype,
                            cudaStream_t stream) {
    if (n_rows == 0 || intermediate == 0) return LLM_OK;
    const int per_vector = dtype == LLM_F32 ? 4 : 8;
    const int threads = 256;
    const bool vector_form = intermediate % per_vector == 0 && aligned16(gate_up) && aligned16(out);
    const size_t work = vector_form ? (size_t)n_rows * (intermediate / per_vector) : (size_t)n_rows * intermediate;
    size_t blocks = (work + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (vector_form) {
        LLM_DISPATCH_DTYPE(dtype, (llm_launch(silu_mul_vec_kernel<T>, (unsigned)blocks, threads, 0, stream, 
                                      (const T*)gate_up, (T*)out, intermediate, work)));
    } else {
        LLM_DISPATCH_DTYPE(dtype, (llm_launch(silu_mul_kernel<T>, (unsigned)blocks, threads, 0, stream, 
                                      (const T*)gate_up, (T*)out, intermediate, work)));
    }
    return llm_check_launch("silu_mul");
}
