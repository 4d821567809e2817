// SwiGLU gate: out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i], gate half first
// (utils/layers.py:205-217).  The sigmoid and the product are 32-bit and the result is rounded once;
// the reference's fused kernel rounds silu(gate) to the activation type before the product
// (utils/fused_ops.py:80-88).  16-byte accesses when the intermediate size allows, else element-wise.
//
// With `group` > 0 the gate and up columns are interleaved in groups: columns [2 b group, 2 b group + group) hold the
// gate values of outputs [b group, (b + 1) group) and the next `group` columns their up values (the layout in which a
// 128-row tile of the fused gate/up weight holds 64 gate rows and their 64 up rows).
#include "common.cuh"

// silu(x) * y in 32-bit.  For 16-bit activations the exponential and the reciprocal are the hardware
// approximations (a few units in the last place of a 32-bit float, far below the rounding of the result).
template <typename T>
__device__ __forceinline__ float silu_times(float gate, float up) {
    if (sizeof(T) == 2) return __fdividef(gate, 1.0f + __expf(-gate)) * up;
    return gate / (1.0f + expf(-gate)) * up;
}

// Where output column `column` finds its gate value in a row of gate_up, and how far behind the up value lies.
__device__ __forceinline__ int gate_column(int column, int group) {
    return group > 0 ? (column / group) * 2 * group + column % group : column;
}

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int intermediate,
                                    size_t total_vectors, int group) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    constexpr int kCount = Vec16<T>::kCount;
    const int vectors_per_row = intermediate / kCount;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    // two vectors per thread and turn: four 16-byte loads are in flight before the first result is needed
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < total_vectors; v += 2 * stride) {
        const size_t w = v + stride;
        const bool second = w < total_vectors;
        const size_t row_v = v / vectors_per_row, row_w = second ? w / vectors_per_row : row_v;
        const int column_v = (int)(v - row_v * vectors_per_row) * kCount;
        const int column_w = second ? (int)(w - row_w * vectors_per_row) * kCount : column_v;
        const T* src_v = gate_up + row_v * 2 * (size_t)intermediate + gate_column(column_v, group);
        const T* src_w = gate_up + row_w * 2 * (size_t)intermediate + gate_column(column_w, group);
        const int to_up = group > 0 ? group : intermediate;
        float gate_v[kCount], up_v[kCount], gate_w[kCount], up_w[kCount], result[kCount];
        Vec16<T>::load(src_v, gate_v);
        Vec16<T>::load(src_v + to_up, up_v);
        Vec16<T>::load(src_w, gate_w);
        Vec16<T>::load(src_w + to_up, up_w);
#pragma unroll
        for (int i = 0; i < kCount; ++i) result[i] = silu_times<T>(gate_v[i], up_v[i]);
        Vec16<T>::store(out + row_v * (size_t)intermediate + column_v, result);
        if (second) {
#pragma unroll
            for (int i = 0; i < kCount; ++i) result[i] = silu_times<T>(gate_w[i], up_w[i]);
            Vec16<T>::store(out + row_w * (size_t)intermediate + column_w, result);
        }
    }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int intermediate, size_t total, int group) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t row = e / intermediate;
        const int column = (int)(e % intermediate);
        const T* src = gate_up + row * 2 * (size_t)intermediate + gate_column(column, group);
        const float gate = Num<T>::load(src);
        const float up = Num<T>::load(src + (group > 0 ? group : intermediate));
        Num<T>::store(out + e, gate / (1.0f + expf(-gate)) * up);
    }
}

LLM_EXPORT int llm_silu_mul(const void* gate_up, void* out, int n_rows, int intermediate, int group, int dtype,
                            cudaStream_t stream) {
    if (n_rows == 0 || intermediate == 0) return LLM_OK;
    if (group < 0 || (group > 0 && intermediate % group)) {
        llm_set_error("silu_mul: the intermediate size %d is no multiple of the group %d", intermediate, group);
        return LLM_REFUSED;
    }
    const int per_vector = dtype == LLM_F32 ? 4 : 8;
    const int threads = 256;
    const bool vector_form = intermediate % per_vector == 0 && group % per_vector == 0 && aligned16(gate_up) && aligned16(out);
    const size_t work = vector_form ? (size_t)n_rows * (intermediate / per_vector) : (size_t)n_rows * intermediate;
    size_t blocks = (work + threads - 1) / threads;
    if (vector_form) blocks = (blocks + 1) / 2;      // two vectors per thread and turn
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (vector_form) {
        LLM_DISPATCH_DTYPE(dtype, (llm_launch(silu_mul_vec_kernel<T>, (unsigned)blocks, threads, 0, stream, 
                                      (const T*)gate_up, (T*)out, intermediate, work, group)));
    } else {
        LLM_DISPATCH_DTYPE(dtype, (llm_launch(silu_mul_kernel<T>, (unsigned)blocks, threads, 0, stream, 
                                      (const T*)gate_up, (T*)out, intermediate, work, group)));
    }
    return llm_check_launch("silu_mul");
}
