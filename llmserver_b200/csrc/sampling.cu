// Sampling over 32-bit logits: greedy argmax and temperature sampling in one kernel.
//
// The reference samples greedily only (utils/engine.py:295-297).  Temperature sampling here is the
// Gumbel-max form: token = argmax_i(logit_i / T + g_i), g_i = -log(-log(u_i)), with u_i a
// counter-based uniform of (seed, step, i).  No state is kept and no row reads another row's
// numbers, so a request's draw cannot depend on what else is in the batch.  T == 0 is greedy.
// Ties go to the lowest index, as torch.argmax does.
#include "common.cuh"

__device__ __forceinline__ uint32_t mix32(uint32_t v) {
    v ^= v >> 16;
    v *= 0x7FEB352Du;
    v ^= v >> 15;
    v *= 0x846CA68Bu;
    v ^= v >> 16;
    return v;
}

__device__ __forceinline__ float uniform_for(uint64_t seed, uint32_t step, uint32_t index) {
    uint32_t word = mix32((uint32_t)seed ^ 0x9E3779B9u);
    word = mix32(word ^ (uint32_t)(seed >> 32));
    word = mix32(word ^ step);
    word = mix32(word ^ index);
    return ((float)(word >> 9) + 0.5f) * (1.0f / 8388608.0f);  // exact in 32-bit, never 0 or 1
}

// Keeps the larger score; equal scores keep the lower index.
__device__ __forceinline__ void take_better(float& best, int& best_index, float score, int index) {
    if (score > best || (score == best && index < best_index)) {
        best = score;
        best_index = index;
    }
}

__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperatures,
                              const uint64_t* __restrict__ seeds, const int* __restrict__ steps,
                              int* __restrict__ out, int vocab) {
    __shared__ float best_values[32];
    __shared__ int best_indices[32];
    const int row = blockIdx.x;
    const float* src = logits + (size_t)row * vocab;
    const float temperature = temperatures ? temperatures[row] : 0.0f;
    const uint64_t seed = seeds ? seeds[row] : 0;
    const uint32_t step = steps ? (uint32_t)steps[row] : 0;
    float best = -INFINITY;
    int best_index = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float score = src[i];
        if (temperature > 0.0f) {
            const float u = uniform_for(seed, step, (uint32_t)i);
            score = score / temperature - logf(-logf(u));
        }
        if (score != score) score = -INFINITY;  // a NaN never wins
        take_better(best, best_index, score, i);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        take_better(best, best_index, other, other_index);
    }
    if (lane == 0) {
        best_values[warp] = best;
        best_indices[warp] = best_index;
    }
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        best = lane < warps ? best_values[lane] : -INFINITY;
        best_index = lane < warps ? best_indices[lane] : 0x7fffffff;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
            take_better(best, best_index, other, other_index);
        }
        if (lane == 0) out[row] = best_index == 0x7fffffff ? 0 : best_index;
    }
}

LLM_EXPORT int llm_sample(const float* logits, const float* temperatures, const uint64_t* seeds, const int* steps,
                          int* out, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    const int threads = vocab >= 8192 ? 1024 : 256;
    sample_kernel<<<n_rows, threads, 0, stream>>>(logits, temperatures, seeds, steps, out, vocab);
    return llm_check_launch("sample");
}
