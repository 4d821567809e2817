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

// One block scans a slice of a row; grid (slices, rows).  With one slice the token goes straight to
// `out`; with more, each block leaves its best (score, index) in `partial` and sample_merge_kernel picks.
__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperatures,
                              const uint64_t* __restrict__ seeds, const int* __restrict__ steps,
                              int* __restrict__ out, int vocab, float* __restrict__ partial_scores,
                              int* __restrict__ partial_indices) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float best_values[32];
    __shared__ int best_indices[32];
    const int row = blockIdx.y, slices = gridDim.x;
    const float* src = logits + (size_t)row * vocab;
    const float temperature = temperatures ? temperatures[row] : 0.0f;
    const uint64_t seed = seeds ? seeds[row] : 0;
    const uint32_t step = steps ? (uint32_t)steps[row] : 0;
    const int per_slice = (vocab + slices - 1) / slices;
    const int begin = blockIdx.x * per_slice;
    const int end = min(vocab, begin + per_slice);
    float best = -INFINITY;
    int best_index = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
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
        if (lane == 0) {
            if (slices == 1) {
                out[row] = best_index == 0x7fffffff ? 0 : best_index;
            } else {
                partial_scores[row * slices + blockIdx.x] = best;
                partial_indices[row * slices + blockIdx.x] = best_index;
            }
        }
    }
}

__global__ void sample_merge_kernel(const float* __restrict__ partial_scores, const int* __restrict__ partial_indices,
                                    int* __restrict__ out, int slices) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    const int row = blockIdx.x, lane = threadIdx.x;
    float best = -INFINITY;
    int best_index = 0x7fffffff;
    for (int s = lane; s < slices; s += 32) take_better(best, best_index, partial_scores[row * slices + s], partial_indices[row * slices + s]);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        take_better(best, best_index, other, other_index);
    }
    if (lane == 0) out[row] = best_index == 0x7fffffff ? 0 : best_index;
}

// How many slices a row of `vocab` logits is scanned in (the caller sizes the scratch by it).
LLM_EXPORT int llm_sample_slices(int n_rows, int vocab) {
    if (vocab < 16384) return 1;
    int slices = (vocab + 8191) / 8192;
    if (slices > 32) slices = 32;
    return slices;
}

// partial_scores / partial_indices: [n_rows, slices] each, needed only when slices > 1.
LLM_EXPORT int llm_sample(const float* logits, const float* temperatures, const uint64_t* seeds, const int* steps,
                          int* out, int n_rows, int vocab, float* partial_scores, int* partial_indices,
                          cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    if (n_rows > 65535) {
        llm_set_error("sample: at most 65535 rows per launch, got %d", n_rows);
        return LLM_REFUSED;
    }
    const int slices = llm_sample_slices(n_rows, vocab);
    if (slices > 1 && (partial_scores == nullptr || partial_indices == nullptr)) {
        llm_set_error("sample: a vocabulary of %d is scanned in %d slices and needs scratch for them", vocab, slices);
        return LLM_REFUSED;
    }
    const int threads = vocab >= 4096 ? 512 : 256;
    dim3 grid(slices, n_rows);
    llm_launch(sample_kernel, grid, threads, 0, stream, logits, temperatures, seeds, steps, out, vocab, partial_scores,
                                                partial_indices);
    int status = llm_check_launch("sample");
    if (status != LLM_OK || slices == 1) return status;
    llm_launch(sample_merge_kernel, n_rows, 32, 0, stream, partial_scores, partial_indices, out, slices);
    return llm_check_launch("sample_merge");
}
