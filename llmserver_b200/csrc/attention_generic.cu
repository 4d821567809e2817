// Attention over the paged cache, any sizes, 32-bit arithmetic: the kernel of the true 32-bit path
// and the fallback of the bfloat16 path for head sizes its tensor-core kernels refuse.
//
// One warp per (query token, query head).  The query at absolute position p sees keys
// max(0, p - window + 1) .. p of its own sequence (window 0 = all), read through the sequence's
// block table; the new tokens' keys are already in the cache when this runs.  Scores, the running
// maximum, the normaliser and the output accumulate in 32-bit with the online-softmax recurrence
// the reference's paged path uses (utils/attention.py:75-96, utils/paged_attention.py:60-75);
// query head h reads kv head h / group (utils/attention.py:186-190); scale multiplies the dot
// product (utils/architecture.py:105).
//
// Keys are visited 32 at a time from the first visible one, each lane owning one key's dot
// product, so the order of every sum depends only on the query's position: the result for a token
// is bit-identical however the prompt was cut into steps and whatever else is in the batch.
#include "common.cuh"

#define ATTN_MAX_D 512

template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages,
                                         const T* __restrict__ v_pages, const int* __restrict__ block_tables,
                                         int max_blocks, const int* __restrict__ seq_of_token,
                                         const int* __restrict__ positions, T* __restrict__ out, int n_q_heads,
                                         int n_kv_heads, int head_dim, int page_size, int num_pages, float scale,
                                         int window, int* __restrict__ error_flag) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    extern __shared__ float q_shared[];  // [warps][head_dim]
    const int token = blockIdx.x;
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * warps_per_block + warp;
    if (head >= n_q_heads) return;
    const int kv_head = head / (n_q_heads / n_kv_heads);
    const int position = positions[token];
    const int* table = block_tables + (size_t)seq_of_token[token] * max_blocks;

    float* q_row = q_shared + warp * head_dim;
    const T* q_src = q + (size_t)token * q_stride + (size_t)head * head_dim;
    for (int i = lane; i < head_dim; i += 32) q_row[i] = Num<T>::load(q_src + i);
    __syncwarp();

    float accumulator[ATTN_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < ATTN_MAX_D / 32; ++i) accumulator[i] = 0.0f;
    float running_max = -INFINITY, normaliser = 0.0f;

    const int first = (window > 0 && position - window + 1 > 0) ? position - window + 1 : 0;
    for (int base = first; base <= position; base += 32) {
        const int key = base + lane;
        const bool valid = key <= position;
        long long offset = 0;  // element offset of this lane's key (and value) row inside the pages
        float score = -INFINITY;
        if (valid) {
            int page = table[key / page_size];
            if ((unsigned)page >= (unsigned)num_pages) {      // no page of the pool: report it, read page 0 instead
                if (error_flag) atomicExch(error_flag, 5);
                page = 0;
            }
            offset = (((long long)page * n_kv_heads + kv_head) * page_size + key % page_size) * head_dim;
            const T* k_row = k_pages + offset;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += q_row[d] * Num<T>::load(k_row + d);
            score = dot * scale;
        }
        const float chunk_max = warp_max(score);
        const float new_max = fmaxf(running_max, chunk_max);
        const float correction = expf(running_max - new_max);  // 0 on the first chunk
        const float weight = valid ? expf(score - new_max) : 0.0f;
        normaliser = normaliser * correction + warp_sum(weight);
#pragma unroll
        for (int i = 0; i < ATTN_MAX_D / 32; ++i) accumulator[i] *= correction;
        const int in_chunk = min(32, position - base + 1);
        for (int j = 0; j < in_chunk; ++j) {
            const float w = __shfl_sync(0xffffffffu, weight, j);
            const long long row = __shfl_sync(0xffffffffu, offset, j);
            const T* v_row = v_pages + row;
#pragma unroll
            for (int i = 0; i < ATTN_MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) accumulator[i] += w * Num<T>::load(v_row + d);
            }
        }
        running_max = new_max;
    }
    T* dst = out + (size_t)token * n_q_heads * head_dim + (size_t)head * head_dim;
    const float inverse = 1.0f / normaliser;
#pragma unroll
    for (int i = 0; i < ATTN_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) Num<T>::store(dst + d, accumulator[i] * inverse);
    }
}

LLM_EXPORT int llm_attention_generic(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                     const int* block_tables, int max_blocks, const int* seq_of_token,
                                     const int* positions, void* out, int n_tokens, int n_q_heads, int n_kv_heads,
                                     int head_dim, int page_size, int num_pages, float scale, int window,
                                     int* error_flag, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (head_dim > ATTN_MAX_D || head_dim <= 0) {
        llm_set_error("attention_generic: head_dim %d is outside 1..%d", head_dim, ATTN_MAX_D);
        return LLM_REFUSED;
    }
    if (num_pages <= 0) {
        llm_set_error("attention_generic: the page pool has %d pages", num_pages);
        return LLM_REFUSED;
    }
    if (n_kv_heads <= 0 || n_q_heads % n_kv_heads) {
        llm_set_error("attention_generic: %d query heads are no multiple of %d kv heads", n_q_heads, n_kv_heads);
        return LLM_REFUSED;
    }
    const int warps = 4;
    dim3 grid(n_tokens, (n_q_heads + warps - 1) / warps);
    const size_t shared = (size_t)warps * head_dim * sizeof(float);
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(attention_generic_kernel<T>, grid, warps * 32, shared, stream, 
                                  (const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_tables,
                                  max_blocks, seq_of_token, positions, (T*)out, n_q_heads, n_kv_heads, head_dim,
                                  page_size, num_pages, scale, window, error_flag)));
    return llm_check_launch("attention_generic");
}
