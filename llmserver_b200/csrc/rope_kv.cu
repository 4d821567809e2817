// Fused per-head Q/K RMSNorm + rotary position encoding + paged K/V write.
//
// One warp per (token, head) of the packed projection qkv[n, (Hq + 2 Hkv) * D]:
//   * Q heads: q = rmsnorm(q) * w_q, rotated, written back in place (attention reads them there);
//   * K heads: the same with w_k, written into the token's slot of the K pages;
//   * V heads: copied into the V pages unchanged.
// Order and formulas follow the reference: norm before rotation, V untouched
// (utils/attention.py:143-158), x' = x cos + rotate_half(x) sin with both halves carrying the same
// angle = position * inv_freq (utils/layers.py:155-177), K cached after norm and rotation, V raw
// (utils/attention.py:172-176).  The reference's fused kernel (utils/fused_ops.py:90-134) rounds to
// the activation type after the norm, after the weight and after x*cos; here all of it is 32-bit
// (angles and cos/sin too) and each value is rounded once.
//
// Pages are laid out [page, kv_head, slot, D]: one (page, head) is a contiguous page_size * D run.
// A token's page is block_tables[seq_of_token[n], position / page_size].
#include "common.cuh"

__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store_pair(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
}

template <typename T, typename W>
__global__ void qk_norm_rope_kv_write_kernel(T* __restrict__ qkv, const W* __restrict__ q_weight,
                                             const W* __restrict__ k_weight, const float* __restrict__ inv_freq,
                                             const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                             const int* __restrict__ block_tables, int max_blocks,
                                             T* __restrict__ k_pages, T* __restrict__ v_pages, int n_q_heads,
                                             int n_kv_heads, int head_dim, int page_size, int num_pages, float eps,
                                             int write_cache, int* __restrict__ error_flag, int vector_form) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    const int token = blockIdx.y;
    const int warps_per_block = blockDim.x >> 5;
    const int head = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    if (head >= total_heads) return;
    const int half = head_dim >> 1;
    T* src = qkv + (size_t)token * total_heads * head_dim + (size_t)head * head_dim;
    const int position = positions[token];

    T* dst = nullptr;  // where the rotated / copied head goes
    const bool is_q = head < n_q_heads;
    const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
    if (is_q) {
        dst = src;
    } else {
        if (!write_cache) return;
        const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads;
        const int page = block_tables[(size_t)seq_of_token[token] * max_blocks + position / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicExch(error_flag, 1 + token);  // host turns this into an exception
            return;
        }
        T* pages = is_k ? k_pages : v_pages;
        dst = pages + (((size_t)page * n_kv_heads + kv_head) * page_size + position % page_size) * head_dim;
    }

    if (!is_q && !is_k) {  // V: plain copy
        if (vector_form) {
            constexpr int kPerVector = 16 / sizeof(T);
            for (int i = lane * kPerVector; i < head_dim; i += 32 * kPerVector)
                *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
        } else {
            for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
        }
        return;
    }

    const W* weight = is_q ? q_weight : k_weight;
    if (vector_form) {
        // lanes own element pairs (2p, 2p + 1) of the low half and the same pairs of the high half
        const int pairs = half >> 1;
        float inverse = 1.0f;
        if (weight) {
            float sum_squares = 0.0f;
            for (int p = lane; p < pairs; p += 32) {
                const float2 low = load_pair(src + 2 * p), high = load_pair(src + half + 2 * p);
                sum_squares += low.x * low.x + low.y * low.y + high.x * high.x + high.y * high.y;
            }
            inverse = rsqrtf(warp_sum(sum_squares) / (float)head_dim + eps);
        }
        for (int p = lane; p < pairs; p += 32) {
            float2 low = load_pair(src + 2 * p), high = load_pair(src + half + 2 * p);
            if (weight) {
                const float2 w_low = load_pair(weight + 2 * p), w_high = load_pair(weight + half + 2 * p);
                low.x = low.x * inverse * w_low.x;
                low.y = low.y * inverse * w_low.y;
                high.x = high.x * inverse * w_high.x;
                high.y = high.y * inverse * w_high.y;
            }
            if (inv_freq) {
                const float angle_x = (float)position * inv_freq[2 * p], angle_y = (float)position * inv_freq[2 * p + 1];
                const float cx = cosf(angle_x), sx = sinf(angle_x), cy = cosf(angle_y), sy = sinf(angle_y);
                const float2 rotated_low = make_float2(low.x * cx - high.x * sx, low.y * cy - high.y * sy);
                const float2 rotated_high = make_float2(high.x * cx + low.x * sx, high.y * cy + low.y * sy);
                low = rotated_low;
                high = rotated_high;
            }
            store_pair(dst + 2 * p, low);
            store_pair(dst + half + 2 * p, high);
        }
        return;
    }
    float inverse = 1.0f;
    if (weight) {
        float sum_squares = 0.0f;
        for (int i = lane; i < head_dim; i += 32) {
            const float v = Num<T>::load(src + i);
            sum_squares += v * v;
        }
        inverse = rsqrtf(warp_sum(sum_squares) / (float)head_dim + eps);
    }
    for (int i = lane; i < half; i += 32) {
        float low = Num<T>::load(src + i), high = Num<T>::load(src + half + i);
        if (weight) {
            low = low * inverse * Num<W>::load(weight + i);
            high = high * inverse * Num<W>::load(weight + half + i);
        }
        if (inv_freq) {
            const float angle = (float)position * inv_freq[i];
            const float c = cosf(angle), s = sinf(angle);
            const float rotated_low = low * c - high * s;   // rotate_half puts -high under the low half
            const float rotated_high = high * c + low * s;
            low = rotated_low;
            high = rotated_high;
        }
        Num<T>::store(dst + i, low);
        Num<T>::store(dst + half + i, high);
    }
}

LLM_EXPORT int llm_qk_norm_rope_kv_write(void* qkv, const void* q_weight, const void* k_weight, const float* inv_freq,
                                         const int* positions, const int* seq_of_token, const int* block_tables,
                                         int max_blocks, void* k_pages, void* v_pages, int n_tokens, int n_q_heads,
                                         int n_kv_heads, int head_dim, int page_size, int num_pages, float eps,
                                         int write_cache, int* error_flag, int dtype, int weight_dtype,
                                         cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (head_dim % 2) {
        llm_set_error("qk_norm_rope_kv_write: head_dim must be even, got %d", head_dim);
        return LLM_REFUSED;
    }
    if (n_tokens > 65535) {
        llm_set_error("qk_norm_rope_kv_write: at most 65535 tokens per launch, got %d", n_tokens);
        return LLM_REFUSED;
    }
    const int warps = 4;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    // pair and 16-byte accesses need head_dim to be a multiple of 8 (bfloat16) or 4 (float) and aligned bases
    const int per_vector = dtype == LLM_F32 ? 4 : 8;
    const int vector_form = head_dim % per_vector == 0 && head_dim % 4 == 0 && aligned16(qkv) && aligned16(k_pages) &&
                            aligned16(v_pages) && aligned16(q_weight) && aligned16(k_weight);
    dim3 grid((total_heads + warps - 1) / warps, n_tokens);
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, (llm_launch(qk_norm_rope_kv_write_kernel<T, W>, grid, warps * 32, 0, stream, 
                                  (T*)qkv, (const W*)q_weight, (const W*)k_weight, inv_freq, positions, seq_of_token,
                                  block_tables, max_blocks, (T*)k_pages, (T*)v_pages, n_q_heads, n_kv_heads, head_dim,
                                  page_size, num_pages, eps, write_cache, error_flag, vector_form)));
    return llm_check_launch("qk_norm_rope_kv_write");
}
