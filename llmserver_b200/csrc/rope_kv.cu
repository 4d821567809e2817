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
// Only the first `rotary_dim` elements of a head are rotated (the rest pass through after the norm), paired either
// as halves (i with i + rotary_dim / 2, the reference's form) or interleaved (2i with 2i + 1); anything but the
// reference's form (all of the head, halves) runs in the plain one-element-per-lane form of the first kernel.
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

template <typename T, typename W, int kHeld>
__global__ void qk_norm_rope_kv_write_kernel(T* __restrict__ qkv, const W* __restrict__ q_weight,
                                             const W* __restrict__ k_weight, const float* __restrict__ inv_freq,
                                             const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                             const int* __restrict__ block_tables, int max_blocks,
                                             T* __restrict__ k_pages, T* __restrict__ v_pages, int n_q_heads,
                                             int n_kv_heads, int head_dim, int page_size, int num_pages, float eps,
                                             int write_cache, int* __restrict__ error_flag, int vector_form, int heads_per_block,
                                             int rotary_dim, int interleaved) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    extern __shared__ float2 rotation[];   // (cos, sin) of angle = position * inv_freq[i], i < rotary_dim / 2
    const int token = blockIdx.x;
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    const int half = rotary_dim >> 1;      // the vector form below is used only when rotary_dim == head_dim
    const int position = positions[token];
    // the angles depend on the token only: computed once per block, used by every head the block handles
    if (inv_freq) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float angle = (float)position * inv_freq[i];
            rotation[i] = make_float2(cosf(angle), sinf(angle));
        }
    }
    __syncthreads();
    const int first_head = blockIdx.y * heads_per_block;
    const int end_head = min(first_head + heads_per_block, total_heads);
    for (int head = first_head + (threadIdx.x >> 5); head < end_head; head += warps_per_block) {
        T* src = qkv + (size_t)token * total_heads * head_dim + (size_t)head * head_dim;
        T* dst = nullptr;  // where the rotated / copied head goes
        const bool is_q = head < n_q_heads;
        const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
        if (is_q) {
            dst = src;
        } else {
            if (!write_cache) continue;
            const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads;
            const int page = block_tables[(size_t)seq_of_token[token] * max_blocks + position / page_size];
            if (page < 0 || page >= num_pages) {
                if (lane == 0) atomicExch(error_flag, 1 + token);  // host turns this into an exception
                continue;
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
            continue;
        }

        const W* weight = is_q ? q_weight : k_weight;
        if (vector_form) {
            // lanes own element pairs (2p, 2p + 1) of the low half and the same pairs of the high half; a head
            // of up to 128 * kHeld elements is read once and held in registers between the statistics and the rotation
            const int pairs = half >> 1;
            float2 held_low[kHeld], held_high[kHeld];
            float sum_squares = 0.0f;
#pragma unroll
            for (int i = 0; i < kHeld; ++i) {
                const int p = lane + 32 * i;
                if (p < pairs) {
                    held_low[i] = load_pair(src + 2 * p);
                    held_high[i] = load_pair(src + half + 2 * p);
                    sum_squares += held_low[i].x * held_low[i].x + held_low[i].y * held_low[i].y +
                                   held_high[i].x * held_high[i].x + held_high[i].y * held_high[i].y;
                }
            }
            float inverse = 1.0f;
            if (weight) inverse = rsqrtf(warp_sum(sum_squares) / (float)head_dim + eps);
#pragma unroll
            for (int i = 0; i < kHeld; ++i) {
                const int p = lane + 32 * i;
                if (p >= pairs) continue;
                float2 low = held_low[i], high = held_high[i];
                if (weight) {
                    const float2 w_low = load_pair(weight + 2 * p), w_high = load_pair(weight + half + 2 * p);
                    low.x = low.x * inverse * w_low.x;
                    low.y = low.y * inverse * w_low.y;
                    high.x = high.x * inverse * w_high.x;
                    high.y = high.y * inverse * w_high.y;
                }
                if (inv_freq) {
                    const float2 x = rotation[2 * p], y = rotation[2 * p + 1];    // (cos, sin)
                    const float2 rotated_low = make_float2(low.x * x.x - high.x * x.y, low.y * y.x - high.y * y.y);
                    const float2 rotated_high = make_float2(high.x * x.x + low.x * x.y, high.y * y.x + low.y * y.y);
                    low = rotated_low;
                    high = rotated_high;
                }
                store_pair(dst + 2 * p, low);
                store_pair(dst + half + 2 * p, high);
            }
            continue;
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
            // the two elements that rotate together: halves (i, i + rotary_dim / 2) or neighbours (2i, 2i + 1)
            const int first = interleaved ? 2 * i : i, second = interleaved ? 2 * i + 1 : half + i;
            float low = Num<T>::load(src + first), high = Num<T>::load(src + second);
            if (weight) {
                low = low * inverse * Num<W>::load(weight + first);
                high = high * inverse * Num<W>::load(weight + second);
            }
            if (inv_freq) {
                const float c = rotation[i].x, sn = rotation[i].y;
                const float rotated_low = low * c - high * sn;   // rotate_half puts -high under the low half
                const float rotated_high = high * c + low * sn;
                low = rotated_low;
                high = rotated_high;
            }
            Num<T>::store(dst + first, low);
            Num<T>::store(dst + second, high);
        }
        for (int i = rotary_dim + lane; i < head_dim; i += 32) {      // beyond the rotated part: the norm only
            float value = Num<T>::load(src + i);
            if (weight) value = value * inverse * Num<W>::load(weight + i);
            Num<T>::store(dst + i, value);
        }
    }
}

// The same operation for head sizes 64, 128 and 256 with aligned operands: LANES = head_dim / 16 lanes share a
// head, each holding 8 elements of the low half and the 8 elements of the high half that rotate with them
// (16-byte accesses), so a warp works on 32 / LANES heads at a time.
template <typename T, typename W, int LANES>
__global__ void qk_norm_rope_kv_write_wide_kernel(T* __restrict__ qkv, const W* __restrict__ q_weight,
                                                  const W* __restrict__ k_weight, const float* __restrict__ inv_freq,
                                                  const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                                  const int* __restrict__ block_tables, int max_blocks,
                                                  T* __restrict__ k_pages, T* __restrict__ v_pages, int n_q_heads,
                                                  int n_kv_heads, int page_size, int num_pages, float eps, int write_cache,
                                                  int* __restrict__ error_flag, int heads_per_block) {
    pdl_trigger();
    pdl_wait();
    constexpr int kHalf = LANES * 8, kDim = 2 * kHalf;
    __shared__ float2 rotation[kHalf];
    const int token = blockIdx.x;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    const int position = positions[token];
    if (inv_freq) {
        for (int i = threadIdx.x; i < kHalf; i += blockDim.x) {
            const float angle = (float)position * inv_freq[i];
            rotation[i] = make_float2(cosf(angle), sinf(angle));
        }
    }
    __syncthreads();
    const int groups_per_block = blockDim.x / LANES;
    const int group = threadIdx.x / LANES, sub = threadIdx.x % LANES;
    const int first_head = blockIdx.y * heads_per_block;
    const int end_head = min(first_head + heads_per_block, total_heads);
    const int rounds = (end_head - first_head + groups_per_block - 1) / groups_per_block;
    for (int round = 0; round < rounds; ++round) {        // the same number of rounds for every lane of a warp
        const int head = first_head + round * groups_per_block + group;
        bool active = head < end_head;
        const bool is_q = head < n_q_heads;
        const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
        T* src = qkv + (size_t)token * total_heads * kDim + (size_t)(active ? head : first_head) * kDim;
        T* dst = src;
        if (active && !is_q) {
            if (!write_cache) {
                active = false;
            } else {
                const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads;
                const int page = block_tables[(size_t)seq_of_token[token] * max_blocks + position / page_size];
                if (page < 0 || page >= num_pages) {
                    if (sub == 0) atomicExch(error_flag, 1 + token);
                    active = false;
                } else {
                    T* pages = is_k ? k_pages : v_pages;
                    dst = pages + (((size_t)page * n_kv_heads + kv_head) * page_size + position % page_size) * kDim;
                }
            }
        }
        float low[8], high[8];
        if (active) {
            load8<T>(src + sub * 8, low);
            load8<T>(src + kHalf + sub * 8, high);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) low[j] = high[j] = 0.0f;
        }
        // every lane of the warp takes part in the shuffles, whatever kind of head its group holds
        float sum_squares = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum_squares += low[j] * low[j] + high[j] * high[j];
#pragma unroll
        for (int offset = LANES / 2; offset > 0; offset >>= 1) sum_squares += __shfl_xor_sync(0xffffffffu, sum_squares, offset);
        const W* weight = is_q ? q_weight : (is_k ? k_weight : nullptr);
        if (active && (is_q || is_k)) {
            if (weight) {
                const float inverse = rsqrtf(sum_squares / (float)kDim + eps);
                float w_low[8], w_high[8];
                load8<W>(weight + sub * 8, w_low);
                load8<W>(weight + kHalf + sub * 8, w_high);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    low[j] = low[j] * inverse * w_low[j];
                    high[j] = high[j] * inverse * w_high[j];
                }
            }
            if (inv_freq) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float2 r = rotation[sub * 8 + j];      // (cos, sin)
                    const float rotated_low = low[j] * r.x - high[j] * r.y;
                    const float rotated_high = high[j] * r.x + low[j] * r.y;
                    low[j] = rotated_low;
                    high[j] = rotated_high;
                }
            }
        }
        if (active) {
            store8<T>(dst + sub * 8, low);
            store8<T>(dst + kHalf + sub * 8, high);
        }
    }
}

LLM_EXPORT int llm_qk_norm_rope_kv_write(void* qkv, const void* q_weight, const void* k_weight, const float* inv_freq,
                                         const int* positions, const int* seq_of_token, const int* block_tables,
                                         int max_blocks, void* k_pages, void* v_pages, int n_tokens, int n_q_heads,
                                         int n_kv_heads, int head_dim, int page_size, int num_pages, float eps,
                                         int write_cache, int* error_flag, int rotary_dim, int interleaved, int dtype,
                                         int weight_dtype, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (inv_freq == nullptr) {        // no rotation at all: the pairs are only the order in which elements are visited
        rotary_dim = head_dim;
        interleaved = 0;
    }
    if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 2) {
        llm_set_error("qk_norm_rope_kv_write: rotary_dim must be even and at most head_dim %d, got %d", head_dim, rotary_dim);
        return LLM_REFUSED;
    }
    const bool whole_head_in_halves = rotary_dim == head_dim && !interleaved;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    // many tokens (prompts): one block of 8 warps per token takes all heads and computes the token's angles
    // once; few tokens (decode): four heads per block of four warps, for more blocks in flight
    const int warps = n_tokens >= 256 ? 8 : 4;
    const int heads_per_block = n_tokens >= 256 ? total_heads : warps;
    // pair and 16-byte accesses need head_dim to be a multiple of 8 (bfloat16) or 4 (float) and aligned bases
    const int per_vector = dtype == LLM_F32 ? 4 : 8;
    const int vector_form = whole_head_in_halves && head_dim % per_vector == 0 && head_dim % 4 == 0 && head_dim <= 512 && aligned16(qkv) && aligned16(k_pages) &&
                            aligned16(v_pages) && aligned16(q_weight) && aligned16(k_weight);
    dim3 grid(n_tokens, (total_heads + heads_per_block - 1) / heads_per_block);
    const size_t shared = (size_t)(rotary_dim / 2 + 1) * sizeof(float2);
    // head sizes 64 / 128 / 256 with aligned operands: the wide form
    const bool wide = vector_form && (head_dim == 64 || head_dim == 128 || head_dim == 256) && aligned16(q_weight) && aligned16(k_weight);
    if (wide) {
        const int wide_threads = 256;
        const int lanes = head_dim / 16;
        const int wide_heads_per_block = n_tokens >= 256 ? total_heads : (wide_threads / lanes < total_heads ? wide_threads / lanes : total_heads);
        dim3 wide_grid(n_tokens, (total_heads + wide_heads_per_block - 1) / wide_heads_per_block);
#define LLM_ROPE_WIDE(LANES)                                                                                          \
        LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, (llm_launch(qk_norm_rope_kv_write_wide_kernel<T, W, LANES>, wide_grid, wide_threads, 0, stream, \
                                      (T*)qkv, (const W*)q_weight, (const W*)k_weight, inv_freq, positions, seq_of_token, \
                                      block_tables, max_blocks, (T*)k_pages, (T*)v_pages, n_q_heads, n_kv_heads, \
                                      page_size, num_pages, eps, write_cache, error_flag, wide_heads_per_block)));
        if (lanes == 4) {
            LLM_ROPE_WIDE(4)
        } else if (lanes == 8) {
            LLM_ROPE_WIDE(8)
        } else {
            LLM_ROPE_WIDE(16)
        }
#undef LLM_ROPE_WIDE
        return llm_check_launch("qk_norm_rope_kv_write");
    }
#define LLM_ROPE_LAUNCH(HELD)                                                                                        \
        LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, (llm_launch(qk_norm_rope_kv_write_kernel<T, W, HELD>, grid, warps * 32, shared, stream,  \
                                      (T*)qkv, (const W*)q_weight, (const W*)k_weight, inv_freq, positions, seq_of_token, \
                                      block_tables, max_blocks, (T*)k_pages, (T*)v_pages, n_q_heads, n_kv_heads, head_dim, \
                                      page_size, num_pages, eps, write_cache, error_flag, vector_form, heads_per_block, \
                                      rotary_dim, interleaved))); \

    if (head_dim <= 128) {
        LLM_ROPE_LAUNCH(1)
    } else if (head_dim <= 256) {
        LLM_ROPE_LAUNCH(2)
    } else {
        LLM_ROPE_LAUNCH(4)
    }
#undef LLM_ROPE_LAUNCH
    return llm_check_launch("qk_norm_rope_kv_write");
}
