// RMSNorm and residual-add + RMSNorm over the 32-bit residual stream.
//
//   residual[r] += delta[r]            (32-bit sum; skipped when delta is null)
//   out[o]       = residual[r] * rsqrt(mean(residual[r]^2) + eps) * weight
//
// Statistics, the product with the weight and the residual sum are 32-bit; the result is rounded
// once to the activation type.  The reference's fused kernel (utils/fused_ops.py:65-78) rounds
// the residual sum to the activation type first; keeping the stream in 32-bit is more exact.
// `rows` (optional) selects the source rows: output row o reads row rows[o]; used for the final
// norm, which runs only where logits are wanted (utils/model.py:147-157).
// With `squares_out` the division by the root mean square is left to the consumer: out = residual * weight, and
// squares_out[o] = sum(residual[r]^2), for a product kernel that scales its accumulators row by row.
//
// Two forms of the same arithmetic: a vector form (16-byte accesses, the row held in registers between
// the two passes) for widths that are a multiple of 8 and at most 16384, and a scalar form for the rest.
// The sum of squares is taken in the same order in both passes of a form, and the order depends on the
// width only, never on how many rows the call has.
#include "common.cuh"

namespace {
constexpr int kChunk = 8;        // elements a thread handles at a time in the vector form
constexpr int kMaxChunks = 4;    // per thread
}

template <typename T, typename W>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const W* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int width, float eps, int write_residual,
                                       float* __restrict__ squares_out) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    const T* del = delta ? delta + (size_t)r * width : nullptr;
    const int chunks = width / kChunk;
    float values[kMaxChunks][kChunk];
    float sum_squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            load8<float>(res + c * kChunk, values[i]);
            if (del) {
                float added[kChunk];
                load8<T>(del + c * kChunk, added);
#pragma unroll
                for (int j = 0; j < kChunk; ++j) values[i][j] += added[j];
                if (write_residual) store8<float>(res + c * kChunk, values[i]);
            }
#pragma unroll
            for (int j = 0; j < kChunk; ++j) sum_squares += values[i][j] * values[i][j];
        }
    }
    const float total = block_sum(sum_squares, scratch);
    const float inverse = squares_out ? 1.0f : rsqrtf(total / (float)width + eps);
    if (squares_out && threadIdx.x == 0) squares_out[o] = total;
    T* dst = out + (size_t)o * width;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            float scale[kChunk], scaled[kChunk];
            load8<W>(weight + c * kChunk, scale);
#pragma unroll
            for (int j = 0; j < kChunk; ++j) scaled[j] = values[i][j] * inverse * scale[j];
            store8<T>(dst + c * kChunk, scaled);
        }
    }
}

template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const W* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps, int write_residual,
                                       float* __restrict__ squares_out) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    const T* del = delta ? delta + (size_t)r * width : nullptr;
    float sum_squares = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (del) {
            v += Num<T>::load(del + i);
            if (write_residual) res[i] = v;
        }
        sum_squares += v * v;
    }
    const float total = block_sum(sum_squares, scratch);
    const float inverse = squares_out ? 1.0f : rsqrtf(total / (float)width + eps);
    if (squares_out && threadIdx.x == 0) squares_out[o] = total;
    T* dst = out + (size_t)o * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (del && !write_residual) v += Num<T>::load(del + i);
        Num<T>::store(dst + i, v * inverse * Num<W>::load(weight + i));
    }
}

// Plain RMSNorm of activation-typed rows (used by parts that normalise something other than the
// residual stream).  Same arithmetic.
template <typename T, typename W>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const W* __restrict__ weight, T* __restrict__ out,
                               int width, float eps) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float scratch[33];
    const T* src = x + (size_t)blockIdx.x * width;
    float sum_squares = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = Num<T>::load(src + i);
        sum_squares += v * v;
    }
    const float total = block_sum(sum_squares, scratch);
    const float inverse = rsqrtf(total / (float)width + eps);
    T* dst = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        Num<T>::store(dst + i, Num<T>::load(src + i) * inverse * Num<W>::load(weight + i));
}

static int norm_threads(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }

LLM_EXPORT int llm_add_rmsnorm(float* residual, const void* delta, const void* weight, void* out, const int* rows,
                               int n_rows, int width, float eps, int write_residual, int dtype,
                               int weight_dtype, float* squares_out, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    const int chunks = width / kChunk;
    // the block size depends on the width only, so a row is summed in the same order in every call
    int threads = ((chunks + 31) / 32) * 32;
    if (threads > 512) threads = 512;
    const bool vector_form = width % kChunk == 0 && width >= kChunk && aligned16(residual) && aligned16(out) &&
                             aligned16(delta) && aligned16(weight) && chunks <= threads * kMaxChunks;
    if (vector_form) {
        LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                                  (llm_launch(add_rmsnorm_vec_kernel<T, W>, n_rows, threads, 0, stream, 
                                      residual, (const T*)delta, (const W*)weight, (T*)out, rows, width, eps,
                                      write_residual, squares_out)));
        return llm_check_launch("add_rmsnorm");
    }
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                              (llm_launch(add_rmsnorm_kernel<T, W>, n_rows, norm_threads(width), 0, stream, 
                                  residual, (const T*)delta, (const W*)weight, (T*)out, rows, width, eps,
                                  write_residual, squares_out)));
    return llm_check_launch("add_rmsnorm");
}

LLM_EXPORT int llm_rmsnorm(const void* x, const void* weight, void* out, int n_rows, int width, float eps,
                           int dtype, int weight_dtype, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                              (llm_launch(rmsnorm_kernel<T, W>, n_rows, norm_threads(width), 0, stream, 
                                  (const T*)x, (const W*)weight, (T*)out, width, eps)));
    return llm_check_launch("rmsnorm");
}
