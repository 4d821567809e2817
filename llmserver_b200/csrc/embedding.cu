// Token embedding: residual[n, :] = table[ids[n], :], widened to the 32-bit residual stream.
// The reference does a plain row lookup with no scaling (utils/model.py:56-59,110).
#include "common.cuh"

template <typename T>
__global__ void embedding_gather_kernel(float* __restrict__ out, const T* __restrict__ table,
                                        const int* __restrict__ ids, int hidden, int vocab, int vector_form) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    const int token = blockIdx.x;
    int id = ids[token];
    // ids are validated on the host; clamp so that a bad id can never read outside the table
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)token * hidden;
    if (vector_form) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float values[8];
            load8<T>(row + i, values);
            store8<float>(dst + i, values);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Num<T>::load(row + i);
    }
}

LLM_EXPORT int llm_embedding_gather(float* out, const void* table, const int* ids, int n_tokens, int hidden,
                                    int vocab, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    const int vector_form = hidden % 8 == 0 && aligned16(out) && aligned16(table);
    int threads = vector_form ? (hidden / 8 + 31) / 32 * 32 : (hidden >= 1024 ? 256 : 128);
    if (threads > 512) threads = 512;
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(embedding_gather_kernel<T>, n_tokens, threads, 0, stream, 
                                  out, (const T*)table, ids, hidden, vocab, vector_form)));
    return llm_check_launch("embedding_gather");
}
