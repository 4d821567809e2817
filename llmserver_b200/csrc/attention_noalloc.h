// Split-KV decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in AshvinSehgal/LLMServer; it exists for users of this library
// who call it from places where cudaMalloc (or a framework allocator that may fall back to it) is not
// an option: a serving loop that has handed every free byte of the GPU to its KV cache and must not
// fail or stall on an allocation in the middle of a step, a latency-critical thread that may not take
// the driver's allocation locks, or a plain C host program that links this library without PyTorch
// and has no caching allocator at all.
//
// It computes exactly what llm_attention_mma computes for a batch of single-token (decode) sequences,
// but the scratch memory of the split-KV algorithm (per-split partial outputs, maxima and sums) lives
// in a fixed array inside the library instead of being passed in.
//
//   * The array is LLM_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory per GPU that loads the library,
//     held until the process exits.  A call needs
//         n_seqs * n_q_heads * max_splits * (head_dim + 2) * 4 bytes
//     of it and is refused with LLM_REFUSED (-1) and a message (llm_last_error) if that is more.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and sets the
//     kernels' shared-memory limit on that device (both are remembered per device).  Make that first call
//     outside any stream capture.
//   * Every call uses the same array, and what the previous call left there is simply overwritten:
//     each slot that a call reads it has written first, so nothing has to be cleared.  For the same
//     reason two calls that run at the same time on one GPU (different streams) would corrupt each
//     other: keep calls on one stream, or order them yourself.
//   * No cudaMalloc, cudaFree or other allocating routine is called, here or in the kernels.
//
// Arguments are those of llm_attention_mma restricted to decode: `q` holds head h of the sequence whose
// token index is t at q[t * q_stride + h * head_dim] (bfloat16); pages are [num_pages, kv_head, slot,
// head_dim]; block_tables is int32 [n_seqs, max_blocks]; q_start is int32 [n_seqs + 1] with
// q_start[s + 1] - q_start[s] == 1 for every sequence that is to be computed (q_start[s] is its token
// index t, normally 0, 1, 2, ...; the scratch slots are counted by s, not by t) and context_len int32
// [n_seqs] (tokens the sequence holds, the new one included), both on the device; `out` is bfloat16, row t
// of [tokens, n_q_heads * head_dim].  split_len is a positive multiple of 64, with max_splits at least
// ceil(longest context / split_len) + 1; or minus the number of equal parts every context is divided into,
// with max_splits at least that number.  Returns 0 when the kernels were launched.
//
// What the block tables must hold.  Keys travel in tiles of 64, so the kernels look at every table entry up
// to the end of the last 64-key tile of a context (and, with a window, from the tile the window starts in),
// also where those keys are masked out.  Entries in that range should name pages of the pool.  An entry
// outside 0 .. num_pages - 1 is never followed: its keys are read as zeros, and the status word is set to 5.
// The V slots of every page that can be named there must hold finite numbers (a pool that was zeroed once is
// enough): a masked key has probability 0, and 0 x NaN would still be NaN.  A sequence with context_len <= 0
// gets zeros.
//
// Errors the kernels find cannot be returned by the call that launches them; they are kept in a status word
// beside the scratch array, cleared at the start of every call and read with
// llm_attention_decode_noalloc_status(stream), which waits for the stream: 0 nothing, 3 a bounded wait on a
// copy ran out, 5 a block-table entry named no page of the pool, 6 a context needed more than max_splits
// splits (its last keys were left out; the scratch array itself is never overrun).
#pragma once

#include <cuda_runtime.h>

#define LLM_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int llm_attention_decode_noalloc(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                 const int* block_tables, int max_blocks, const int* q_start, const int* context_len,
                                 void* out, int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                 int num_pages, float scale, int window, int split_len, int max_splits,
                                 cudaStream_t stream);

int llm_attention_decode_noalloc_status(cudaStream_t stream);

#ifdef __cplusplus
}
#endif
