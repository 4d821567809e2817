// C[M, N] = A[M, K] * W[N, K]^T in true 32-bit: FMA on the CUDA cores, no tensor cores, no TF32.
//
// This is the matrix product of the 32-bit path (the reference leaves the TF32 switch to PyTorch's
// global flags, utils/attention.py:119-124; here the 32-bit path cannot use reduced precision at
// all).  Each output element is one thread's running sum over k = 0 .. K-1 in ascending order, so a
// row's result does not depend on how many other rows the call has: the 32-bit path gives
// bit-identical activations however a prompt is cut.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each
}

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w,
                                                       float* __restrict__ c, int m_total, int n_total, int k_total,
                                                       int lda, int ldw, int ldc) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float a_tile[BK][BM + 4];
    __shared__ float w_tile[BK][BN + 4];
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int thread = threadIdx.x;
    const int row_group = thread / 16, col_group = thread % 16;  // outputs (row_group*4.., col_group*4..)
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    const int load_k = thread % BK, load_row = thread / BK;  // 16 rows per pass, 4 passes
    for (int k0 = 0; k0 < k_total; k0 += BK) {
#pragma unroll
        for (int pass = 0; pass < BM / 16; ++pass) {
            const int row = load_row + pass * 16;
            const int k = k0 + load_k;
            const int gm = m0 + row, gn = n0 + row;
            a_tile[load_k][row] = (gm < m_total && k < k_total) ? a[(size_t)gm * lda + k] : 0.0f;
            w_tile[load_k][row] = (gn < n_total && k < k_total) ? w[(size_t)gn * ldw + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a_values[TM], w_values[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a_values[i] = a_tile[k][row_group * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w_values[j] = w_tile[k][col_group * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a_values[i], w_values[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + row_group * TM + i;
        if (gm >= m_total) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + col_group * TN + j;
            if (gn < n_total) c[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

LLM_EXPORT int llm_gemm_f32(const float* a, const float* w, float* c, int m, int n, int k, int lda, int ldw, int ldc,
                            cudaStream_t stream) {
    if (m == 0 || n == 0) return LLM_OK;
    const int blocks_m = (m + BM - 1) / BM;
    if ((n + BN - 1) / BN > 65535) {
        llm_set_error("gemm_f32: at most %d output columns per launch, got %d", 65535 * BN, n);
        return LLM_REFUSED;
    }
    dim3 grid(blocks_m, (n + BN - 1) / BN);
    llm_launch(gemm_f32_kernel, grid, 256, 0, stream, a, w, c, m, n, k, lda, ldw, ldc);
    return llm_check_launch("gemm_f32");
}
