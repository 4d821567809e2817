// y[M, N] = x[M, K] * W[N, K]^T in bfloat16 with 32-bit accumulation, for few rows (M <= 64: decode steps
// and the output head), written for the fifth-generation tensor cores: TMA loads into 128-byte-swizzled
// shared tiles, tcgen05.mma with the accumulator in tensor memory, tcgen05.ld for the epilogue.
//
// With few rows the product is a stream of W through the SM: every weight is read once and used M times.
// So the roles of the operands are swapped for the hardware: a CTA owns 128 rows of W as the MMA's
// M = 128 dimension and the (padded) token rows as its N dimension (16..64), walks its share of K in
// blocks of 64 through a ring of shared-memory stages, and ends with a 128 x M tile of y^T in tensor
// memory, which the epilogue writes transposed.  When N / 128 tiles are too few to fill 148 SMs, K is
// split across a thread-block cluster; the partial tiles are added through distributed shared memory in
// a fixed order (rank 0, 1, ...), so results do not depend on timing.
//
// The epilogue moves the tile through shared memory as [token][128 rows] and hands whole token rows to warps: a
// token's 128 elements are four per lane, so per-head and per-row reductions are warp reductions, rotation partners
// and gate/up pairs a shuffle away, stores 8 or 16 bytes per lane, and the warps work on different tokens
// without a block barrier (per-token block barriers cost 9 to 14 us of a q/k/v product at 32 to 64 tokens).
//
// One elected thread issues the TMA copies, one issues the MMAs; mbarriers carry "stage full" (TMA
// transaction bytes), "stage free" and "accumulator ready" (tcgen05.commit).  The thread that initialises the
// barriers requests the weight tiles of the first ring of stages at once, before the block's first barrier and
// before griddepcontrol.wait (weights do not depend on the kernel in front); the token tiles follow after the
// wait.  Every wait is bounded: a wait that runs out sets an error flag that the host reads, and the CTA still
// frees its tensor memory and leaves in step with its cluster.
//
// Two optional epilogues finish a decode step's results where they are, instead of in a kernel of their own:
// the q/k/v projection with heads of 128 (the 128 rows of W a CTA owns are one head) normalises and rotates each
// head and writes K and V into the cache pages (RopeEpilogue); the fused gate/up projection, whose weight holds
// 64 gate rows and their 64 up rows per tile, writes silu(gate) * up (silu_gate).
//
// Two more options take the stand-alone residual-add + RMSNorm kernels out of a decode step.  A product whose result
// is added to the 32-bit residual stream does so in its epilogue (StreamEpilogue), and leaves for the RMSNorm that
// follows the stream times the norm's weight, rounded to bfloat16, and the sums of squares of the updated stream per
// token and per warp's 32 columns.  The product that consumes the norm's output takes those (RowScale): it adds the
// partial sums in a fixed order, and multiplies its 32-bit accumulators token by token with 1 / rms, since
// W (s w x) = s W (w x) for a scalar s per token.  Statistics, scale and residual sum stay 32-bit.
//
// Out-of-range rows of W (N not a multiple of 128), token rows beyond M and a K that is no multiple of
// 64 are zero-filled by TMA.  K must be a multiple of 8 (16-byte row pitch) and the pointers 16-byte
// aligned; otherwise the launcher refuses and the caller uses the library product.
#include "common.cuh"
#include "tma.cuh"

#include <stdlib.h>

namespace {

constexpr int kBlockRows = 128;     // rows of W per CTA (UMMA M)
constexpr int kAtomK = 64;          // one 128-byte swizzle atom of bfloat16
constexpr int kAtoms = 2;           // atoms per pipeline stage
constexpr int kBlockK = kAtomK * kAtoms;
constexpr int kThreads = 256;       // at most: four warps up to 16 tokens, eight beyond (two have a role in the main
                                    // loop, all work in the epilogue, whose time per token is instruction issue)
constexpr int kMaxStages = 12;
constexpr int kMaxSplit = 8;

// Optional epilogue of the fused q/k/v projection of a decode step (head_dim 128: the 128 rows of W a CTA owns are
// exactly one head): per-head RMSNorm of Q and K, rotation by the token's position, Q written to the output, K and V
// written straight into the token's slot of the cache pages.  Same arithmetic as the stand-alone kernel of rope_kv.cu,
// but on the 32-bit sums of the product instead of their bfloat16 roundings.
struct RopeEpilogue {
    int on;
    const void* q_weight;      // [128] norm weights (null: no norm), bfloat16 or float
    const void* k_weight;
    int weight_is_f32;
    const float* inv_freq;     // [64] (null: no rotation)
    const int* positions;      // [m]
    const int* seq_of_token;   // [m]
    const int* block_tables;   // [sequences][max_blocks]
    int max_blocks;
    __nv_bfloat16* k_pages;    // [pages][kv heads][page_size][128]
    __nv_bfloat16* v_pages;
    int n_q_heads, n_kv_heads, page_size, num_pages;
    float eps;
    int write_cache;
    int* page_error;           // set to 1 + token when a token's page is outside the pool
};

// The input rows are a residual stream times a norm's weight, not yet divided by their root mean square: the sums of
// squares of the stream rows lie in parts[i * stride + token], i < n_parts; the accumulators of token m are multiplied
// with rsqrt(sum_i parts[i][m] / k + eps).  parts == null: no scaling.
struct RowScale {
    const float* parts;
    int n_parts, stride;
    float eps;
};

// The product is added to the residual stream [m, n] (32-bit, row pitch n) where it lies.  With next_weight, the
// updated stream times next_weight [n] is written to `scaled` (bfloat16, row pitch n) and the sums of squares of
// the updated stream over each tile's 128 columns to parts[tile * stride + token], for the RowScale of the next product.
struct StreamEpilogue {
    int on;
    float* residual;
    const void* next_weight;
    int weight_is_f32;
    __nv_bfloat16* scaled;
    float* parts;
    int stride;
};

struct GemmParams {
    void* out;
    int out_is_f32;
    int m, n, k;        // tokens, rows of W, inner size
    int ldc;
    int token_pad;      // UMMA N: m rounded up to 16
    int stages;
    int split;          // cluster size along K
    int* error_flag;
    RopeEpilogue rope;
    int silu_gate;      // 1: rows 0..63 of a tile are gate rows and rows 64..127 their up rows; the epilogue writes
                        // silu(gate) * up into an output of n / 2 columns
    RowScale scale;
    StreamEpilogue stream;
    int vector_out;     // the output (and the cache pages of the q/k/v epilogue) take 8- and 16-byte stores of four results
    int vector_stream;  // so do the stream and the next norm's input
};

using tma::mbar_expect_tx;
using tma::mbar_init;
using tma::mbar_wait;
using tma::smem_u32;

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    tma::load_2d(dst, map, bar, x, y);
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows are 128 bytes, groups of
// 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_descriptor(uint32_t smem_address) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_address & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)1 << 16;                                   // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                         // stride byte offset: 8 rows * 128 bytes
    d |= (uint64_t)1 << 46;                                   // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                   // SWIZZLE_128B
    return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M x N tile.
__device__ __forceinline__ uint32_t umma_instruction(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load_16(uint32_t address, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"   // one statement: no use of the registers can be scheduled before the wait
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// ---- The epilogues.  A finished token row of a tile is handled by ONE WARP: lane i holds the four elements
// 4 i .. 4 i + 3 of the tile's 128, so a head's sum of squares or a stream row's is one warp reduction, the partner of
// a rotation (64 elements further) and the up value of a gate sit in lane i ^ 16, and every store is 8 or 16 bytes per
// lane and 256 or 512 contiguous bytes per warp.  The warps of a block take different tokens at the same time
// and never meet at a block barrier; what a token needs beside the sums (its position, its page, the stream's values)
// is asked for together with the sums' parts.

// The two halves of a cluster barrier, for a block that says "I have read all I need of your shared memory" as soon
// as that is so and waits for the others' word only before it leaves.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ float4 load_peer4(uint32_t local_address, uint32_t rank) {
    uint32_t remote;
    float4 value;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(value.x), "=f"(value.y), "=f"(value.z), "=f"(value.w) : "r"(remote) : "memory");
    return value;
}

__device__ __forceinline__ void load_weights4(const void* weight, int is_f32, int first, int limit, float (&w)[4]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        w[c] = 1.0f;
        if (weight != nullptr && first + c < limit)
            w[c] = is_f32 ? reinterpret_cast<const float*>(weight)[first + c]
                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(weight)[first + c]);
    }
}

// Four consecutive results as bfloat16 (8 bytes at once where `vector` says the place is aligned) or float (16 bytes);
// `valid`: how many of the four exist.
__device__ __forceinline__ void store4_bf16(__nv_bfloat16* dst, const float (&v)[4], int valid, bool vector) {
    if (valid >= 4 && vector) {
        __nv_bfloat162 low = __floats2bfloat162_rn(v[0], v[1]), high = __floats2bfloat162_rn(v[2], v[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&low);
        packed.y = *reinterpret_cast<uint32_t*>(&high);
        *reinterpret_cast<uint2*>(dst) = packed;
    } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (c < valid) dst[c] = __float2bfloat16_rn(v[c]);
    }
}
__device__ __forceinline__ void store4_f32(float* dst, const float (&v)[4], int valid, bool vector) {
    if (valid >= 4 && vector) {
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (c < valid) dst[c] = v[c];
    }
}

// What the q/k/v epilogue needs of a token beside the product.
struct RopeRow {
    int position;
    int page;       // of the K and V heads' token slot; -1 outside the pool
};
__device__ __forceinline__ RopeRow rope_row(const GemmParams& p, int m, int tile) {
    const RopeEpilogue& e = p.rope;
    RopeRow r;
    r.position = e.positions[m];
    r.page = 0;
    if (tile >= e.n_q_heads && e.write_cache) {
        r.page = e.block_tables[(size_t)e.seq_of_token[m] * e.max_blocks + r.position / e.page_size];
        if (r.page < 0 || r.page >= e.num_pages) r.page = -1;
    }
    return r;
}

// What finishing token m needs beside the product: its position and page (q/k/v epilogue) or the stream's values at
// columns n4 .. n4 + 3 (stream epilogue).  Nothing for a token that does not exist.
__device__ __forceinline__ void token_inputs(const GemmParams& p, int m, int tile, int n4, RopeRow& info, float (&before)[4]) {
    info.position = info.page = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) before[c] = 0.0f;
    if (m >= p.m) return;
    if (p.rope.on) info = rope_row(p, m, tile);
    if (p.stream.on) {
        if (p.vector_stream && n4 + 3 < p.n) {
            const float4 v = *reinterpret_cast<const float4*>(p.stream.residual + (size_t)m * p.n + n4);
            before[0] = v.x, before[1] = v.y, before[2] = v.z, before[3] = v.w;
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (n4 + c < p.n) before[c] = p.stream.residual[(size_t)m * p.n + n4 + c];
        }
    }
}

// Token m of head `tile` of the q/k/v projection: per-head norm, rotation, Q to the output, K and V into the cache.
// `weight`: the head norm's weights of this lane's elements, `frequency`: the rotation's of elements 4 lane + c mod 64.
__device__ __forceinline__ void rope_finish(const GemmParams& p, int m, int lane, int tile, float (&value)[4],
                                            const float (&weight)[4], const float (&frequency)[4], RopeRow info) {
    const RopeEpilogue& e = p.rope;
    const bool is_q = tile < e.n_q_heads;
    const bool is_k = !is_q && tile < e.n_q_heads + e.n_kv_heads;
    if (is_q || is_k) {
        if ((is_q ? e.q_weight : e.k_weight) != nullptr) {
            const float squares = warp_sum(value[0] * value[0] + value[1] * value[1] + value[2] * value[2] + value[3] * value[3]);
            const float inverse = rsqrtf(squares / (float)kBlockRows + e.eps);
#pragma unroll
            for (int c = 0; c < 4; ++c) value[c] = value[c] * inverse * weight[c];
        }
        if (e.inv_freq != nullptr) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float partner = __shfl_xor_sync(0xffffffffu, value[c], 16);      // the element 64 further or back
                const float angle = (float)info.position * frequency[c];
                const float cs = cosf(angle), sn = sinf(angle);
                value[c] = lane < 16 ? value[c] * cs - partner * sn : value[c] * cs + partner * sn;
            }
        }
    }
    if (is_q) {
        store4_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldc + (size_t)tile * kBlockRows + 4 * lane, value, 4, p.vector_out != 0);
    } else if (e.write_cache) {
        const int kv_head = is_k ? tile - e.n_q_heads : tile - e.n_q_heads - e.n_kv_heads;
        if (info.page < 0) {
            if (lane == 0) atomicExch(e.page_error, 1 + m);
        } else {
            __nv_bfloat16* pages = is_k ? e.k_pages : e.v_pages;
            store4_bf16(pages + (((size_t)info.page * e.n_kv_heads + kv_head) * e.page_size + info.position % e.page_size) * kBlockRows + 4 * lane,
                        value, 4, p.vector_out != 0);
        }
    }
}

// Token m of a tile of the fused gate/up projection: elements 0..63 of the tile are gate values, 64..127 the up values
// of the same outputs, so lane i < 16 finds its up values in lane i + 16.  The arithmetic is that of the stand-alone
// kernel of activation.cu for 16-bit activations, on the 32-bit sums of the product.
__device__ __forceinline__ void silu_finish(const GemmParams& p, int m, int lane, int tile, const float (&value)[4]) {
    constexpr int kHalf = kBlockRows / 2;
    float result[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float up = __shfl_xor_sync(0xffffffffu, value[c], 16);
        result[c] = __fdividef(value[c], 1.0f + __expf(-value[c])) * up;
    }
    if (lane < 16) {
        const int column = tile * kHalf + 4 * lane;
        store4_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldc + column, result, p.n / 2 - column, p.vector_out != 0);
    }
}

// Token m of a product that is added to the residual stream: columns n4 .. n4 + 3; `before`: the stream's values
// there, `weight`: the next norm's weights of those columns.
__device__ __forceinline__ void stream_finish(const GemmParams& p, int m, int lane, int tile, int n4, const float (&value)[4],
                                              const float (&before)[4], const float (&weight)[4]) {
    const StreamEpilogue& e = p.stream;
    const int valid = p.n - n4;       // <= 0: this lane's columns lie outside the matrix
    float updated[4], scaled[4], squares = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        updated[c] = c < valid ? before[c] + value[c] : 0.0f;
        scaled[c] = updated[c] * weight[c];
        squares += updated[c] * updated[c];
    }
    if (valid > 0) {
        store4_f32(e.residual + (size_t)m * p.n + n4, updated, valid, p.vector_stream != 0);
        if (e.next_weight != nullptr) store4_bf16(e.scaled + (size_t)m * p.n + n4, scaled, valid, p.vector_stream != 0);
    }
    if (e.next_weight != nullptr) {
        squares = warp_sum(squares);
        if (lane == 0) e.parts[(size_t)tile * e.stride + m] = squares;
    }
}

__global__ void __launch_bounds__(kThreads) gemm_small_m_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                const GemmParams p) {
    // Static shared memory has to stay within 1 KiB.  Up to 16 tokens a block takes 72 KiB of stages + 1 KiB to align
    // them + this + 1 KiB that the system reserves = 75 KiB, and three blocks share an SM (225 of 227 KiB): two of this
    // kernel and one of the next, whose weights are then on their way while this kernel still runs.  With 2 KiB more
    // only two fit: a decode step of the 8B shape then took 4.23 ms instead of 3.67.
    extern __shared__ __align__(1024) unsigned char shared_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t accum_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    __shared__ float row_scale[64];                 // RowScale: 1 / rms of each token's stream row

    // the dynamic region is aligned to 1024 bytes by hand (the swizzle atoms need it)
    const uint32_t raw = smem_u32(shared_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* aligned = shared_raw + (base - raw);
    const uint32_t a_bytes = kBlockRows * kAtomK * 2;                 // 16 KiB per atom of W
    const uint32_t b_bytes = (uint32_t)p.token_pad * kAtomK * 2;      // 2..8 KiB per atom of tokens
    const uint32_t b_pitch = (b_bytes + 1023u) & ~1023u;
    const uint32_t b_offset = kAtoms * a_bytes;                       // token atoms follow the W atoms of a stage
    const uint32_t stage_bytes = b_offset + kAtoms * b_pitch;

    pdl_trigger();   // let the next kernel start launching
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const uint32_t rank = p.split > 1 ? cluster_rank() : 0;
    const int tile = blockIdx.x / p.split;
    const int n0 = tile * kBlockRows;
    const int total_kb = (p.k + kBlockK - 1) / kBlockK;
    const int kb_begin = (int)((long long)total_kb * rank / p.split);
    const int kb_end = (int)((long long)total_kb * (rank + 1) / p.split);
    const int n_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&accum_bar), 1);
        tma::mbar_fence_init();
        // The weights do not depend on the kernel before this one: the W tiles of the first ring of stages are
        // requested at once, before the block has even met at its first barrier and long before pdl_wait().
        const int first = n_kb < p.stages ? n_kb : p.stages;
        for (int i = 0; i < first; ++i) {
            const uint32_t bar = smem_u32(&full_bar[i]);
            mbar_expect_tx(bar, kAtoms * (a_bytes + b_bytes));
#pragma unroll
            for (int atom = 0; atom < kAtoms; ++atom)
                tma_load_2d(base + i * stage_bytes + atom * a_bytes, &map_w, bar, (kb_begin + i) * kBlockK + atom * kAtomK, n0);
        }
    }
    if (warp == 1) {   // this warp owns the tensor-memory allocation (64 columns: up to 64 token columns of float)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(64));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA copies of the W tile and the token tile of each K block.  The W tiles of the first
        // ring are on their way already (see above); the token tiles, which the kernel before this one may just
        // have written, follow after pdl_wait().
        const int first = n_kb < p.stages ? n_kb : p.stages;
        pdl_wait();
        for (int i = 0; i < first; ++i)
#pragma unroll
            for (int atom = 0; atom < kAtoms; ++atom)
                tma_load_2d(base + i * stage_bytes + b_offset + atom * b_pitch, &map_x, smem_u32(&full_bar[i]),
                            (kb_begin + i) * kBlockK + atom * kAtomK, 0);
        for (int i = first; i < n_kb; ++i) {
            const int s = i % p.stages;
            if (!mbar_wait(smem_u32(&empty_bar[s]), ((i / p.stages) - 1) & 1)) {
                failed = 1;
                break;
            }
            const uint32_t stage = base + s * stage_bytes;
            const uint32_t bar = smem_u32(&full_bar[s]);
            mbar_expect_tx(bar, kAtoms * (a_bytes + b_bytes));
#pragma unroll
            for (int atom = 0; atom < kAtoms; ++atom) {
                tma_load_2d(stage + atom * a_bytes, &map_w, bar, (kb_begin + i) * kBlockK + atom * kAtomK, n0);
                tma_load_2d(stage + b_offset + atom * b_pitch, &map_x, bar, (kb_begin + i) * kBlockK + atom * kAtomK, 0);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        const uint32_t idesc = umma_instruction(kBlockRows, p.token_pad);
        bool ok = true;
        for (int i = 0; i < n_kb && ok; ++i) {
            const int s = i % p.stages;
            if (!mbar_wait(smem_u32(&full_bar[s]), (i / p.stages) & 1)) {
                failed = 1;
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_src = base + s * stage_bytes, b_src = a_src + b_offset;
#pragma unroll
            for (int atom = 0; atom < kAtoms; ++atom) {
                const uint64_t desc_a = umma_descriptor(a_src + atom * a_bytes), desc_b = umma_descriptor(b_src + atom * b_pitch);
#pragma unroll
                for (int k = 0; k < kAtomK / 16; ++k)   // 16 bfloat16 = 32 bytes further along the swizzled row
                    umma_bf16(tmem_base, desc_a + (uint64_t)(k * 2), desc_b + (uint64_t)(k * 2), idesc,
                              (i > 0 || atom > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&empty_bar[s]));     // the stage is free once these MMAs have read it
        }
        umma_commit(smem_u32(&accum_bar));            // the accumulator is complete once all MMAs are done
    } else if (warp >= 2 && p.scale.parts != nullptr) {
        // ---- the two warps without a role in the main loop add the sums of squares, in an order that depends on
        // the number of parts only, and leave 1 / rms per token for the epilogue
        pdl_wait();
        for (int m = warp - 2; m < p.m; m += n_warps - 2) {
            float squares = 0.0f;
            for (int i = lane; i < p.scale.n_parts; i += 32) squares += p.scale.parts[(size_t)i * p.scale.stride + m];
            squares = warp_sum(squares);
            if (lane == 0) row_scale[m] = rsqrtf(squares / (float)p.k + p.scale.eps);
        }
    }

    // ---- epilogue: all warps
    __syncwarp();
    pdl_wait();     // global memory is written below: the kernels before this one must be done with it
    // What the epilogue needs beside the product is asked for now, while the product is still being made: the norm
    // weights and frequencies of this lane's four elements, and for the first token this warp will finish its
    // position and page (a chain of three dependent loads) or the stream's values.
    const int r4 = 4 * lane, n4 = n0 + r4;
    const int token_step = n_warps * p.split;         // between two tokens of one warp (rows are dealt round-robin to
    const int first_token = (int)rank + p.split * warp;   // the ranks, a rank's rows round-robin to its warps)
    float weight[4] = {1.0f, 1.0f, 1.0f, 1.0f}, frequency[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    RopeRow info;
    float before[4];
    if (p.rope.on) {
        const bool is_q = tile < p.rope.n_q_heads, is_k = !is_q && tile < p.rope.n_q_heads + p.rope.n_kv_heads;
        if (is_q || is_k) {
            load_weights4(is_q ? p.rope.q_weight : p.rope.k_weight, p.rope.weight_is_f32, r4, kBlockRows, weight);
            if (p.rope.inv_freq != nullptr) {
#pragma unroll
                for (int c = 0; c < 4; ++c) frequency[c] = p.rope.inv_freq[(r4 + c) & (kBlockRows / 2 - 1)];
            }
        }
    } else if (p.stream.on) {
        load_weights4(p.stream.next_weight, p.stream.weight_is_f32, n4, p.n, weight);
    }
    token_inputs(p, first_token, tile, n4, info, before);
    bool ready = true;
    if (n_kb > 0) ready = mbar_wait(smem_u32(&accum_bar), 0);
    if (!ready) failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();            // every copy has landed and every MMA retired (or the wait ran out)
    const bool bad = failed != 0;
    if (bad) {
        // a wait ran out: report it, give copies that may still be in flight time to land, then leave in order
        if (threadIdx.x == 0) atomicExch(p.error_flag, 2);
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }

    // The tile of sums goes from tensor memory (lane = row of W, column = token) into shared memory as
    // [token][128 rows], over the stages, which nobody reads any more; with K split, every rank's part lies in its own
    // shared memory then.
    // warp w reads tensor-memory lanes 32 (w mod 4) .. + 31 = rows of the tile; warps 0-3 and 4-7 take turns with the
    // groups of 16 tokens
    const int row = (warp & 3) * 32 + lane;
    float* parts_tile = reinterpret_cast<float*>(aligned);
    for (int c0 = (warp >> 2) * 16; c0 < p.token_pad; c0 += 4 * n_warps) {
        if (c0 >= p.m) break;
        float values[16];
        if (n_kb > 0 && !bad) {
            tmem_load_16(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)c0, values);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) values[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) parts_tile[(c0 + i) * kBlockRows + row] = values[i];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (p.split > 1) cluster_sync();
    else __syncthreads();
    // every warp has read its part of the tensor memory (each load waited for its data before the barrier): it is
    // given back now, so that nothing but the rows' results stands between a warp and its exit
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(64));
    }

    // Lane i finishes elements 4 i .. 4 i + 3 of the tile for its warp's tokens, one token after the other.
    const bool scaled = p.scale.parts != nullptr;
    const uint32_t parts_address = smem_u32(parts_tile);
    bool arrived = false;
    for (int m = first_token; m < p.m; m += token_step) {
        if (m != first_token) token_inputs(p, m, tile, n4, info, before);
        // the ranks' parts of the token, all asked for before the first is used, added in the order of the ranks
        float4 parts[kMaxSplit];
#pragma unroll
        for (int peer = 0; peer < kMaxSplit; ++peer) {
            if (peer >= p.split) {
                parts[peer] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            } else if (p.split > 1) {
                parts[peer] = load_peer4(parts_address + (uint32_t)(m * kBlockRows + r4) * 4u, (uint32_t)peer);
            } else {
                parts[peer] = *reinterpret_cast<const float4*>(parts_tile + m * kBlockRows + r4);
            }
        }
        float total[4] = {parts[0].x, parts[0].y, parts[0].z, parts[0].w};
#pragma unroll
        for (int peer = 1; peer < kMaxSplit; ++peer) {      // absent peers add 0
            total[0] += parts[peer].x;
            total[1] += parts[peer].y;
            total[2] += parts[peer].z;
            total[3] += parts[peer].w;
        }
        if (p.split > 1 && m + token_step >= p.m) {      // this warp's last token: its parts are here (they were added)
            cluster_arrive();
            arrived = true;
        }
        if (scaled) {
            const float s = row_scale[m];
#pragma unroll
            for (int c = 0; c < 4; ++c) total[c] *= s;
        }
        if (p.stream.on) {
            stream_finish(p, m, lane, tile, n4, total, before, weight);
        } else if (p.rope.on) {
            rope_finish(p, m, lane, tile, total, weight, frequency, info);
        } else if (p.silu_gate) {
            silu_finish(p, m, lane, tile, total);
        } else if (n4 < p.n) {
            if (p.out_is_f32) store4_f32(reinterpret_cast<float*>(p.out) + (size_t)m * p.ldc + n4, total, p.n - n4, p.vector_out != 0);
            else store4_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldc + n4, total, p.n - n4, p.vector_out != 0);
        }
    }
    if (p.split > 1) {          // nobody leaves while a peer may still read its shared memory
        if (!arrived) cluster_arrive();
        cluster_wait();
    }
}

// Tensor map of a row-major [rows, k] bfloat16 matrix, box = [box_rows, 64] with 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* pointer, int rows, int k, int box_rows) {
    return tma::make_map_bf16(map, pointer, (uint64_t)rows, (uint64_t)k, (uint32_t)box_rows);   // box of 64 columns
}

}  // namespace

// 1 when the kernel takes the sizes, else 0 (the caller then uses the library product).
LLM_EXPORT int llm_gemm_small_m_supports(int m, int n, int k) {
    return m >= 1 && m <= 64 && n >= 1 && k >= 8 && k % 8 == 0;
}

static RowScale row_scale_of(const float* parts, int n_parts, int stride, float eps) {
    RowScale scale;
    scale.parts = n_parts > 0 ? parts : nullptr;
    scale.n_parts = n_parts;
    scale.stride = stride;
    scale.eps = eps;
    return scale;
}

static int small_m_launch(const void* x, const void* w, void* out, int m, int n, int k, int ldc, int out_is_f32,
                          int requested_split, int* error_flag, const RopeEpilogue* rope, cudaStream_t stream,
                          int silu_gate, const RowScale& scale, const StreamEpilogue* stream_out = nullptr) {
    if (m == 0 || n == 0) return LLM_OK;
    if (!llm_gemm_small_m_supports(m, n, k) || !aligned16(x) || !aligned16(w)) {
        llm_set_error("gemm_small_m: takes 1..64 rows, K a multiple of 8 and 16-byte aligned operands (got m %d, n %d, k %d)", m, n, k);
        return LLM_REFUSED;
    }
    GemmParams p;
    p.out = out;
    p.out_is_f32 = out_is_f32;
    p.m = m;
    p.n = n;
    p.k = k;
    p.ldc = ldc;
    p.token_pad = ((m + 15) / 16) * 16;
    p.error_flag = error_flag;
    if (rope != nullptr) {
        p.rope = *rope;
    } else {
        p.rope = RopeEpilogue{};
        p.rope.on = 0;
    }
    p.silu_gate = silu_gate;
    p.scale = scale;
    if (scale.parts != nullptr && (scale.stride < m || m > 64)) {
        llm_set_error("gemm_small_m: the sums of squares have room for %d tokens, the product has %d", scale.stride, m);
        return LLM_REFUSED;
    }
    if (stream_out != nullptr) {
        p.stream = *stream_out;
    } else {
        p.stream = StreamEpilogue{};
        p.stream.on = 0;
    }
    p.vector_out = out != nullptr && aligned16(out) && ldc % 4 == 0 &&
                   (rope == nullptr || (aligned16(rope->k_pages) && aligned16(rope->v_pages)));
    p.vector_stream = p.stream.on && aligned16(p.stream.residual) && (p.stream.scaled == nullptr || aligned16(p.stream.scaled)) && n % 4 == 0;
    const int tiles = (n + kBlockRows - 1) / kBlockRows;
    const int total_kb = (k + kBlockK - 1) / kBlockK;
    // K is split across a cluster so that the tiles fill the machine; each rank keeps >= 4 K blocks.  The
    // caller may name the split (it times a few once per shape); 0 asks for about one wave of 148 SMs.
    int split = requested_split > 0 ? requested_split : 148 / tiles;
    if (split > total_kb / 2) split = total_kb / 2;
    if (split > kMaxSplit) split = kMaxSplit;
    if (split < 1) split = 1;
    p.split = split;
    const size_t a_bytes = (size_t)kBlockRows * kAtomK * 2;
    const size_t b_bytes = ((size_t)p.token_pad * kAtomK * 2 + 1023) & ~(size_t)1023;
    const size_t stage_bytes = kAtoms * (a_bytes + b_bytes);
    // The ring of stages (about 100 KiB: two CTAs fit on an SM) lets a CTA that was launched early, while the kernels
    // before it still run, request that many bytes of weights before it has to wait for its input.
    static int ring_kib = -1;
    if (ring_kib < 0) {
        const char* value = getenv("LLMSERVER_B200_GEMM_RING_KIB");
        ring_kib = value ? atoi(value) : 100;
        if (ring_kib < 32) ring_kib = 32;
        if (ring_kib > 200) ring_kib = 200;
    }
    int stages = (int)(((size_t)ring_kib * 1024) / stage_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    const int my_kb = (total_kb + split - 1) / split;
    if (stages > my_kb) stages = my_kb < 1 ? 1 : my_kb;
    p.stages = stages;
    size_t shared = (size_t)stages * stage_bytes;
    const size_t reduce_bytes = (size_t)p.token_pad * kBlockRows * sizeof(float);
    if (shared < reduce_bytes) shared = reduce_bytes;
    shared += 1024;   // room to align the region to 1024 bytes

    CUtensorMap map_w, map_x;
    if (!make_map(&map_w, w, n, k, kBlockRows) || !make_map(&map_x, x, m, k, p.token_pad)) {
        llm_set_error("gemm_small_m: cuTensorMapEncodeTiled failed (m %d, n %d, k %d)", m, n, k);
        return LLM_REFUSED;
    }
    if (int limit_status = llm_raise_shared_limit(reinterpret_cast<const void*>(gemm_small_m_kernel), (size_t)226 * 1024, "gemm_small_m")) return limit_status;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(tiles * split), 1, 1);
    config.blockDim = dim3(m > 16 ? kThreads : kThreads / 2, 1, 1);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    int count = 0;
    if (llm_pdl_enabled()) {
        attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    if (split > 1) {
        attribute[count].id = cudaLaunchAttributeClusterDimension;
        attribute[count].val.clusterDim.x = (unsigned)split;
        attribute[count].val.clusterDim.y = 1;
        attribute[count].val.clusterDim.z = 1;
        ++count;
    }
    config.attrs = attribute;
    config.numAttrs = count;
    cudaError_t status = cudaLaunchKernelEx(&config, gemm_small_m_kernel, map_w, map_x, p);
    if (status != cudaSuccess) {
        llm_set_error("gemm_small_m launch: %s", cudaGetErrorString(status));
        return (int)status;
    }
    return llm_check_launch("gemm_small_m");
}

// scale_parts .. scale_eps: the RowScale of the input rows (scale_n_parts 0: none), here and in the products below.
LLM_EXPORT int llm_gemm_small_m(const void* x, const void* w, void* out, int m, int n, int k, int ldc, int out_is_f32,
                                int requested_split, const float* scale_parts, int scale_n_parts, int scale_stride,
                                float scale_eps, int* error_flag, cudaStream_t stream) {
    return small_m_launch(x, w, out, m, n, k, ldc, out_is_f32, requested_split, error_flag, nullptr, stream, 0,
                          row_scale_of(scale_parts, scale_n_parts, scale_stride, scale_eps));
}

// How many partial sums of squares per token llm_gemm_into_stream leaves for a stream of n columns.
LLM_EXPORT int llm_gemm_into_stream_parts(int n) { return (n + kBlockRows - 1) / kBlockRows; }

// residual[m, n] += x[m, k] W^T (32-bit stream, contiguous).  With next_weight [n] (bfloat16, or float when
// weight_is_f32): scaled[m, n] = bfloat16(residual * next_weight) and parts[i * parts_stride + token], i <
// llm_gemm_into_stream_parts(n), the partial sums of squares of the updated rows: the input and the RowScale of the
// product that consumes the RMSNorm with that weight.  Without next_weight only the stream is updated.
LLM_EXPORT int llm_gemm_into_stream(const void* x, const void* w, float* residual, int m, int n, int k, int requested_split,
                                    const void* next_weight, int weight_is_f32, void* scaled, float* parts, int parts_stride,
                                    int* error_flag, cudaStream_t stream) {
    if (residual == nullptr || (next_weight != nullptr && (scaled == nullptr || parts == nullptr || parts_stride < m))) {
        llm_set_error("gemm_into_stream: the stream, and with a norm weight its two outputs (room for %d tokens), must be given", m);
        return LLM_REFUSED;
    }
    StreamEpilogue e;
    e.on = 1;
    e.residual = residual;
    e.next_weight = next_weight;
    e.weight_is_f32 = weight_is_f32;
    e.scaled = (__nv_bfloat16*)scaled;
    e.parts = parts;
    e.stride = parts_stride;
    return small_m_launch(x, w, nullptr, m, n, k, n, 1, requested_split, error_flag, nullptr, stream, 0,
                          row_scale_of(nullptr, 0, 0, 0.0f), &e);
}

// 1 when the fused q/k/v projection takes the sizes: heads of 128 (a head is a tile of the product), up to 64 tokens
// (each costs a block-wide reduction in the epilogue of the block that finishes it: with many tokens the caller
// measures whether the fused form still wins), and what llm_gemm_small_m itself needs.
LLM_EXPORT int llm_gemm_qkv_rope_supports(int m, int n_q_heads, int n_kv_heads, int head_dim, int k) {
    return head_dim == kBlockRows && m >= 1 && m <= 64 && n_q_heads >= 1 && n_kv_heads >= 1 &&
           llm_gemm_small_m_supports(m, (n_q_heads + 2 * n_kv_heads) * head_dim, k);
}

// qkv[m, (Hq + 2 Hkv) 128] = x[m, k] W^T with the epilogue of RopeEpilogue: Q heads normalised, rotated and written
// to `qkv` (bfloat16, row pitch ldc); K heads normalised, rotated and written to the K pages, V heads to the V pages
// (when write_cache is set), nothing of K and V to `qkv`.  Arguments as llm_qk_norm_rope_kv_write and
// llm_gemm_small_m; the whole head rotates, paired as halves.
LLM_EXPORT int llm_gemm_qkv_rope(const void* x, const void* w, void* qkv, int m, int k, int ldc, int requested_split,
                                 const void* q_weight, const void* k_weight, int weight_is_f32, const float* inv_freq,
                                 const int* positions, const int* seq_of_token, const int* block_tables, int max_blocks,
                                 void* k_pages, void* v_pages, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                 int num_pages, float eps, int write_cache, int* page_error, const float* scale_parts,
                                 int scale_n_parts, int scale_stride, float scale_eps, int* error_flag,
                                 cudaStream_t stream) {
    if (!llm_gemm_qkv_rope_supports(m, n_q_heads, n_kv_heads, head_dim, k)) {
        llm_set_error("gemm_qkv_rope: takes heads of 128 and 1..64 tokens (got head_dim %d, m %d, k %d)", head_dim, m, k);
        return LLM_REFUSED;
    }
    if (positions == nullptr || seq_of_token == nullptr || block_tables == nullptr || page_error == nullptr ||
        (write_cache && (k_pages == nullptr || v_pages == nullptr)) || page_size <= 0 || num_pages <= 0) {
        llm_set_error("gemm_qkv_rope: positions, tables, pages and the error flag must be given");
        return LLM_REFUSED;
    }
    RopeEpilogue rope;
    rope.on = 1;
    rope.q_weight = q_weight;
    rope.k_weight = k_weight;
    rope.weight_is_f32 = weight_is_f32;
    rope.inv_freq = inv_freq;
    rope.positions = positions;
    rope.seq_of_token = seq_of_token;
    rope.block_tables = block_tables;
    rope.max_blocks = max_blocks;
    rope.k_pages = (__nv_bfloat16*)k_pages;
    rope.v_pages = (__nv_bfloat16*)v_pages;
    rope.n_q_heads = n_q_heads;
    rope.n_kv_heads = n_kv_heads;
    rope.page_size = page_size;
    rope.num_pages = num_pages;
    rope.eps = eps;
    rope.write_cache = write_cache;
    rope.page_error = page_error;
    return small_m_launch(x, w, qkv, m, (n_q_heads + 2 * n_kv_heads) * head_dim, k, ldc, 0, requested_split, error_flag, &rope, stream,
                          0, row_scale_of(scale_parts, scale_n_parts, scale_stride, scale_eps));
}

// out[m, n / 2] = silu(gate) * up of the fused gate/up projection x W^T, W [n, k] with gate and up rows interleaved in
// groups of 64 (rows [128 b, 128 b + 64) are gate rows of outputs [64 b, 64 b + 64), the next 64 rows their up rows);
// n must be a multiple of 128.  bfloat16 in and out; ldc is the row pitch of `out`.
LLM_EXPORT int llm_gemm_gate_up_silu(const void* x, const void* w, void* out, int m, int n, int k, int ldc,
                                     int requested_split, const float* scale_parts, int scale_n_parts, int scale_stride,
                                     float scale_eps, int* error_flag, cudaStream_t stream) {
    if (n % kBlockRows) {
        llm_set_error("gemm_gate_up_silu: %d rows of the fused weight are no multiple of %d", n, kBlockRows);
        return LLM_REFUSED;
    }
    return small_m_launch(x, w, out, m, n, k, ldc, 0, requested_split, error_flag, nullptr, stream, 1,
                          row_scale_of(scale_parts, scale_n_parts, scale_stride, scale_eps));
}
