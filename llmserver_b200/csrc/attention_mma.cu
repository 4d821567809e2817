// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, 32-bit accumulation
// and 32-bit online softmax), for head sizes 64 and 128, any number of heads and groups, any page size.
//
// Two kernels share one warp-level tile routine:
//
//   * portions (q_len > 1): one block per (sequence, kv head, 64-row tile).  "Rows" are (token, head of
//     the group) pairs of one kv head, so the G query heads that share a kv head also share every K/V
//     tile the block loads.  Four warps take 16 rows each and walk the sequence's keys in tiles of 64,
//     from the first key the tile's window can see to the last token's own position (causal).
//   * decode (q_len == 1): one block per (split of the keys, kv head, sequence).  The G heads are the
//     rows (padded to 16); the four warps take 16 keys each of every 64-key tile, then merge.  With more
//     than one split per sequence the splits' results are merged (split-KV, as the reference's paged
//     decode: utils/paged_attention.py:168-237): up to 8 splits form a thread-block cluster and merge
//     through distributed shared memory inside the TMA kernel; otherwise they go to scratch memory and a
//     second kernel merges them.  Both add the splits in the same order with the same arithmetic.
//
// K and V tiles travel global -> shared with cp.async (16-byte chunks, two stages), each key's page
// looked up in the block table, so a page size is only a divisor here.  Shared tiles are XOR-swizzled by
// 16-byte chunk so that ldmatrix reads are conflict-free.  Scores are S = Q K^T * scale with keys after
// the query's position (and, with a window, keys at or before position - window) masked; softmax and
// the P V sum follow utils/attention.py:186-198 with the running-max recurrence of
// utils/attention.py:75-96.  Probabilities are rounded to bfloat16 for the P V product; the normaliser
// is summed in 32-bit from the unrounded values.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
#include <stdlib.h>
#include <type_traits>

namespace {

constexpr int kThreads = 128;
constexpr int kTileKeys = 64;
constexpr int kTileRows = 64;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
    const __nv_bfloat16* q;
    int q_stride;
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    const int* block_tables;
    int max_blocks;
    int num_pages;           // pages in the pool: block-table entries outside 0 .. num_pages - 1 are not followed
    const int* q_start;      // [S + 1]
    const int* context_len;  // [S]
    __nv_bfloat16* out;      // [N, Hq * D]
    int n_seqs, n_q_heads, n_kv_heads, page_size;
    float scale_log2;
    int window;
    int skip_single;         // portions kernel: leave sequences with one token to the decode kernel
    int split_len;           // decode kernel: keys per split (multiple of 64); negative: -split_len equal parts per sequence
    int max_splits;
    float* partial_out;      // [N, Hq, max_splits, D]
    float* partial_ml;       // [N, Hq, max_splits, 2]
    int old_keys_settled;    // TMA decode kernel: every key but each sequence's newest was written before the kernel in
                             // front of this one started (by an earlier step), so their copies need not wait for it
    int cluster_merge;       // TMA decode kernel: the splits of a sequence form a thread-block cluster and merge their
                             // partial results through distributed shared memory (no scratch, no merge kernel)
    int slot_by_seq;         // scratch slots are counted by sequence instead of by the sequence's token index
    int* error_flag;         // 3: a bounded wait of the TMA decode kernel ran out; 5: a block-table entry names no page
                             // of the pool; 6: a context needs more splits than max_splits (may be null)
};

// A block-table entry as the kernels may follow it: an entry that names no page of the pool is reported and replaced
// by page 0, so nothing outside the pool is ever addressed (the keys it stands for are wrong, and the flag says so).
__device__ __forceinline__ int checked_page(const AttnParams& p, int page) {
    if ((unsigned)page < (unsigned)p.num_pages) return page;
    if (p.error_flag) atomicExch(p.error_flag, 5);
    return 0;
}

// Keys per split of a sequence that sees `span` keys: the fixed length, or (split_len < 0) the span divided into
// -split_len equal parts, in whole tiles and no shorter than three tiles.  With equal parts every sequence of a
// batch gets the same number of blocks, all about equally long, whatever its length: the launch shape of a captured
// graph (sized for the longest context it may meet) then fits shorter contexts as well.
__device__ __forceinline__ int split_length(const AttnParams& p, int span) {
    if (p.split_len > 0) return p.split_len;
    const int parts = -p.split_len;
    const int length = ((span + parts - 1) / parts + kTileKeys - 1) / kTileKeys * kTileKeys;
    return length < 3 * kTileKeys ? 3 * kTileKeys : length;
}

__device__ __forceinline__ uint32_t smem_address(const void* pointer) {
    return (uint32_t)__cvta_generic_to_shared(pointer);
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(address));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float low, float high) {
    __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<uint32_t*>(&pair);
}

// Thread-block cluster: a barrier over the threads of the cluster that have not exited, and a load from the shared
// memory of another block of the cluster.
__device__ __forceinline__ void cluster_arrive_wait() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The two halves on their own: a thread arrives as soon as it has read what it needs of the other blocks' shared
// memory and waits for the others only before it leaves.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ float2 load_cluster2(uint32_t local_address, uint32_t rank) {
    uint32_t remote;
    float2 value;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(value.x), "=f"(value.y) : "r"(remote) : "memory");
    return value;
}
__device__ __forceinline__ float load_cluster(uint32_t local_address, uint32_t rank) {
    uint32_t remote;
    float value;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(remote) : "memory");
    return value;
}

// Element offset of (row, 16-byte chunk) in a swizzled tile whose rows hold D bfloat16.
template <int D>
__device__ __forceinline__ int swizzled(int row, int chunk) {
    return row * D + ((chunk ^ (row & 7)) << 3);
}

// The two shared-memory tile layouts.  XorLayout: rows of D elements, chunks XOR-ed with the row (tiles
// filled by cp.async).  TmaLayout: what TMA writes with 128-byte swizzle: the tile is split into column
// halves of 64 elements, each half holds ROWS rows of 128 bytes whose 16-byte chunks are XOR-ed with the row.
template <int D>
struct XorLayout {
    static __device__ __forceinline__ int at(int row, int chunk) { return swizzled<D>(row, chunk); }
};
template <int D, int ROWS>
struct TmaLayout {
    static __device__ __forceinline__ int at(int row, int chunk) {
        return (chunk >> 3) * (ROWS * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
    }
};
// PageLayout (head_dim 128): what one 5-D TMA box per cache page writes: groups of 8 keys, each group holding its low
// 64 columns and then its high 64 columns as 1024-byte swizzle atoms (half as many, twice as large copies as two
// boxes per page).
struct PageLayout {
    static __device__ __forceinline__ int at(int row, int chunk) {
        return (row >> 3) * 1024 + (chunk >> 3) * 512 + (row & 7) * 64 + (((chunk & 7) ^ (row & 7)) << 3);
    }
};

// Loads rows [first_key, first_key + 64) of one kv head into a swizzled shared tile; keys at or past
// `end_key` are zero-filled.  All 128 threads take part.
template <int D>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* k_tile, __nv_bfloat16* v_tile, const AttnParams& p,
                                             const int* table, int kv_head, int first_key, int end_key) {
    constexpr int kChunks = D / 8;                        // 16-byte chunks per row
    constexpr int kPerThread = kTileKeys * kChunks / kThreads;
    constexpr int kRowsPerPass = kThreads / kChunks;
    const int chunk = threadIdx.x % kChunks;
    const int row0 = threadIdx.x / kChunks;
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
        const int row = row0 + i * kRowsPerPass;
        const int key = first_key + row;
        const bool valid = key < end_key;
        size_t offset = 0;
        if (valid) {
            const int page = checked_page(p, table[key / p.page_size]);
            offset = (((size_t)page * p.n_kv_heads + kv_head) * p.page_size + key % p.page_size) * D + chunk * 8;
        }
        const int destination = swizzled<D>(row, chunk);
        cp_async_16(smem_address(k_tile + destination), p.k_pages + offset, valid ? 16 : 0);
        cp_async_16(smem_address(v_tile + destination), p.v_pages + offset, valid ? 16 : 0);
    }
}

// One warp: 16 query rows against NT * 8 keys of a shared tile, starting at tile row `key_row`, whose
// absolute key index is `key_index`.  Rows g = lane / 4 and g + 8 of the warp see keys in
// [row_low[h], row_high[h]] (row_high < 0: the row does not exist).
template <int D, int NT, class Layout = XorLayout<D>>
__device__ __forceinline__ void warp_tile(const uint32_t (&q_frag)[D / 16][4], const __nv_bfloat16* k_tile,
                                          const __nv_bfloat16* v_tile, int key_row, int key_index,
                                          const int (&row_low)[2], const int (&row_high)[2], float scale_log2,
                                          float (&o_acc)[D / 8][4], float (&row_max)[2], float (&row_sum)[2]) {
    const int lane = threadIdx.x & 31;
    const int matrix = lane >> 3, matrix_row = lane & 7;
    float s_acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s_acc[n][i] = 0.0f;

    // S = Q K^T
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int pair = 0; pair < NT / 2; ++pair) {
            uint32_t b[4];
            const int row = key_row + pair * 16 + (matrix >> 1) * 8 + matrix_row;
            ldmatrix_x4(b, smem_address(k_tile + Layout::at(row, 2 * ks + (matrix & 1))));
            mma_bf16(s_acc[2 * pair], q_frag[ks], b[0], b[1]);
            mma_bf16(s_acc[2 * pair + 1], q_frag[ks], b[2], b[3]);
        }
    }

    // mask, scale, running maximum
    const int t = lane & 3;
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = i >> 1;
            const int key = key_index + n * 8 + 2 * t + (i & 1);
            const bool seen = key >= row_low[h] && key <= row_high[h];
            s_acc[n][i] = seen ? s_acc[n][i] * scale_log2 : -INFINITY;
            tile_max[h] = fmaxf(tile_max[h], s_acc[n][i]);
        }
    }
    float correction[2], reference[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
        tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
        const float new_max = fmaxf(row_max[h], tile_max[h]);
        reference[h] = new_max == -INFINITY ? 0.0f : new_max;   // nothing seen yet: exp2(-inf - 0) = 0
        correction[h] = exp2f(row_max[h] - reference[h]);
        row_max[h] = new_max;
        row_sum[h] *= correction[h];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        o_acc[n][0] *= correction[0];
        o_acc[n][1] *= correction[0];
        o_acc[n][2] *= correction[1];
        o_acc[n][3] *= correction[1];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = i >> 1;
            s_acc[n][i] = exp2f(s_acc[n][i] - reference[h]);
            row_sum[h] += s_acc[n][i];
        }
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
        a[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
        a[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
        a[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
            uint32_t b[4];
            const int row = key_row + kk * 16 + (matrix & 1) * 8 + matrix_row;
            ldmatrix_x4_trans(b, smem_address(v_tile + Layout::at(row, 2 * j + (matrix >> 1))));
            mma_bf16(o_acc[2 * j], a, b[0], b[1]);
            mma_bf16(o_acc[2 * j + 1], a, b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// portions of prompts
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads) attention_portions_kernel(const AttnParams p) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    extern __shared__ __align__(16) unsigned char shared_raw[];
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(shared_raw);   // [64][D]
    __nv_bfloat16* kv_tiles = q_tile + kTileRows * D;                        // [2 stages][K, V][64][D]

    const int group = p.n_q_heads / p.n_kv_heads;
    const int kv_head = blockIdx.y;
    // which sequence and which of its row tiles this block has
    int seq = 0, tile = blockIdx.x;
    for (; seq < p.n_seqs; ++seq) {
        const int q_len = p.q_start[seq + 1] - p.q_start[seq];
        const int tiles = (q_len == 1 && p.skip_single) ? 0 : (q_len * group + kTileRows - 1) / kTileRows;
        if (tile < tiles) {
            tile = tiles - 1 - tile;   // later tiles see more keys: start the long ones first
            break;
        }
        tile -= tiles;
    }
    if (seq >= p.n_seqs) return;
    const int token0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - token0;
    const int context = p.context_len[seq];
    const int n_rows = q_len * group;
    const int first_row = tile * kTileRows;
    const int* table = p.block_tables + (size_t)seq * p.max_blocks;

    // gather the Q rows of the tile: row r is token r / group, head kv_head * group + r % group
    {
        constexpr int kChunks = D / 8;
        for (int c = threadIdx.x; c < kTileRows * kChunks; c += kThreads) {
            const int row = c / kChunks, chunk = c % kChunks;
            const int r = first_row + row;
            const bool valid = r < n_rows;
            const __nv_bfloat16* src = p.q;
            if (valid)
                src = p.q + (size_t)(token0 + r / group) * p.q_stride + (size_t)(kv_head * group + r % group) * D + chunk * 8;
            cp_async_16(smem_address(q_tile + swizzled<D>(row, chunk)), src, valid ? 16 : 0);
        }
    }
    // key range of the tile: from the first token's window start to the last token's position
    const int first_token = first_row / group;
    const int last_row = min(first_row + kTileRows, n_rows) - 1;
    const int last_token = last_row / group;
    const int base_position = context - q_len;
    const int high_key = base_position + last_token;
    int low_key = 0;
    if (p.window > 0) low_key = max(0, base_position + first_token - p.window + 1);
    const int first_tile_key = (low_key / kTileKeys) * kTileKeys;
    const int n_tiles = (high_key - first_tile_key) / kTileKeys + 1;

    load_kv_tile<D>(kv_tiles, kv_tiles + kTileKeys * D, p, table, kv_head, first_tile_key, context);
    cp_async_commit();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2;
    int row_low[2], row_high[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = first_row + warp * 16 + g + 8 * h;
        if (r < n_rows) {
            const int position = base_position + r / group;
            row_high[h] = position;
            row_low[h] = p.window > 0 ? max(0, position - p.window + 1) : 0;
        } else {
            row_high[h] = -1;
            row_low[h] = 0;
        }
    }
    float o_acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    uint32_t q_frag[D / 16][4];
    const int warp_high = __reduce_max_sync(0xffffffffu, max(row_high[0], row_high[1]));

    for (int it = 0; it < n_tiles; ++it) {
        const int stage = it & 1;
        __nv_bfloat16* k_tile = kv_tiles + stage * 2 * kTileKeys * D;
        __nv_bfloat16* v_tile = k_tile + kTileKeys * D;
        if (it + 1 < n_tiles) {
            __nv_bfloat16* next_k = kv_tiles + (stage ^ 1) * 2 * kTileKeys * D;
            load_kv_tile<D>(next_k, next_k + kTileKeys * D, p, table, kv_head, first_tile_key + (it + 1) * kTileKeys, context);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
            const int matrix = lane >> 3, matrix_row = lane & 7;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int row = warp * 16 + (matrix & 1) * 8 + matrix_row;
                ldmatrix_x4(q_frag[ks], smem_address(q_tile + swizzled<D>(row, 2 * ks + (matrix >> 1))));
            }
        }
        const int tile_key = first_tile_key + it * kTileKeys;
        // a warp whose rows all end before this tile has nothing to add (the causal upper triangle)
        if (tile_key <= warp_high)
            warp_tile<D, 8>(q_frag, k_tile, v_tile, 0, tile_key, row_low, row_high, p.scale_log2, o_acc, row_max, row_sum);
        __syncthreads();   // the stage is overwritten by the load issued in the next iteration
    }

    // normalise and store: thread holds rows g, g + 8 and columns 8 n + 2 t, + 1
    const int t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float total = row_sum[h];
        total += __shfl_xor_sync(0xffffffffu, total, 1);
        total += __shfl_xor_sync(0xffffffffu, total, 2);
        const int r = first_row + warp * 16 + g + 8 * h;
        if (r >= n_rows) continue;
        const float inverse = 1.0f / total;
        __nv_bfloat16* dst = p.out + (size_t)(token0 + r / group) * p.n_q_heads * D + (size_t)(kv_head * group + r % group) * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const uint32_t packed = pack_bf16(o_acc[n][2 * h] * inverse, o_acc[n][2 * h + 1] * inverse);
            *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = packed;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// decode: one token per sequence, keys split across blocks
// ------------------------------------------------------------------------------------------------
// A decode row whose sequence holds no token (context_len <= 0) has nothing to attend to: its output is zero.
template <int D>
__device__ __forceinline__ void zero_output(const AttnParams& p, int token, int kv_head, int group) {
    for (int index = threadIdx.x; index < group * D; index += blockDim.x)
        p.out[(size_t)token * p.n_q_heads * D + (size_t)(kv_head * group) * D + index] = __float2bfloat16_rn(0.0f);
}

template <int D>
__global__ void __launch_bounds__(kThreads) attention_decode_kernel(const AttnParams p) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    extern __shared__ __align__(16) unsigned char shared_raw[];
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(shared_raw);   // [16][D]
    __nv_bfloat16* kv_tiles = q_tile + 16 * D;                               // [2 stages][K, V][64][D]

    const int seq = blockIdx.z, kv_head = blockIdx.y, split = blockIdx.x;
    const int token = p.q_start[seq];
    if (p.q_start[seq + 1] - token != 1) return;
    const int group = p.n_q_heads / p.n_kv_heads;
    const int context = p.context_len[seq];
    const int position = context - 1;
    const int low_key = p.window > 0 ? max(0, position - p.window + 1) : 0;
    const int first_key = (low_key / kTileKeys) * kTileKeys;
    const int split_len = split_length(p, context - first_key);
    const int n_splits = (context - first_key + split_len - 1) / split_len;
    if (n_splits > p.max_splits && split == 0 && kv_head == 0 && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 6);
    if (context <= 0 && split == 0) zero_output<D>(p, token, kv_head, group);     // nothing to attend to
    if (split >= n_splits) return;
    const int split_begin = first_key + split * split_len;
    const int split_end = min(split_begin + split_len, context);
    const int n_tiles = (split_end - split_begin + kTileKeys - 1) / kTileKeys;
    const int* table = p.block_tables + (size_t)seq * p.max_blocks;

    {
        constexpr int kChunks = D / 8;
        for (int c = threadIdx.x; c < 16 * kChunks; c += kThreads) {
            const int row = c / kChunks, chunk = c % kChunks;
            const bool valid = row < group;
            const __nv_bfloat16* src = p.q;
            if (valid) src = p.q + (size_t)token * p.q_stride + (size_t)(kv_head * group + row) * D + chunk * 8;
            cp_async_16(smem_address(q_tile + swizzled<D>(row, chunk)), src, valid ? 16 : 0);
        }
    }
    load_kv_tile<D>(kv_tiles, kv_tiles + kTileKeys * D, p, table, kv_head, split_begin, split_end);
    cp_async_commit();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2;
    int row_low[2], row_high[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const bool exists = g + 8 * h < group;
        row_high[h] = exists ? position : -1;
        row_low[h] = low_key;
    }
    float o_acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    uint32_t q_frag[D / 16][4];

    for (int it = 0; it < n_tiles; ++it) {
        const int stage = it & 1;
        __nv_bfloat16* k_tile = kv_tiles + stage * 2 * kTileKeys * D;
        __nv_bfloat16* v_tile = k_tile + kTileKeys * D;
        if (it + 1 < n_tiles) {
            __nv_bfloat16* next_k = kv_tiles + (stage ^ 1) * 2 * kTileKeys * D;
            load_kv_tile<D>(next_k, next_k + kTileKeys * D, p, table, kv_head, split_begin + (it + 1) * kTileKeys, split_end);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
            const int matrix = lane >> 3, matrix_row = lane & 7;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int row = (matrix & 1) * 8 + matrix_row;
                ldmatrix_x4(q_frag[ks], smem_address(q_tile + swizzled<D>(row, 2 * ks + (matrix >> 1))));
            }
        }
        // each warp takes 16 of the tile's 64 keys
        const int key_index = split_begin + it * kTileKeys + warp * 16;
        if (key_index < split_end)
            warp_tile<D, 2>(q_frag, k_tile, v_tile, warp * 16, key_index, row_low, row_high, p.scale_log2, o_acc, row_max, row_sum);
        __syncthreads();
    }

    // merge the four warps through shared memory (the K/V stages are free now)
    float* merge = reinterpret_cast<float*>(kv_tiles);        // [4 warps][16 rows][D + 2]
    const int t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float total = row_sum[h];
        total += __shfl_xor_sync(0xffffffffu, total, 1);
        total += __shfl_xor_sync(0xffffffffu, total, 2);
        float* row = merge + ((size_t)warp * 16 + g + 8 * h) * (D + 2);
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            row[n * 8 + 2 * t] = o_acc[n][2 * h];
            row[n * 8 + 2 * t + 1] = o_acc[n][2 * h + 1];
        }
        if (t == 0) {
            row[D] = row_max[h];
            row[D + 1] = total;
        }
    }
    __syncthreads();
    for (int index = threadIdx.x; index < group * D; index += kThreads) {
        const int r = index / D, d = index % D;
        float best = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) best = fmaxf(best, merge[((size_t)w * 16 + r) * (D + 2) + D]);
        float numerator = 0.0f, denominator = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* row = merge + ((size_t)w * 16 + r) * (D + 2);
            const float weight = row[D] == -INFINITY ? 0.0f : exp2f(row[D] - best);
            numerator += row[d] * weight;
            denominator += row[D + 1] * weight;
        }
        const int head = kv_head * group + r;
        if (n_splits == 1) {
            p.out[(size_t)token * p.n_q_heads * D + (size_t)head * D + d] = __float2bfloat16_rn(numerator / denominator);
        } else {
            const size_t slot = ((size_t)(p.slot_by_seq ? seq : token) * p.n_q_heads + head) * p.max_splits + split;
            p.partial_out[slot * D + d] = numerator / denominator;
            if (d == 0) {
                p.partial_ml[slot * 2] = best;
                p.partial_ml[slot * 2 + 1] = denominator;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// decode with TMA: the same split-KV kernel, but K and V travel page by page as TMA tiles
// (cp.async.bulk.tensor, 128-byte swizzle) into a ring of kDecodeStages stages, each completion counted
// by an mbarrier.  One elected thread issues a 64-key tile as (64 / page_size) pages x (D / 64) column
// halves x {K, V} copies of page_size x 128 bytes; no thread computes addresses per 16 bytes.  Needs a
// page size of 8, 16, 32 or 64 tokens (whole pages per tile, whole swizzle atoms per page).
// ------------------------------------------------------------------------------------------------
constexpr int kDecodeStages = 3;
constexpr int kDecodeThreads = kThreads + 32;   // four consumer warps and one producer warp

template <int D>
__global__ void __launch_bounds__(kDecodeThreads) attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                              const __grid_constant__ CUtensorMap map_v,
                                                                              const AttnParams p) {
    pdl_trigger();   // let the next kernel start launching
    // Normally everything before this kernel must be complete before it reads anything.  When the caller vouches that
    // only each sequence's newest key is written by the kernel in front (a decode step: older keys come from earlier
    // steps, behind the step's batch copy), the copies of older keys start at once and overlap that kernel's end; Q,
    // the newest key's tile and every write wait.  Each block still waits before it leaves, so that this kernel never
    // completes before the one in front has.
    const bool early = p.old_keys_settled != 0;
    if (!early) pdl_wait();
    extern __shared__ __align__(16) unsigned char shared_raw[];
    __shared__ __align__(8) uint64_t full_bar[kDecodeStages];
    __shared__ __align__(8) uint64_t empty_bar[kDecodeStages];
    __shared__ int failed;
    using Layout = typename std::conditional<D == 128, PageLayout, TmaLayout<D, kTileKeys>>::type;
    constexpr int kHalves = D / 64;
    constexpr uint32_t kTileBytes = kTileKeys * D * 2;          // one of K or V
    constexpr uint32_t kStageBytes = 2 * kTileBytes;

    const uint32_t raw = tma::smem_u32(shared_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // swizzle atoms need 1024-byte alignment
    unsigned char* stages = shared_raw + (base - raw);
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(stages + kDecodeStages * kStageBytes);   // [16][D]

    const int seq = blockIdx.z, kv_head = blockIdx.y, split = blockIdx.x;
    const int token = p.q_start[seq];
    if (p.q_start[seq + 1] - token != 1) {
        if (early) pdl_wait();
        return;
    }
    const int group = p.n_q_heads / p.n_kv_heads;
    const int context = p.context_len[seq];
    const int position = context - 1;
    const int low_key = p.window > 0 ? max(0, position - p.window + 1) : 0;
    const int first_key = (low_key / kTileKeys) * kTileKeys;
    const int split_len = split_length(p, context - first_key);
    const int n_splits = (context - first_key + split_len - 1) / split_len;
    if (n_splits > p.max_splits && split == 0 && kv_head == 0 && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 6);
    if (context <= 0 && split == 0) {       // nothing to attend to
        if (early) pdl_wait();
        zero_output<D>(p, token, kv_head, group);
    }
    // every thread of a cluster whose splits merge in shared memory meets at the same two cluster barriers, also the
    // blocks beyond the sequence's last split and the producer warps, which have nothing to add
    const bool meets_cluster = p.cluster_merge && n_splits > 1;
    if (split >= n_splits) {
        if (early) pdl_wait();
        if (meets_cluster) {
            cluster_arrive_wait();
            cluster_arrive_wait();
        }
        return;
    }
    const int split_begin = first_key + split * split_len;
    const int split_end = min(split_begin + split_len, context);
    const int n_tiles = (split_end - split_begin + kTileKeys - 1) / kTileKeys;
    const int* table = p.block_tables + (size_t)seq * p.max_blocks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < kDecodeStages; ++s) {
            tma::mbar_init(tma::smem_u32(&full_bar[s]), 1);
            tma::mbar_init(tma::smem_u32(&empty_bar[s]), 4);      // one arrival per consumer warp
        }
        tma::mbar_fence_init();
    }
    __syncthreads();

    if (warp == 4) {
        // ---- producer warp.  A tile is (64 / page_size) pages x (D / 64) column halves x {K, V} copies of
        // page_size x 128 bytes; each lane issues one of them.  Every tile is copied whole: pages past the
        // end of the sequence come from whatever the (zero-padded) block table names there, an existing
        // page whose finite contents are masked out, so no row of a stage holds bits that were not loaded.
        // (head_dim 128: one 5-D box per page and operand instead of one per column half)
        constexpr int kBoxesPerPage = D == 128 ? 1 : kHalves;
        const int pages_per_tile = kTileKeys / p.page_size;
        const int copies = pages_per_tile * kBoxesPerPage * 2;
        const int my_page = lane / (kBoxesPerPage * 2), my_half = (lane / 2) % kBoxesPerPage, my_v = lane & 1;
        bool waited = !early;
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t % kDecodeStages;
            // the tile that may hold the sequence's newest key (the last tile of the last split) is written by the
            // kernel in front of this one
            if (!waited && split == n_splits - 1 && t == n_tiles - 1) {
                pdl_wait();
                waited = true;
            }
            bool ok = true;
            if (t >= kDecodeStages) ok = tma::mbar_wait(tma::smem_u32(&empty_bar[s]), ((t / kDecodeStages) - 1) & 1);
            if (!ok) {
                failed = 1;
                break;
            }
            const uint32_t bar = tma::smem_u32(&full_bar[s]);
            if (lane == 0) tma::mbar_expect_tx(bar, 2u * kTileBytes);
            __syncwarp();
            if (lane < copies) {
                const int key = split_begin + t * kTileKeys + my_page * p.page_size;
                // an entry that names no page of the pool lies outside the tensor map's extent and is copied as zeros
                const int page = table[min(key / p.page_size, p.max_blocks - 1)];
                if ((unsigned)page >= (unsigned)p.num_pages && p.error_flag) atomicExch(p.error_flag, 5);
                const int y = (page * p.n_kv_heads + kv_head) * p.page_size;
                if (D == 128) {
                    const uint32_t dst = base + s * kStageBytes + (my_v ? kTileBytes : 0u) + (uint32_t)(my_page * p.page_size) * 256u;
                    tc5::tma_load_5d(dst, my_v ? &map_v : &map_k, bar, 0, 0, 0, 0, page * p.n_kv_heads + kv_head);
                } else {
                    const uint32_t dst = base + s * kStageBytes + (my_v ? kTileBytes : 0u) + my_half * (kTileKeys * 128u) +
                                         (uint32_t)(my_page * p.page_size) * 128u;
                    tma::load_2d(dst, my_v ? &map_v : &map_k, bar, my_half * 64, y);
                }
            }
        }
        if (!waited) pdl_wait();
        if (meets_cluster) {
            cluster_arrive_wait();
            cluster_arrive_wait();
        }
        return;
    }

    // ---- consumer warps: gather Q (plain loads into the XOR layout), then walk the tiles
    if (early) pdl_wait();        // Q comes from the kernel in front
    {
        constexpr int kChunks = D / 8;
        for (int c = threadIdx.x; c < 16 * kChunks; c += kThreads) {
            const int row = c / kChunks, chunk = c % kChunks;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (row < group)
                value = *reinterpret_cast<const uint4*>(p.q + (size_t)token * p.q_stride + (size_t)(kv_head * group + row) * D + chunk * 8);
            *reinterpret_cast<uint4*>(q_tile + swizzled<D>(row, chunk)) = value;
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");     // the four consumer warps only
    const int g = lane >> 2;
    int row_low[2], row_high[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const bool exists = g + 8 * h < group;
        row_high[h] = exists ? position : -1;
        row_low[h] = low_key;
    }
    float o_acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    uint32_t q_frag[D / 16][4];
    {
        const int matrix = lane >> 3, matrix_row = lane & 7;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int row = (matrix & 1) * 8 + matrix_row;
            ldmatrix_x4(q_frag[ks], smem_address(q_tile + swizzled<D>(row, 2 * ks + (matrix >> 1))));
        }
    }

    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
        const int s = it % kDecodeStages;
        if (ok && !tma::mbar_wait(tma::smem_u32(&full_bar[s]), (it / kDecodeStages) & 1)) ok = false;
        const __nv_bfloat16* k_tile = reinterpret_cast<const __nv_bfloat16*>(stages + s * kStageBytes);
        const __nv_bfloat16* v_tile = k_tile + kTileKeys * D;
        const int key_index = split_begin + it * kTileKeys + warp * 16;
        if (key_index < split_end)
            warp_tile<D, 2, Layout>(q_frag, k_tile, v_tile, warp * 16, key_index, row_low, row_high, p.scale_log2, o_acc, row_max, row_sum);
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(tma::smem_u32(&empty_bar[s]));     // this warp is done with the stage
    }
    if (!ok) failed = 1;
    asm volatile("bar.sync 1, 128;" ::: "memory");     // all tiles consumed; the stages can be reused
    if (failed && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 3);

    // merge the four warps through shared memory (every copy has landed: each tile was waited for)
    float* merge = reinterpret_cast<float*>(stages);        // [4 warps][16 rows][D + 2]
    const int t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float total = row_sum[h];
        total += __shfl_xor_sync(0xffffffffu, total, 1);
        total += __shfl_xor_sync(0xffffffffu, total, 2);
        if (g + 8 * h >= group) continue;       // rows beyond the group hold nothing and are not read below
        float* row = merge + ((size_t)warp * 16 + g + 8 * h) * (D + 2);
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<float2*>(row + n * 8 + 2 * t) = make_float2(o_acc[n][2 * h], o_acc[n][2 * h + 1]);
        if (t == 0) {
            row[D] = row_max[h];
            row[D + 1] = total;
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // this split's result per head of the group: [16][D + 2] floats (normalised output, maximum, sum) behind the
    // four warps' rows, for the splits that merge inside a cluster
    float* mine = merge + (size_t)4 * 16 * (D + 2);
    const bool in_cluster = meets_cluster;
    // a warp takes whole heads of the group (their maxima and weights are made once per head, not once per element),
    // a lane two neighbouring elements at a time
    for (int r = warp; r < group; r += 4) {
        float weights[4], best = -INFINITY, denominator = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) best = fmaxf(best, merge[((size_t)w * 16 + r) * (D + 2) + D]);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* row = merge + ((size_t)w * 16 + r) * (D + 2);
            weights[w] = row[D] == -INFINITY ? 0.0f : exp2f(row[D] - best);
            denominator += row[D + 1] * weights[w];
        }
        const int head = kv_head * group + r;
        const size_t slot = ((size_t)(p.slot_by_seq ? seq : token) * p.n_q_heads + head) * p.max_splits + split;
        for (int d = 2 * lane; d < D; d += 64) {
            float numerator[2] = {0.0f, 0.0f};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 pair = *reinterpret_cast<const float2*>(merge + ((size_t)w * 16 + r) * (D + 2) + d);
                numerator[0] += pair.x * weights[w];
                numerator[1] += pair.y * weights[w];
            }
            if (n_splits == 1) {
                *reinterpret_cast<__nv_bfloat162*>(p.out + (size_t)token * p.n_q_heads * D + (size_t)head * D + d) =
                    __floats2bfloat162_rn(numerator[0] / denominator, numerator[1] / denominator);
            } else if (in_cluster) {
                *reinterpret_cast<float2*>(mine + r * (D + 2) + d) = make_float2(numerator[0] / denominator, numerator[1] / denominator);
            } else {
                *reinterpret_cast<float2*>(p.partial_out + slot * D + d) = make_float2(numerator[0] / denominator, numerator[1] / denominator);
            }
        }
        if (lane == 0 && n_splits > 1) {
            if (in_cluster) {
                mine[r * (D + 2) + D] = best;
                mine[r * (D + 2) + D + 1] = denominator;
            } else {
                p.partial_ml[slot * 2] = best;
                p.partial_ml[slot * 2 + 1] = denominator;
            }
        }
    }
    if (in_cluster) {
        // The splits of this (sequence, kv head) are the ranks 0 .. n_splits - 1 of one cluster (ranks beyond have left
        // already; a cluster barrier waits for threads that have not exited).  Every rank takes a share of the group's
        // output elements and adds the splits' results in the order of the ranks, with the arithmetic of the merge
        // kernel below, reading the other ranks' shared memory.
        cluster_arrive_wait();
        const uint32_t mine_address = smem_address(mine);
        constexpr int kMaxRanks = 16;     // the largest cluster the launcher forms: it merges more splits by the merge kernel
        bool arrived = false;
        for (int index = split * kThreads + threadIdx.x; index < group * D; index += n_splits * kThreads) {
            const int r = index / D, d = index % D;
            // all ranks' values are asked for before the first is used: a load from another block's shared memory
            // takes some hundred cycles, and one after the other they were most of this kernel's time with few keys
            float maxima[kMaxRanks], sums[kMaxRanks], outputs[kMaxRanks];
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s) {
                const bool present = s < n_splits;
                // a head's maximum and sum lie side by side (8-byte aligned: D + 2 is even)
                const float2 statistics = present ? load_cluster2(mine_address + (uint32_t)(r * (D + 2) + D) * 4u, (uint32_t)s)
                                                  : make_float2(-INFINITY, 0.0f);
                maxima[s] = statistics.x;
                sums[s] = statistics.y;
                outputs[s] = present ? load_cluster(mine_address + (uint32_t)(r * (D + 2) + d) * 4u, (uint32_t)s) : 0.0f;
            }
            float best = -INFINITY;
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s) best = fmaxf(best, maxima[s]);
            float numerator = 0.0f, denominator = 0.0f;
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s) {
                if (s < n_splits) {       // in the order of the ranks, with the merge kernel's arithmetic
                    const float weight = sums[s] * exp2f(maxima[s] - best);
                    numerator += outputs[s] * weight;
                    denominator += weight;
                }
            }
            if (index + n_splits * kThreads >= group * D) {      // the last element of this thread: its values are here
                cluster_arrive();
                arrived = true;
            }
            p.out[(size_t)token * p.n_q_heads * D + (size_t)(kv_head * group + r) * D + d] = __float2bfloat16_rn(numerator / denominator);
        }
        if (!arrived) cluster_arrive();
        cluster_wait();      // nobody leaves while another rank may still read its shared memory
    }
}

// out = sum_s O_s * l_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)   (utils/paged_attention.py:220-237)
template <int D>
__global__ void attention_decode_merge_kernel(const AttnParams p) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    const int seq = blockIdx.y, head = blockIdx.x;
    const int token = p.q_start[seq];
    if (p.q_start[seq + 1] - token != 1) return;
    const int context = p.context_len[seq];
    const int low_key = p.window > 0 ? max(0, context - p.window) : 0;
    const int first_key = (low_key / kTileKeys) * kTileKeys;
    const int split_len = split_length(p, context - first_key);
    const int n_splits = min((context - first_key + split_len - 1) / split_len, p.max_splits);
    if (n_splits <= 1) return;
    const size_t slot0 = ((size_t)(p.slot_by_seq ? seq : token) * p.n_q_heads + head) * p.max_splits;
    float best = -INFINITY;
    for (int s = 0; s < n_splits; ++s) best = fmaxf(best, p.partial_ml[(slot0 + s) * 2]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float numerator = 0.0f, denominator = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float weight = p.partial_ml[(slot0 + s) * 2 + 1] * exp2f(p.partial_ml[(slot0 + s) * 2] - best);
            numerator += p.partial_out[(slot0 + s) * D + d] * weight;
            denominator += weight;
        }
        p.out[(size_t)token * p.n_q_heads * D + (size_t)head * D + d] = __float2bfloat16_rn(numerator / denominator);
    }
}

template <int D>
int launch_portions(const AttnParams& p, int total_tiles, cudaStream_t stream) {
    const size_t shared = (size_t)(kTileRows * D + 4 * kTileKeys * D) * sizeof(__nv_bfloat16);
    if (int limit_status = llm_raise_shared_limit(reinterpret_cast<const void*>(attention_portions_kernel<D>), shared, "attention_portions")) return limit_status;
    dim3 grid(total_tiles, p.n_kv_heads);
    llm_launch(attention_portions_kernel<D>, grid, kThreads, shared, stream, p);
    return llm_check_launch("attention_portions");
}

template <int D>
int launch_decode_cp_async(const AttnParams& p, cudaStream_t stream) {
    size_t shared = (size_t)(16 * D + 4 * kTileKeys * D) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)4 * 16 * (D + 2) * sizeof(float) + 16 * D * sizeof(__nv_bfloat16);
    if (merge > shared) shared = merge;
    if (int limit_status = llm_raise_shared_limit(reinterpret_cast<const void*>(attention_decode_kernel<D>), shared, "attention_decode")) return limit_status;
    dim3 grid(p.max_splits, p.n_kv_heads, p.n_seqs);
    llm_launch(attention_decode_kernel<D>, grid, kThreads, shared, stream, p);
    return llm_check_launch("attention_decode");
}

template <int D>
int launch_decode_tma(const AttnParams& p, cudaStream_t stream) {
    // rows of the page pool seen as a [pages * kv_heads * page_size, D] matrix: the real extent, so that a block-table
    // entry that names no page of the pool is copied as zeros and nothing outside the pool is read
    const uint64_t rows = (uint64_t)p.num_pages * p.n_kv_heads * p.page_size;
    CUtensorMap map_k, map_v;
    bool described;
    if (D == 128) {
        tma::EncodeTiled encode = tma::encode_tiled();
        described = encode != nullptr && tc5::make_page_map(&map_k, encode, p.k_pages, p.page_size, (long long)p.num_pages * p.n_kv_heads) &&
                    tc5::make_page_map(&map_v, encode, p.v_pages, p.page_size, (long long)p.num_pages * p.n_kv_heads);
    } else {
        described = tma::make_map_bf16(&map_k, p.k_pages, rows, D, (uint32_t)p.page_size) &&
                    tma::make_map_bf16(&map_v, p.v_pages, rows, D, (uint32_t)p.page_size);
    }
    if (!described) return launch_decode_cp_async<D>(p, stream);
    const size_t shared = (size_t)kDecodeStages * 2 * kTileKeys * D * 2 + (size_t)16 * D * 2 + 1024;
    if (int limit_status = llm_raise_shared_limit(reinterpret_cast<const void*>(attention_decode_tma_kernel<D>), shared, "attention_decode_tma")) return limit_status;
    dim3 grid(p.max_splits, p.n_kv_heads, p.n_seqs);
    if (!p.cluster_merge) {
        llm_launch(attention_decode_tma_kernel<D>, grid, kDecodeThreads, shared, stream, map_k, map_v, p);
        return llm_check_launch("attention_decode_tma");
    }
    // the splits of a (sequence, kv head) pair as one cluster along x
    if (p.max_splits > 8) {
        static bool allowed = false;
        if (!allowed) {
            cudaError_t status = cudaFuncSetAttribute(attention_decode_tma_kernel<D>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (status != cudaSuccess) {
                llm_set_error("attention_decode_tma: clusters of %d are not allowed: %s", p.max_splits, cudaGetErrorString(status));
                return (int)status;
            }
            allowed = true;
        }
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(kDecodeThreads, 1, 1);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    int count = 0;
    if (llm_pdl_enabled()) {
        attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    attribute[count].id = cudaLaunchAttributeClusterDimension;
    attribute[count].val.clusterDim.x = (unsigned)p.max_splits;
    attribute[count].val.clusterDim.y = 1;
    attribute[count].val.clusterDim.z = 1;
    ++count;
    config.attrs = attribute;
    config.numAttrs = count;
    cudaError_t status = cudaLaunchKernelEx(&config, attention_decode_tma_kernel<D>, map_k, map_v, p);
    if (status != cudaSuccess) {
        llm_set_error("attention_decode_tma (cluster of %d): %s", p.max_splits, cudaGetErrorString(status));
        return (int)status;
    }
    return llm_check_launch("attention_decode_tma");
}

template <int D>
int launch_decode(const AttnParams& p, cudaStream_t stream) {
    const bool whole_pages = p.page_size >= 8 && p.page_size <= kTileKeys && kTileKeys % p.page_size == 0 && p.page_size % 8 == 0;
    const bool by_tma = whole_pages && aligned16(p.k_pages) && aligned16(p.v_pages);
    AttnParams q = p;
    // up to 8 splits (the portable cluster size) or exactly 16 (allowed on request) merge inside the kernel; others, or the cp.async kernel, go through the
    // scratch buffers and the merge kernel
    q.cluster_merge = by_tma && p.cluster_merge && p.max_splits > 1 && (p.max_splits <= 8 || p.max_splits == 16);
    if (p.max_splits > 1 && !q.cluster_merge && (p.partial_out == nullptr || p.partial_ml == nullptr)) {
        llm_set_error("attention_decode: %d splits need the scratch buffers for partial results", p.max_splits);
        return LLM_REFUSED;
    }
    int status = by_tma ? launch_decode_tma<D>(q, stream) : launch_decode_cp_async<D>(q, stream);
    if (status != LLM_OK || p.max_splits <= 1 || q.cluster_merge) return status;
    dim3 merge_grid(p.n_q_heads, p.n_seqs);
    llm_launch(attention_decode_merge_kernel<D>, merge_grid, D < 128 ? D : 128, 0, stream, p);
    return llm_check_launch("attention_decode_merge");
}

// LLMSERVER_B200_DECODE_MERGE=kernel sends every split decode through scratch memory and the merge kernel.
bool decode_cluster_merge_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* value = getenv("LLMSERVER_B200_DECODE_MERGE");
        enabled = (value != nullptr && value[0] == 'k') ? 0 : 1;
    }
    return enabled == 1;
}

}  // namespace

// Sizes the tensor-core kernels take; everything else goes to the generic kernel.
LLM_EXPORT int llm_attention_mma_supports(int head_dim, int n_q_heads, int n_kv_heads) {
    if (head_dim != 64 && head_dim != 128) return 0;
    if (n_kv_heads <= 0 || n_q_heads % n_kv_heads) return 0;
    return n_q_heads / n_kv_heads <= 16;
}

// old_keys_settled: the caller vouches that, of the keys the decode rows read, only each sequence's newest was written
// by the kernel launched just before this call (everything older by kernels that completed earlier, e.g. earlier
// steps behind a copy): the decode kernel then starts copying older keys without waiting for that kernel.
// run_portions / run_decode: which of the two kernels to launch (a mixed batch launches both; each
// skips the other's sequences).  total_tiles: sum over sequences of ceil(q_len * group / 64), counting
// sequences of one token only when the decode kernel is not run.
LLM_EXPORT int llm_attention_mma(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                 const int* block_tables, int max_blocks, const int* q_start, const int* context_len,
                                 void* out, int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                 int num_pages, float scale, int window, int run_portions, int total_tiles, int run_decode,
                                 int split_len, int max_splits, float* partial_out, float* partial_ml,
                                 int old_keys_settled, int* error_flag, cudaStream_t stream) {
    if (!llm_attention_mma_supports(head_dim, n_q_heads, n_kv_heads)) {
        llm_set_error("attention_mma: head_dim %d with %d/%d heads is not supported (head_dim 64 or 128, group <= 16)",
                      head_dim, n_q_heads, n_kv_heads);
        return LLM_REFUSED;
    }
    if (run_decode && (split_len == 0 || (split_len > 0 && split_len % kTileKeys) || max_splits <= 0 || -split_len > max_splits)) {
        llm_set_error("attention_mma: split_len %d must be a positive multiple of %d, or minus a number of parts up to max_splits", split_len, kTileKeys);
        return LLM_REFUSED;
    }
    if (n_seqs > 65535 || n_kv_heads > 65535) {
        llm_set_error("attention_mma: at most 65535 sequences per launch, got %d", n_seqs);
        return LLM_REFUSED;
    }
    if (num_pages <= 0) {
        llm_set_error("attention_mma: the page pool has %d pages", num_pages);
        return LLM_REFUSED;
    }
    AttnParams p;
    p.q = (const __nv_bfloat16*)q;
    p.q_stride = q_stride;
    p.k_pages = (const __nv_bfloat16*)k_pages;
    p.v_pages = (const __nv_bfloat16*)v_pages;
    p.block_tables = block_tables;
    p.max_blocks = max_blocks;
    p.num_pages = num_pages;
    p.slot_by_seq = 0;
    p.cluster_merge = decode_cluster_merge_enabled() ? 1 : 0;
    p.old_keys_settled = old_keys_settled;
    p.q_start = q_start;
    p.context_len = context_len;
    p.out = (__nv_bfloat16*)out;
    p.n_seqs = n_seqs;
    p.n_q_heads = n_q_heads;
    p.n_kv_heads = n_kv_heads;
    p.page_size = page_size;
    p.scale_log2 = scale * kLog2e;
    p.window = window;
    p.skip_single = run_decode;
    p.split_len = split_len;
    p.max_splits = max_splits;
    p.partial_out = partial_out;
    p.partial_ml = partial_ml;
    p.error_flag = error_flag;
    int status = LLM_OK;
    if (run_portions && total_tiles > 0)
        status = head_dim == 128 ? launch_portions<128>(p, total_tiles, stream) : launch_portions<64>(p, total_tiles, stream);
    if (status == LLM_OK && run_decode)
        status = head_dim == 128 ? launch_decode<128>(p, stream) : launch_decode<64>(p, stream);
    return status;
}

// ------------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: scratch in a fixed array of the library
// (see attention_noalloc.h for who needs this and for the rules of use).
// ------------------------------------------------------------------------------------------------
#include "attention_noalloc.h"

static __device__ __align__(256) unsigned char g_noalloc_scratch[LLM_NOALLOC_SCRATCH_BYTES];
// What the kernels of the last call reported (0: nothing); see llm_attention_decode_noalloc_status.
static __device__ int g_noalloc_status;

namespace {
constexpr int kMaxDevices = 64;
// Device addresses of g_noalloc_scratch and g_noalloc_status per device.  In host code the names are only
// handles for cudaGetSymbolAddress; the kernels must be given the addresses that call returns.
float* g_noalloc_address[kMaxDevices] = {};
int* g_noalloc_status_address[kMaxDevices] = {};

int noalloc_device(const char* what) {
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess || device < 0 || device >= kMaxDevices) {
        llm_set_error("%s: cannot tell the current device: %s", what, cudaGetErrorString(status));
        return -1;
    }
    return device;
}
}  // namespace

LLM_EXPORT int llm_attention_decode_noalloc(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                            const int* block_tables, int max_blocks, const int* q_start,
                                            const int* context_len, void* out, int n_seqs, int n_q_heads,
                                            int n_kv_heads, int head_dim, int page_size, int num_pages, float scale,
                                            int window, int split_len, int max_splits, cudaStream_t stream) {
    if (n_seqs <= 0) return LLM_OK;
    if (!llm_attention_mma_supports(head_dim, n_q_heads, n_kv_heads)) {
        llm_set_error("attention_decode_noalloc: head_dim %d with %d/%d heads is not supported (head_dim 64 or 128, group <= 16)",
                      head_dim, n_q_heads, n_kv_heads);
        return LLM_REFUSED;
    }
    if (split_len == 0 || (split_len > 0 && split_len % kTileKeys) || max_splits <= 0 || -split_len > max_splits) {
        llm_set_error("attention_decode_noalloc: split_len %d must be a positive multiple of %d, or minus a number of parts up to max_splits %d",
                      split_len, kTileKeys, max_splits);
        return LLM_REFUSED;
    }
    if (n_seqs > 65535) {
        llm_set_error("attention_decode_noalloc: at most 65535 sequences per call, got %d", n_seqs);
        return LLM_REFUSED;
    }
    if (num_pages <= 0) {
        llm_set_error("attention_decode_noalloc: the page pool has %d pages", num_pages);
        return LLM_REFUSED;
    }
    const size_t slots = (size_t)n_seqs * n_q_heads * max_splits;
    const size_t needed = slots * (size_t)(head_dim + 2) * sizeof(float);
    if (needed > LLM_NOALLOC_SCRATCH_BYTES) {
        llm_set_error("attention_decode_noalloc: %d sequences x %d heads x %d splits need %zu bytes of scratch; the "
                      "library's fixed array holds %u (use fewer sequences per call or longer splits)",
                      n_seqs, n_q_heads, max_splits, needed, (unsigned)LLM_NOALLOC_SCRATCH_BYTES);
        return LLM_REFUSED;
    }
    const int device = noalloc_device("attention_decode_noalloc");
    if (device < 0) return LLM_REFUSED;
    if (g_noalloc_address[device] == nullptr) {   // first call on this device
        void* address = nullptr;
        void* status_address = nullptr;
        cudaError_t status = cudaGetSymbolAddress(&address, g_noalloc_scratch);
        if (status == cudaSuccess) status = cudaGetSymbolAddress(&status_address, g_noalloc_status);
        if (status != cudaSuccess || address == nullptr || status_address == nullptr) {
            llm_set_error("attention_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(status));
            return status != cudaSuccess ? (int)status : LLM_REFUSED;
        }
        g_noalloc_status_address[device] = static_cast<int*>(status_address);
        g_noalloc_address[device] = static_cast<float*>(address);
    }
    // the status word starts every call at zero (ordered on the caller's stream, like the kernels)
    cudaError_t cleared = cudaMemsetAsync(g_noalloc_status_address[device], 0, sizeof(int), stream);
    if (cleared != cudaSuccess) {
        llm_set_error("attention_decode_noalloc: cannot clear the status word: %s", cudaGetErrorString(cleared));
        return (int)cleared;
    }
    AttnParams p;
    p.q = (const __nv_bfloat16*)q;
    p.q_stride = q_stride;
    p.k_pages = (const __nv_bfloat16*)k_pages;
    p.v_pages = (const __nv_bfloat16*)v_pages;
    p.block_tables = block_tables;
    p.max_blocks = max_blocks;
    p.num_pages = num_pages;
    p.slot_by_seq = 1;      // the size check above counts sequences, whatever q_start holds
    p.cluster_merge = 0;    // this entry is the one that merges through the fixed scratch array
    p.old_keys_settled = 0;
    p.q_start = q_start;
    p.context_len = context_len;
    p.out = (__nv_bfloat16*)out;
    p.n_seqs = n_seqs;
    p.n_q_heads = n_q_heads;
    p.n_kv_heads = n_kv_heads;
    p.page_size = page_size;
    p.scale_log2 = scale * kLog2e;
    p.window = window;
    p.skip_single = 1;
    p.split_len = split_len;
    p.max_splits = max_splits;
    p.partial_out = g_noalloc_address[device];                       // [slots][head_dim]
    p.partial_ml = g_noalloc_address[device] + slots * head_dim;      // [slots][2]
    p.error_flag = g_noalloc_status_address[device];
    return head_dim == 128 ? launch_decode<128>(p, stream) : launch_decode<64>(p, stream);
}

// What the kernels of the most recent llm_attention_decode_noalloc call on the current device reported, after
// waiting for `stream`: 0 nothing; 3 a bounded wait on a copy ran out; 5 a block-table entry named no page of the
// pool (its keys were read as zeros or from page 0); 6 a context needed more splits than max_splits (its last keys
// were left out).  With any code but 0 the call's output is not valid.  Negative: a CUDA error (llm_last_error).
LLM_EXPORT int llm_attention_decode_noalloc_status(cudaStream_t stream) {
    const int device = noalloc_device("attention_decode_noalloc_status");
    if (device < 0) return LLM_REFUSED;
    if (g_noalloc_status_address[device] == nullptr) return 0;      // no call yet on this device
    int value = 0;
    cudaError_t status = cudaMemcpyAsync(&value, g_noalloc_status_address[device], sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (status == cudaSuccess) status = cudaStreamSynchronize(stream);
    if (status != cudaSuccess) {
        llm_set_error("attention_decode_noalloc_status: %s", cudaGetErrorString(status));
        return -(int)status;
    }
    return value;
}
