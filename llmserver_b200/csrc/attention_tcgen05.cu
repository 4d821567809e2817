// Causal attention of prompt portions over the paged cache on the fifth-generation tensor cores:
// S = Q K^T and O += P V are tcgen05.mma instructions whose accumulators live in tensor memory; Q, K and
// V tiles arrive by TMA (128-byte swizzle); the softmax runs on 128 threads that each own one row.
//
// One CTA takes 128 rows (floor(128 / G) tokens x G heads) of one (sequence, kv head): rows are (token, head of the group) pairs, so the
// G query heads that share a kv head share every K/V tile.  It walks the keys the rows can see in tiles
// of 64 (whole cache pages), from the first key in the tile's window to the last token's position:
//
//   producer warp   TMA: the Q tile once (a 4-D box: 64 columns x G heads x 1 kv head x 128/G tokens), then
//                   per key tile the K pages and the V pages (one 5-D box per page) into rings of three and two stages (a K stage is free again
//                   once its S is computed, a V stage once its P V is)
//   MMA warp        one thread: S_b = Q K_j^T (8 x UMMA 128x64x16) into S buffer b = j mod 2, and, one
//                   tile behind, O += P_{j-1} V_{j-1} (4 x UMMA 128x128x16 with A = P read from tensor
//                   memory, B = V as an MN-major operand)
//   4 softmax warps thread r owns row r = lane r of tensor memory: tcgen05.ld of S_b, mask, scale, running
//                   maximum and sum in 32-bit, exp2, P written back over S_b as packed bfloat16
//                   (tcgen05.st); O is rescaled only when a row's maximum has grown by more than 2^8 since
//                   its reference (the reference, not the maximum, is subtracted in the exponent; the
//                   final division by the sum undoes it); at the end O / sum is stored as bfloat16
//
// Formulas as in attention_mma.cu (utils/attention.py:186-198, utils/attention.py:75-96).  Tensor memory:
// S0 | S1 | O = 64 + 64 + 128 columns; two CTAs fit on an SM (512 columns, 2 x 114 KiB shared memory), so one
// CTA's softmax overlaps the other's MMAs as well as its own next S tile.
// Every mbarrier wait is bounded; a wait that runs out sets the error flag, and the CTA still releases its
// tensor memory.  Takes head_dim 128, groups of 1 to 16 heads, pages of 8, 16, 32 or 64 tokens;
// other sizes use the mma.sync kernel.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int kRows = 128;        // rows per CTA (UMMA M)
constexpr int kKeys = 64;         // keys per tile (UMMA N of S, K of P V)
constexpr int kDim = 128;         // head_dim
constexpr int kKStages = 3;       // K ring: a copy needs more than one tile's time to arrive, so two tiles are in flight
constexpr int kVStages = 2;       // V ring
constexpr int kThreads = 192;     // 4 softmax warps + producer warp + MMA warp
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

constexpr uint32_t kQBytes = kRows * kDim * 2;        // 32 KiB
constexpr uint32_t kKVBytes = kKeys * kDim * 2;       // 16 KiB per K or V tile
constexpr uint32_t kColS0 = 0, kColS1 = 64, kColO = 128, kTmemCols = 256;

constexpr uint32_t kTileBytes = kQBytes + (kKStages + kVStages) * kKVBytes;   // 112 KiB
constexpr uint32_t kControlBytes = 256;
constexpr uint32_t kSharedBytes = 113 * 1024;

struct Control {      // barriers and flags, at the end of the dynamic shared memory
    uint64_t q_full, k_full[kKStages], v_full[kVStages], k_free[kKStages], v_free[kVStages], s_ready[2], p_ready[2], o_done, o_final;
    uint32_t tmem_slot;
    int failed;
};
static_assert(sizeof(Control) <= kControlBytes, "control block");
static_assert(kTileBytes + kControlBytes <= kSharedBytes, "shared memory layout");

struct PrefillParams {
    const int* block_tables;
    int max_blocks;
    int num_pages;       // block-table entries outside 0 .. num_pages - 1 lie outside the tensor maps and read as zeros
    const int* q_start;
    const int* context_len;
    __nv_bfloat16* out;
    int n_seqs, n_q_heads, n_kv_heads, page_size;
    float scale_log2;
    int window;
    int skip_single;
    int pairing;
    int* error_flag;
};

using tma::mbar_arrive;
using tma::mbar_expect_tx;
using tma::mbar_init;
using tma::mbar_wait;
using tma::smem_u32;

using namespace tc5;

__global__ void __launch_bounds__(kThreads, 2) attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                             const __grid_constant__ CUtensorMap map_k,
                                                                             const __grid_constant__ CUtensorMap map_v,
                                                                             const PrefillParams p) {
    // All shared memory is dynamic: tiles (1024-byte aligned for the 128-byte swizzle) and, in the last 256 bytes,
    // the barriers.  113 KiB + 1 KiB the system reserves per CTA = 114 KiB, and two CTAs fill the SM's 228 KiB exactly.
    extern __shared__ __align__(16) unsigned char shared_raw[];
    pdl_trigger();
    pdl_wait();

    const uint32_t raw = smem_u32(shared_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    if (base - raw > kSharedBytes - kTileBytes - kControlBytes) {      // the tiles would not fit behind the padding
        if (threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 5);
        return;
    }
    const uint32_t q_smem = base, k_smem = base + kQBytes, v_smem = k_smem + kKStages * kKVBytes;
    Control& control = *reinterpret_cast<Control*>(shared_raw + (kSharedBytes - kControlBytes));
    uint64_t& q_full = control.q_full;
    uint64_t (&k_full)[kKStages] = control.k_full;
    uint64_t (&v_full)[kVStages] = control.v_full;
    uint64_t (&k_free)[kKStages] = control.k_free;
    uint64_t (&v_free)[kVStages] = control.v_free;
    uint64_t (&s_ready)[2] = control.s_ready;
    uint64_t (&p_ready)[2] = control.p_ready;
    uint64_t& o_done = control.o_done;
    uint64_t& o_final = control.o_final;
    uint32_t& tmem_slot = control.tmem_slot;
    int& failed = control.failed;

    const int group = p.n_q_heads / p.n_kv_heads;
    const int tokens_per_tile = kRows / group;
    const int kv_head = blockIdx.y;
    // Work of this CTA: one or two row tiles of one sequence.  Tile t of a causal prompt sees about t + 1 key
    // tiles, so tile T - 1 - b is paired with tile b: every CTA of a sequence then has the same amount of work.
    int seq = 0, pair = blockIdx.x, first_tile = 0, second_tile = 0;
    for (; seq < p.n_seqs; ++seq) {
        const int q_len = p.q_start[seq + 1] - p.q_start[seq];
        const int tiles = (q_len == 1 && p.skip_single) ? 0 : (q_len + tokens_per_tile - 1) / tokens_per_tile;
        const int pairs = p.pairing ? (tiles + 1) / 2 : tiles;
        if (pair < pairs) {
            first_tile = tiles - 1 - pair;      // heavy tiles first
            second_tile = p.pairing ? pair : first_tile;
            break;
        }
        pair -= pairs;
    }
    if (seq >= p.n_seqs) return;
    const int passes = second_tile < first_tile ? 2 : 1;
    const int token0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - token0;
    const int context = p.context_len[seq];
    const int base_position = context - q_len;
    const int* table = p.block_tables + (size_t)seq * p.max_blocks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) failed = 0;
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_slot;

  for (int pass = 0; pass < passes; ++pass) {
    const int tile = pass == 0 ? first_tile : second_tile;
    const int first_token = tile * tokens_per_tile;
    const int high_key = base_position + min(first_token + tokens_per_tile, q_len) - 1;
    int low_key = 0;
    if (p.window > 0) low_key = max(0, base_position + first_token - p.window + 1);
    const int first_tile_key = (low_key / kKeys) * kKeys;
    const int n_tiles = (high_key - first_tile_key) / kKeys + 1;

    // fresh barriers for every pass: at the end of a pass every copy has landed and every MMA has retired
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_free[s]), 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&v_free[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&s_ready[b]), 1);
            mbar_init(smem_u32(&p_ready[b]), 4);      // one arrival per softmax warp
        }
        mbar_init(smem_u32(&o_done), 1);
        mbar_init(smem_u32(&o_final), 1);
        tma::mbar_fence_init();
    }
    __syncthreads();

    if (warp == 4) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            mbar_expect_tx(smem_u32(&q_full), (uint32_t)(tokens_per_tile * group) * (uint32_t)kDim * 2u);
            tma_load_4d(q_smem, &map_q, smem_u32(&q_full), 0, 0, kv_head, token0 + tile * tokens_per_tile);
            tma_load_4d(q_smem + kRows * 128u, &map_q, smem_u32(&q_full), 64, 0, kv_head, token0 + tile * tokens_per_tile);
        }
        // one copy per page: 8-key groups of [low 64 columns | high 64 columns], 1024 bytes each (a 5-D box)
        const int copies = kKeys / p.page_size;
        const int my_page = lane;
        // K of tile t goes out as soon as S of tile t - 3 has been computed, V of tile t once P V of tile t - 2
        // has: the MMA warp issues S_0 S_1 PV_0 S_2 PV_1 S_3 PV_2 ..., so the copies go K_0 K_1 K_2 V_0 K_3 V_1 ...
        for (int step = 0; step < n_tiles + 2; ++step) {
            bool ok = true;
            if (step < n_tiles) {
                const int t = step, s = t % kKStages;
                if (t >= kKStages) ok = mbar_wait(smem_u32(&k_free[s]), ((t / kKStages) - 1) & 1);
                if (ok) {
                    if (lane == 0) mbar_expect_tx(smem_u32(&k_full[s]), kKVBytes);
                    __syncwarp();
                    if (lane < copies) {
                        // whole tiles always: pages past the sequence's end come from whatever the zero-padded
                        // table names (an existing page with finite contents, masked out below)
                        const int key = first_tile_key + t * kKeys + my_page * p.page_size;
                        const int page = table[min(key / p.page_size, p.max_blocks - 1)];
                        if ((unsigned)page >= (unsigned)p.num_pages && p.error_flag) atomicExch(p.error_flag, 5);
                        const uint32_t offset = s * kKVBytes + (uint32_t)(my_page * p.page_size) * 256u;
                        tma_load_5d(k_smem + offset, &map_k, smem_u32(&k_full[s]), 0, 0, 0, 0, page * p.n_kv_heads + kv_head);
                    }
                }
            }
            if (ok && step >= 2) {
                const int t = step - 2, s = t % kVStages;
                if (t >= kVStages) ok = mbar_wait(smem_u32(&v_free[s]), ((t / kVStages) - 1) & 1);
                if (ok) {
                    if (lane == 0) mbar_expect_tx(smem_u32(&v_full[s]), kKVBytes);
                    __syncwarp();
                    if (lane < copies) {
                        const int key = first_tile_key + t * kKeys + my_page * p.page_size;
                        const int page = table[min(key / p.page_size, p.max_blocks - 1)];
                        const uint32_t offset = s * kKVBytes + (uint32_t)(my_page * p.page_size) * 256u;
                        tma_load_5d(v_smem + offset, &map_v, smem_u32(&v_full[s]), 0, 0, 0, 0, page * p.n_kv_heads + kv_head);
                    }
                }
            }
            if (!ok) {
                failed = 1;
                break;
            }
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = instruction(kRows, kKeys, false);
            const uint32_t idesc_o = instruction(kRows, kDim, true);
            bool ok = mbar_wait(smem_u32(&q_full), 0);
            for (int j = 0; j <= n_tiles && ok; ++j) {
                if (j < n_tiles) {        // S_b = Q K_j^T
                    const int s = j % kKStages, b = j & 1;
                    ok = mbar_wait(smem_u32(&k_full[s]), (j / kKStages) & 1);
                    if (!ok) break;
                    fence_after();
#pragma unroll
                    for (int ks = 0; ks < kDim / 16; ++ks) {
                        const uint32_t half = ks >> 2, within = (ks & 3) * 32;
                        mma_ss(tmem + (b ? kColS1 : kColS0), desc_k_major(q_smem + half * (kRows * 128u) + within, 1024u),
                               desc_k_major(k_smem + s * kKVBytes + half * 1024u + within, 2048u), idesc_s, ks > 0 ? 1u : 0u);
                    }
                    mma_commit(smem_u32(&s_ready[b]));
                    mma_commit(smem_u32(&k_free[s]));
                }
                if (j > 0) {              // O += P_{j-1} V_{j-1}
                    const int t = j - 1, s = t % kVStages, b = t & 1;
                    ok = mbar_wait(smem_u32(&p_ready[b]), (t >> 1) & 1) && mbar_wait(smem_u32(&v_full[s]), (t / kVStages) & 1);
                    if (!ok) break;
                    fence_after();
#pragma unroll
                    for (int kk = 0; kk < kKeys / 16; ++kk)     // 16 keys = 8 packed columns of P, two 8-key groups of V
                        mma_ts(tmem + kColO, tmem + (b ? kColS1 : kColS0) + kk * 8,
                               desc_mn_major(v_smem + s * kKVBytes + kk * 4096u, 1024u, 2048u), idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
                    mma_commit(smem_u32(&v_free[s]));
                    mma_commit(smem_u32(&o_done));
                    if (t == n_tiles - 1) mma_commit(smem_u32(&o_final));
                }
            }
            if (!ok) failed = 1;
        }
    } else {
        // ---------------------------------------------------------------- softmax: thread = row
        const int row = warp * 32 + lane;
        // rows are (token, head of the group) pairs; with a group that does not divide 128 the last rows of a tile are idle
        const int token = first_token + row / group, head = kv_head * group + row % group;
        const bool exists = row < tokens_per_tile * group && token < q_len;
        const int position = exists ? base_position + token : -1;
        const int low = (exists && p.window > 0) ? max(0, position - p.window + 1) : 0;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float reference = -INFINITY;     // what is subtracted in the exponent (a stale maximum)
        float row_sum = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            if (ok && !mbar_wait(smem_u32(&s_ready[b]), (j >> 1) & 1)) ok = false;
            fence_after();
            const uint32_t s_address = lane_base + (b ? kColS1 : kColS0);
            uint32_t raw[64];
            tmem_load_64(s_address, raw);
            const int tile_key = first_tile_key + j * kKeys;
            // only tiles that touch the diagonal, the window's edge or the end of the rows need the mask
            if (tile_key + kKeys - 1 > position || tile_key < low) {
#pragma unroll
                for (int c = 0; c < 64; ++c)
                    if (!(tile_key + c >= low && tile_key + c <= position)) raw[c] = 0xff800000u;      // -inf
            }
            // The maximum is taken over the raw scores (the scale is positive); the scale and the reference enter
            // the exponent in one fused multiply-add.  Eight running maxima and four running sums keep the
            // dependent chains short: with two softmax warps per scheduler, latency is what this loop is bound by.
            // Four running maxima fed two scores at a time, the scale and the reference applied to two scores per
            // instruction, two pairs of running sums: the softmax warps are bound by instruction issue, so every
            // halved instruction count shows.
            float running[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) running[c] = fmaxf(__uint_as_float(raw[2 * c]), __uint_as_float(raw[2 * c + 1]));
#pragma unroll
            for (int c = 4; c < 32; ++c) running[c & 3] = max3(running[c & 3], __uint_as_float(raw[2 * c]), __uint_as_float(raw[2 * c + 1]));
            const float raw_max = fmaxf(fmaxf(running[0], running[1]), fmaxf(running[2], running[3]));
            const float tile_max = raw_max * p.scale_log2;
            // the reference moves only when the maximum has outgrown it by the threshold (or nothing was seen yet)
            float factor = 1.0f;
            if (tile_max > reference + kRescaleThreshold || (reference == -INFINITY && tile_max > -INFINITY)) {
                factor = reference == -INFINITY ? 0.0f : exp2_approx(reference - tile_max);
                reference = tile_max;
            }
            const float subtract = reference == -INFINITY ? 0.0f : reference;
            const uint64_t scale_pair = pair_of(p.scale_log2, p.scale_log2), minus_pair = pair_of(-subtract, -subtract);
            float weight[64];
#pragma unroll
            for (int c = 0; c < 32; ++c)
                halves_of(fma_pair(pair_of(__uint_as_float(raw[2 * c]), __uint_as_float(raw[2 * c + 1])), scale_pair, minus_pair),
                          weight[2 * c], weight[2 * c + 1]);
#pragma unroll
            for (int c = 0; c < 64; ++c) weight[c] = exp2_approx(weight[c]);
            uint64_t sums[2] = {pair_of(0.0f, 0.0f), pair_of(0.0f, 0.0f)};
#pragma unroll
            for (int c = 0; c < 32; ++c) sums[c & 1] = add_pair(sums[c & 1], pair_of(weight[2 * c], weight[2 * c + 1]));
            float sum_low, sum_high;
            halves_of(add_pair(sums[0], sums[1]), sum_low, sum_high);
            const float tile_sum = sum_low + sum_high;
            uint32_t packed[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) packed[c] = pack2(weight[2 * c], weight[2 * c + 1]);      // keys 2c, 2c + 1
            row_sum = row_sum * factor + tile_sum;
            // O is rescaled (by the whole warp, rows that need nothing use 1) once the previous P V is done
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.0f)) {
                if (ok && !mbar_wait(smem_u32(&o_done), (j - 1) & 1)) ok = false;
                fence_after();
#pragma unroll
                for (int chunk = 0; chunk < kDim / 32; ++chunk) {
                    uint32_t o_raw[32];
                    tmem_load_32(lane_base + kColO + chunk * 32, o_raw);
#pragma unroll
                    for (int c = 0; c < 32; ++c) o_raw[c] = __float_as_uint(__uint_as_float(o_raw[c]) * factor);
                    tmem_store_32(lane_base + kColO + chunk * 32, o_raw);
                }
            }
            tmem_store_32(s_address, packed);          // P over the first 32 columns of S_b
            tmem_wait_store();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_ready[b]));
        }
        // the last P V, then O / sum.  It has a barrier of its own: o_done may still be a phase behind here (the
        // softmax of the last tile needs S only, not the P V before it), and a parity wait cannot tell a phase
        // that is two behind from the one it waits for.
        if (ok && !mbar_wait(smem_u32(&o_final), 0)) ok = false;
        fence_after();
        if (!ok) failed = 1;
        const float inverse = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
        __nv_bfloat16* dst = exists ? p.out + (size_t)(token0 + token) * p.n_q_heads * kDim + (size_t)head * kDim
                                    : nullptr;
#pragma unroll
        for (int chunk = 0; chunk < kDim / 32; ++chunk) {
            uint32_t o_raw[32];
            tmem_load_32(lane_base + kColO + chunk * 32, o_raw);
            if (exists) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 words;
                    words.x = pack2(__uint_as_float(o_raw[8 * v]) * inverse, __uint_as_float(o_raw[8 * v + 1]) * inverse);
                    words.y = pack2(__uint_as_float(o_raw[8 * v + 2]) * inverse, __uint_as_float(o_raw[8 * v + 3]) * inverse);
                    words.z = pack2(__uint_as_float(o_raw[8 * v + 4]) * inverse, __uint_as_float(o_raw[8 * v + 5]) * inverse);
                    words.w = pack2(__uint_as_float(o_raw[8 * v + 6]) * inverse, __uint_as_float(o_raw[8 * v + 7]) * inverse);
                    *reinterpret_cast<uint4*>(dst + chunk * 32 + v * 8) = words;
                }
            }
        }
    }
    fence_before();
    __syncthreads();      // end of the pass: tensor memory, shared tiles and barriers are idle
    fence_after();
    if (pass + 1 < passes && threadIdx.x == 0) {
        tma::mbar_inval(smem_u32(&q_full));
        for (int s = 0; s < kKStages; ++s) {
            tma::mbar_inval(smem_u32(&k_full[s]));
            tma::mbar_inval(smem_u32(&k_free[s]));
        }
        for (int s = 0; s < kVStages; ++s) {
            tma::mbar_inval(smem_u32(&v_full[s]));
            tma::mbar_inval(smem_u32(&v_free[s]));
        }
        for (int b = 0; b < 2; ++b) {
            tma::mbar_inval(smem_u32(&s_ready[b]));
            tma::mbar_inval(smem_u32(&p_ready[b]));
        }
        tma::mbar_inval(smem_u32(&o_done));
        tma::mbar_inval(smem_u32(&o_final));
    }
  }
    if (failed && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 4);
    if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}

}  // namespace

LLM_EXPORT int llm_attention_prefill_tcgen05_supports(int head_dim, int n_q_heads, int n_kv_heads, int page_size) {
    if (head_dim != kDim || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return 0;
    const int group = n_q_heads / n_kv_heads;
    if (group > 16) return 0;
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64;
}

// total_pairs: the number of CTAs: with pairing, the sum over the sequences it handles of ceil(ceil(q_len * group / 128) / 2)
// (each CTA takes a row tile and its mirror, which evens out the work of a causal prompt); without, one CTA per tile; sequences of one token are skipped when skip_single is set (the decode kernel takes them).
LLM_EXPORT int llm_attention_prefill_tcgen05(const void* q, int q_stride, int n_tokens, const void* k_pages, const void* v_pages,
                                             const int* block_tables, int max_blocks, const int* q_start,
                                             const int* context_len, void* out, int n_seqs, int n_q_heads, int n_kv_heads,
                                             int head_dim, int page_size, int num_pages, float scale, int window, int skip_single, int pairing,
                                             int total_pairs, int* error_flag, cudaStream_t stream) {
    if (total_pairs <= 0) return LLM_OK;
    if (num_pages <= 0) {
        llm_set_error("attention_prefill_tcgen05: the page pool has %d pages", num_pages);
        return LLM_REFUSED;
    }
    if (!llm_attention_prefill_tcgen05_supports(head_dim, n_q_heads, n_kv_heads, page_size) || !aligned16(q) || q_stride % 8 ||
        !(scale > 0.0f)) {
        llm_set_error("attention_prefill_tcgen05: unsupported sizes (head_dim %d, %d/%d heads, page %d)", head_dim, n_q_heads,
                      n_kv_heads, page_size);
        return LLM_REFUSED;
    }
    if (n_kv_heads > 65535) {
        llm_set_error("attention_prefill_tcgen05: too many kv heads (%d)", n_kv_heads);
        return LLM_REFUSED;
    }
    const int group = n_q_heads / n_kv_heads;
    tma::EncodeTiled encode = tma::encode_tiled();
    if (encode == nullptr) {
        llm_set_error("attention_prefill_tcgen05: cuTensorMapEncodeTiled is not available");
        return LLM_REFUSED;
    }
    CUtensorMap map_q, map_k, map_v;
    if (!make_query_map(&map_q, encode, q, q_stride, n_tokens, head_dim, group, n_kv_heads, kRows / group) ||
        !make_page_map(&map_k, encode, k_pages, page_size, (long long)num_pages * n_kv_heads) ||
        !make_page_map(&map_v, encode, v_pages, page_size, (long long)num_pages * n_kv_heads)) {
        llm_set_error("attention_prefill_tcgen05: cannot describe Q or the cache pages to TMA");
        return LLM_REFUSED;
    }
    PrefillParams p;
    p.block_tables = block_tables;
    p.max_blocks = max_blocks;
    p.num_pages = num_pages;
    p.q_start = q_start;
    p.context_len = context_len;
    p.out = (__nv_bfloat16*)out;
    p.n_seqs = n_seqs;
    p.n_q_heads = n_q_heads;
    p.n_kv_heads = n_kv_heads;
    p.page_size = page_size;
    p.scale_log2 = scale * kLog2e;
    p.window = window;
    p.skip_single = skip_single;
    p.pairing = pairing;
    p.error_flag = error_flag;
    const size_t shared = kSharedBytes;
    if (int limit_status = llm_raise_shared_limit(reinterpret_cast<const void*>(attention_prefill_tcgen05_kernel), shared, "attention_prefill_tcgen05", true)) return limit_status;
    dim3 grid(total_pairs, n_kv_heads);
    llm_launch(attention_prefill_tcgen05_kernel, grid, kThreads, shared, stream, map_q, map_k, map_v, p);
    return llm_check_launch("attention_prefill_tcgen05");
}
