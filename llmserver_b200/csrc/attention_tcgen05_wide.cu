// Causal attention of long prompt portions over the paged cache on the fifth-generation tensor cores, 256 rows per
// CTA.  Same formulas and the same building blocks as attention_tcgen05.cu (utils/attention.py:186-198,
// utils/attention.py:75-96); what differs is how the work is laid out on an SM:
//
//   one CTA per SM takes 256 rows of one (sequence, kv head) as two halves A and B of 128 rows (rows are
//   (token, head of the group) pairs) and walks the keys in tiles of 128.  Both halves read the same K and V
//   tiles, so a tile is fetched once for 256 rows, and S = Q K^T is a 128 x 128 x 16 instruction, which the
//   tensor core runs at full rate (the 128 x 64 x 16 form of the 128-row kernel is bound by shared-memory reads).
//
//   producer warp   TMA: Q of both halves once (4-D boxes), then per key tile the K and V pages (one 5-D box
//                   per page) into rings of three and two stages
//   MMA warp        one thread: S_A(0) S_B(0), then per tile  PV_A(j) S_A(j+1) PV_B(j) S_B(j+1): while the softmax
//                   warps of one half work on their S, the tensor core runs the other half's P V and next S
//   8 softmax warps four per half; thread r owns row r of its half: tcgen05.ld of S (two loads of 64 columns),
//                   mask at the edges only, running maximum and sum in 32-bit, 2^x on the special-function unit,
//                   P written as packed bfloat16 over columns 64..127 of the half's S; O is rescaled only when
//                   a row's maximum has grown by more than 2^8 since its reference
//
// Tensor memory (all 512 columns): S_A | S_B | O_A | O_B, 128 columns each.  S_h(j+1) is issued behind PV_h(j) and the
// tensor core works in order, so "S_h(j+1) is ready" also says that PV_h(j) has finished with O_h and P_h.
// Every mbarrier wait is bounded; a wait that runs out sets the error flag, and the CTA still releases its
// tensor memory.  Takes head_dim 128, groups of 1 to 16 heads (floor(128 / G) tokens x G heads per half), pages of 8 to 128 tokens.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc5;
using tma::mbar_arrive;
using tma::mbar_expect_tx;
using tma::mbar_init;
using tma::mbar_wait;
using tma::smem_u32;

constexpr int kHalfRows = 128;    // rows per half (UMMA M)
constexpr int kRows = 2 * kHalfRows;
constexpr int kKeys = 128;        // keys per tile (UMMA N of S, K of P V)
constexpr int kDim = 128;         // head_dim
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kThreads = 320;     // 8 softmax warps + producer warp + MMA warp
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

constexpr uint32_t kQHalfBytes = kHalfRows * kDim * 2;   // 32 KiB
constexpr uint32_t kKVBytes = kKeys * kDim * 2;          // 32 KiB per K or V tile
constexpr uint32_t kTileBytes = 2 * kQHalfBytes + (kKStages + kVStages) * kKVBytes;   // 224 KiB
constexpr uint32_t kControlBytes = 256;
constexpr uint32_t kSharedBytes = kTileBytes + 1024 + kControlBytes;
constexpr uint32_t kTmemCols = 512;
__device__ __forceinline__ uint32_t col_s(int half) { return half ? 128u : 0u; }
__device__ __forceinline__ uint32_t col_o(int half) { return half ? 384u : 256u; }
constexpr uint32_t kColP = 64;    // P of a half lies over columns 64..127 of its S

struct Control {      // barriers and flags, at the end of the dynamic shared memory
    uint64_t q_full, k_full[kKStages], k_free[kKStages], v_full[kVStages], v_free[kVStages], s_ready[2], p_ready[2], o_final[2];
    uint32_t tmem_slot;
    int failed;
};
static_assert(sizeof(Control) <= kControlBytes, "control block");

struct WideParams {
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

__global__ void __launch_bounds__(kThreads, 1) attention_prefill_wide_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                          const __grid_constant__ CUtensorMap map_k,
                                                                          const __grid_constant__ CUtensorMap map_v,
                                                                          const WideParams p) {
    extern __shared__ __align__(16) unsigned char shared_raw[];
    pdl_trigger();
    pdl_wait();

    const uint32_t raw = smem_u32(shared_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t q_smem = base, k_smem = base + 2 * kQHalfBytes, v_smem = k_smem + kKStages * kKVBytes;
    Control& control = *reinterpret_cast<Control*>(shared_raw + (kSharedBytes - kControlBytes));
    int& failed = control.failed;

    const int group = p.n_q_heads / p.n_kv_heads;
    const int tokens_per_half = kHalfRows / group;
    const int kv_head = blockIdx.y;
    // Work of this CTA: one or two 256-row tiles of one sequence.  Tile t of a causal prompt sees about t + 1 key
    // tiles, so tile T - 1 - b is paired with tile b: every CTA of a sequence then has the same amount of work.
    int seq = 0, pair = blockIdx.x, first_tile = 0, second_tile = 0;
    for (; seq < p.n_seqs; ++seq) {
        const int q_len = p.q_start[seq + 1] - p.q_start[seq];
        const int tiles = (q_len == 1 && p.skip_single) ? 0 : (q_len + 2 * tokens_per_half - 1) / (2 * tokens_per_half);
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
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&control.tmem_slot)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = control.tmem_slot;

  for (int pass = 0; pass < passes; ++pass) {
    const int tile = pass == 0 ? first_tile : second_tile;
    const int first_token = tile * 2 * tokens_per_half;
    const int tokens_here = min(2 * tokens_per_half, q_len - first_token);
    const bool has_b = tokens_here > tokens_per_half;
    const int high_key = base_position + first_token + tokens_here - 1;
    int low_key = 0;
    if (p.window > 0) low_key = max(0, base_position + first_token - p.window + 1);
    const int first_tile_key = (low_key / kKeys) * kKeys;
    const int n_tiles = (high_key - first_tile_key) / kKeys + 1;

    // fresh barriers for every pass: at the end of a pass every copy has landed and every MMA has retired
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&control.q_full), 1);
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(smem_u32(&control.k_full[s]), 1);
            mbar_init(smem_u32(&control.k_free[s]), 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(smem_u32(&control.v_full[s]), 1);
            mbar_init(smem_u32(&control.v_free[s]), 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(smem_u32(&control.s_ready[h]), 1);
            mbar_init(smem_u32(&control.p_ready[h]), 4);      // one arrival per softmax warp of the half
            mbar_init(smem_u32(&control.o_final[h]), 1);
        }
        tma::mbar_fence_init();
    }
    __syncthreads();

    if (warp == 8) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            const uint32_t bar = smem_u32(&control.q_full);
            const uint32_t half_bytes = (uint32_t)(tokens_per_half * group) * (uint32_t)kDim * 2u;
            mbar_expect_tx(bar, has_b ? 2 * half_bytes : half_bytes);
            for (int h = 0; h < (has_b ? 2 : 1); ++h) {
                const int token = token0 + first_token + h * tokens_per_half;
                tma_load_4d(q_smem + h * kQHalfBytes, &map_q, bar, 0, 0, kv_head, token);
                tma_load_4d(q_smem + h * kQHalfBytes + kHalfRows * 128u, &map_q, bar, 64, 0, kv_head, token);
            }
        }
        // one copy per page: 8-key groups of [low 64 columns | high 64 columns], 1024 bytes each (a 5-D box)
        const int copies = kKeys / p.page_size;
        // The MMA warp's work finishes in the order S(0) | PV(0) S(1) | PV(1) S(2) | ...: K of tile t can go out once
        // S(t - 3) is done, V of tile t once PV(t - 2) is, so the copies go K_0 | K_1 V_0 | K_2 V_1 | K_3 V_2 | ...
        for (int step = 0; step <= n_tiles; ++step) {
            bool ok = true;
            if (step < n_tiles) {
                const int t = step, s = t % kKStages;
                if (t >= kKStages) ok = mbar_wait(smem_u32(&control.k_free[s]), ((t / kKStages) - 1) & 1);
                if (ok) {
                    if (lane == 0) mbar_expect_tx(smem_u32(&control.k_full[s]), kKVBytes);
                    __syncwarp();
                    if (lane < copies) {
                        // whole tiles always: pages past the sequence's end come from whatever the zero-padded
                        // table names (an existing page with finite contents, masked out below)
                        const int key = first_tile_key + t * kKeys + lane * p.page_size;
                        const int page = table[min(key / p.page_size, p.max_blocks - 1)];
                        if ((unsigned)page >= (unsigned)p.num_pages && p.error_flag) atomicExch(p.error_flag, 5);
                        tma_load_5d(k_smem + s * kKVBytes + (uint32_t)(lane * p.page_size) * 256u, &map_k,
                                    smem_u32(&control.k_full[s]), 0, 0, 0, 0, page * p.n_kv_heads + kv_head);
                    }
                }
            }
            if (ok && step >= 1) {
                const int t = step - 1, s = t % kVStages;
                if (t >= kVStages) ok = mbar_wait(smem_u32(&control.v_free[s]), ((t / kVStages) - 1) & 1);
                if (ok) {
                    if (lane == 0) mbar_expect_tx(smem_u32(&control.v_full[s]), kKVBytes);
                    __syncwarp();
                    if (lane < copies) {
                        const int key = first_tile_key + t * kKeys + lane * p.page_size;
                        const int page = table[min(key / p.page_size, p.max_blocks - 1)];
                        tma_load_5d(v_smem + s * kKVBytes + (uint32_t)(lane * p.page_size) * 256u, &map_v,
                                    smem_u32(&control.v_full[s]), 0, 0, 0, 0, page * p.n_kv_heads + kv_head);
                    }
                }
            }
            if (!ok) {
                failed = 1;
                break;
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = instruction(kHalfRows, kKeys, false);
            const uint32_t idesc_o = instruction(kHalfRows, kDim, true);
            // descriptors are a base plus a byte offset / 16 in the low field (shared addresses stay below 2^18)
            const uint64_t q_desc = desc_k_major(q_smem, 1024u), k_desc = desc_k_major(k_smem, 2048u);
            const uint64_t v_desc = desc_mn_major(v_smem, 1024u, 2048u);
            auto issue_s = [&](int h, int stage) {          // S_h = Q_h K^T
#pragma unroll
                for (int ks = 0; ks < kDim / 16; ++ks) {
                    const uint32_t half = ks >> 2, within = (ks & 3) * 32;
                    mma_ss(tmem + col_s(h), q_desc + ((h * kQHalfBytes + half * (kHalfRows * 128u) + within) >> 4),
                           k_desc + ((stage * kKVBytes + half * 1024u + within) >> 4), idesc_s, ks > 0 ? 1u : 0u);
                }
            };
            auto issue_pv = [&](int h, int stage, bool first) {     // O_h += P_h V
#pragma unroll
                for (int kk = 0; kk < kKeys / 16; ++kk)     // 16 keys = 8 packed columns of P, two 8-key groups of V
                    mma_ts(tmem + col_o(h), tmem + col_s(h) + kColP + kk * 8, v_desc + ((stage * kKVBytes + kk * 4096u) >> 4),
                           idesc_o, (first && kk == 0) ? 0u : 1u);
            };
            bool ok = mbar_wait(smem_u32(&control.q_full), 0) && mbar_wait(smem_u32(&control.k_full[0]), 0);
            if (ok) {
                fence_after();
                issue_s(0, 0);
                mma_commit(smem_u32(&control.s_ready[0]));
                if (has_b) {
                    issue_s(1, 0);
                    mma_commit(smem_u32(&control.s_ready[1]));
                }
                mma_commit(smem_u32(&control.k_free[0]));
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int vs = j % kVStages, ks = (j + 1) % kKStages;
                const bool next = j + 1 < n_tiles;
                ok = mbar_wait(smem_u32(&control.v_full[vs]), (j / kVStages) & 1) && mbar_wait(smem_u32(&control.p_ready[0]), j & 1);
                if (!ok) break;
                fence_after();
                issue_pv(0, vs, j == 0);
                if (!next) mma_commit(smem_u32(&control.o_final[0]));
                if (next) {
                    ok = mbar_wait(smem_u32(&control.k_full[ks]), ((j + 1) / kKStages) & 1);
                    if (!ok) break;
                    fence_after();
                    issue_s(0, ks);
                    mma_commit(smem_u32(&control.s_ready[0]));
                }
                if (has_b) {
                    ok = mbar_wait(smem_u32(&control.p_ready[1]), j & 1);
                    if (!ok) break;
                    fence_after();
                    issue_pv(1, vs, j == 0);
                    if (!next) mma_commit(smem_u32(&control.o_final[1]));
                }
                mma_commit(smem_u32(&control.v_free[vs]));
                if (next) {
                    if (has_b) {
                        issue_s(1, ks);
                        mma_commit(smem_u32(&control.s_ready[1]));
                    }
                    mma_commit(smem_u32(&control.k_free[ks]));
                }
            }
            if (!ok) failed = 1;
        }
    } else if (warp < 4 || has_b) {
        // ---------------------------------------------------------------- softmax: thread = row of its half
        const int h = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        // rows are (token, head of the group) pairs; with a group that does not divide 128 the last rows of a half are idle
        const int token = first_token + h * tokens_per_half + row / group, head = kv_head * group + row % group;
        const bool exists = row < tokens_per_half * group && token < q_len;
        const int position = exists ? base_position + token : -1;
        const int low = (exists && p.window > 0) ? max(0, position - p.window + 1) : 0;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_address = lane_base + col_s(h), o_address = lane_base + col_o(h);
        const uint32_t s_bar = smem_u32(&control.s_ready[h]), p_bar = smem_u32(&control.p_ready[h]);
        float reference = -INFINITY;     // what is subtracted in the exponent (a stale maximum)
        float row_sum = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            if (ok && !mbar_wait(s_bar, j & 1)) ok = false;
            fence_after();
            const int tile_key = first_tile_key + j * kKeys;
            // only tiles that touch the diagonal, the window's edge or the end of the rows need the mask
            const bool edge = tile_key + kKeys - 1 > position || tile_key < low;
            // The exponentials are taken against the reference as it stands, so they do not wait for this tile's
            // maximum; only when the maximum has outgrown the reference by the threshold (or nothing was seen yet) does
            // the reference move, and the tile is done again: S stays readable until P is stored over columns 64..127.
            // Maximum, exponential, sum and packing go element by element, so that the special-function unit and the
            // arithmetic pipes of the one softmax warp a scheduler has at a time work side by side.
            uint32_t packed_upper[32], packed_lower[32];
            float sums[4], running[4];
            auto half = [&](uint32_t (&packed)[32], int first_column, float subtract) {
                uint32_t values[64];
                tmem_load_64(s_address + first_column, values);
                if (edge) {
#pragma unroll
                    for (int c = 0; c < 64; ++c)
                        if (!(tile_key + first_column + c >= low && tile_key + first_column + c <= position)) values[c] = 0xff800000u;   // -inf
                }
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    const float x0 = __uint_as_float(values[c]), x1 = __uint_as_float(values[c + 1]);
                    // the scale and the reference enter the exponent in one fused multiply-add
                    const float e0 = exp2_approx(fmaf(x0, p.scale_log2, -subtract));
                    const float e1 = exp2_approx(fmaf(x1, p.scale_log2, -subtract));
                    running[(c >> 1) & 3] = fmaxf(running[(c >> 1) & 3], fmaxf(x0, x1));
                    sums[(c >> 1) & 3] += e0 + e1;
                    packed[c >> 1] = pack2(e0, e1);
                }
            };
            auto whole_tile = [&]() -> float {
                const float subtract = reference == -INFINITY ? 0.0f : reference;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    sums[c] = 0.0f;
                    running[c] = -INFINITY;
                }
                half(packed_upper, 64, subtract);
                half(packed_lower, 0, subtract);
                // the maximum is taken over the raw scores (the scale is positive)
                return fmaxf(fmaxf(running[0], running[1]), fmaxf(running[2], running[3])) * p.scale_log2;
            };
            const float tile_max = whole_tile();
            float factor = 1.0f;
            const bool moved = tile_max > reference + kRescaleThreshold || (reference == -INFINITY && tile_max > -INFINITY);
            if (__any_sync(0xffffffffu, moved)) {
                if (moved) {
                    factor = reference == -INFINITY ? 0.0f : exp2_approx(reference - tile_max);
                    reference = tile_max;
                }
                whole_tile();
                // O is rescaled (by the whole warp, rows that need nothing use 1): P V of the tile before is done,
                // since this tile's S was computed behind it
                if (j > 0) {
#pragma unroll
                    for (int chunk = 0; chunk < kDim / 32; ++chunk) {
                        uint32_t o_raw[32];
                        tmem_load_32(o_address + chunk * 32, o_raw);
#pragma unroll
                        for (int c = 0; c < 32; ++c) o_raw[c] = __float_as_uint(__uint_as_float(o_raw[c]) * factor);
                        tmem_store_32(o_address + chunk * 32, o_raw);
                    }
                }
            }
            row_sum = row_sum * factor + ((sums[0] + sums[1]) + (sums[2] + sums[3]));
            tmem_store_32(s_address + kColP, packed_lower);          // keys 0..63 of the tile
            tmem_store_32(s_address + kColP + 32, packed_upper);     // keys 64..127
            tmem_wait_store();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_bar);
        }
        // the last P V, then O / sum
        if (ok && !mbar_wait(smem_u32(&control.o_final[h]), 0)) ok = false;
        fence_after();
        if (!ok) failed = 1;
        const float inverse = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
        __nv_bfloat16* dst = exists ? p.out + (size_t)(token0 + token) * p.n_q_heads * kDim + (size_t)head * kDim
                                    : nullptr;
#pragma unroll
        for (int chunk = 0; chunk < kDim / 32; ++chunk) {
            uint32_t o_raw[32];
            tmem_load_32(o_address + chunk * 32, o_raw);
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
        tma::mbar_inval(smem_u32(&control.q_full));
        for (int s = 0; s < kKStages; ++s) {
            tma::mbar_inval(smem_u32(&control.k_full[s]));
            tma::mbar_inval(smem_u32(&control.k_free[s]));
        }
        for (int s = 0; s < kVStages; ++s) {
            tma::mbar_inval(smem_u32(&control.v_full[s]));
            tma::mbar_inval(smem_u32(&control.v_free[s]));
        }
        for (int h = 0; h < 2; ++h) {
            tma::mbar_inval(smem_u32(&control.s_ready[h]));
            tma::mbar_inval(smem_u32(&control.p_ready[h]));
            tma::mbar_inval(smem_u32(&control.o_final[h]));
        }
    }
  }
    if (failed && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 6);
    if (warp == 9) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}

}  // namespace

LLM_EXPORT int llm_attention_prefill_wide_supports(int head_dim, int n_q_heads, int n_kv_heads, int page_size) {
    if (head_dim != kDim || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return 0;
    const int group = n_q_heads / n_kv_heads;
    if (group > 16) return 0;
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

// total_pairs: the number of CTAs: with pairing, the sum over the sequences it handles of ceil(ceil(q_len * group / 256) / 2)
// (each CTA takes a 256-row tile and its mirror, which evens out the work of a causal prompt); without, one CTA per tile; sequences of one token are skipped when skip_single is set (the decode kernel takes them).
LLM_EXPORT int llm_attention_prefill_wide(const void* q, int q_stride, int n_tokens, const void* k_pages, const void* v_pages,
                                          const int* block_tables, int max_blocks, const int* q_start, const int* context_len,
                                          void* out, int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int page_size, int num_pages, float scale, int window, int skip_single, int pairing, int total_pairs, int* error_flag,
                                          cudaStream_t stream) {
    if (total_pairs <= 0) return LLM_OK;
    if (num_pages <= 0) {
        llm_set_error("attention_prefill_wide: the page pool has %d pages", num_pages);
        return LLM_REFUSED;
    }
    if (!llm_attention_prefill_wide_supports(head_dim, n_q_heads, n_kv_heads, page_size) || !aligned16(q) || q_stride % 8 ||
        !(scale > 0.0f)) {
        llm_set_error("attention_prefill_wide: unsupported sizes (head_dim %d, %d/%d heads, page %d)", head_dim, n_q_heads,
                      n_kv_heads, page_size);
        return LLM_REFUSED;
    }
    if (n_kv_heads > 65535) {
        llm_set_error("attention_prefill_wide: too many kv heads (%d)", n_kv_heads);
        return LLM_REFUSED;
    }
    const int group = n_q_heads / n_kv_heads;
    tma::EncodeTiled encode = tma::encode_tiled();
    if (encode == nullptr) {
        llm_set_error("attention_prefill_wide: cuTensorMapEncodeTiled is not available");
        return LLM_REFUSED;
    }
    CUtensorMap map_q, map_k, map_v;
    if (!make_query_map(&map_q, encode, q, q_stride, n_tokens, head_dim, group, n_kv_heads, kHalfRows / group) ||
        !make_page_map(&map_k, encode, k_pages, page_size, (long long)num_pages * n_kv_heads) ||
        !make_page_map(&map_v, encode, v_pages, page_size, (long long)num_pages * n_kv_heads)) {
        llm_set_error("attention_prefill_wide: cannot describe Q or the cache pages to TMA");
        return LLM_REFUSED;
    }
    WideParams p;
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
    if (int limit_status = llm_raise_shared_limit(reinterpret_cast<const void*>(attention_prefill_wide_kernel), kSharedBytes, "attention_prefill_wide")) return limit_status;
    dim3 grid(total_pairs, n_kv_heads);
    llm_launch(attention_prefill_wide_kernel, grid, kThreads, kSharedBytes, stream, map_q, map_k, map_v, p);
    return llm_check_launch("attention_prefill_wide");
}
