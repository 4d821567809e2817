"""bfloat16 tensor-core attention kernels over the paged cache (prompt portions and split-KV decode).

``try_attention`` returns None when the tensor-core kernels do not take the sizes; the caller then
uses the generic 32-bit-arithmetic kernel, which takes every size."""
from __future__ import annotations

import os

import torch

from .library import call, check, library, stream_handle, wait_error_flag

TILE = 64          # rows per block of the portions kernel, keys per tile of both kernels
MIN_SPLIT = 192    # fewest keys one decode block walks
DECODE_BLOCKS_PER_SM = 2    # blocks of the decode kernel an SM holds at a time (shared memory)
# Up to this many splits of a sequence form a thread-block cluster and merge their results in shared memory; more go
# through scratch memory and a merge kernel (as do all, with LLMSERVER_B200_DECODE_MERGE=kernel).
CLUSTER_MERGE = os.environ.get("LLMSERVER_B200_DECODE_MERGE", "cluster") != "kernel"
MAX_CLUSTER_SPLITS = 8
# With so few (sequence, kv head) pairs that 16 blocks each still leave every block an SM of its own (batch 1 of the
# 8B shape), clusters of 16 (beyond the portable size, which the hardware allows on request) get each block's keys in
# flight at once: 3.21 against 3.25 ms per batch-1 step.  With more pairs they are slower (batch 2: 3.49 against 3.30).
WIDE_CLUSTER_SPLITS = 16


# "tcgen05": the 256-row kernel for long portions and the 128-row kernel otherwise; "tcgen05-128" / "tcgen05-256":
# always that kernel; "mma": the mma.sync kernel
PREFILL_KERNEL = os.environ.get("LLMSERVER_B200_PREFILL_ATTENTION", "tcgen05")
PREFILL_TILE = 128   # rows per block of the tcgen05 portions kernel
WIDE_TILE = 256      # rows per block of the 256-row kernel
# the 256-row kernel is used when the longest portion has this many rows (tokens x heads of a group), its request
# holds this many tokens and the group divides 128: measured on the 8B, 14B and 32B head shapes, it wins from about
# there (long key loops, enough row tiles; 8 % at 16384 tokens, 25 % at 32768), and not with groups of 5
WIDE_MIN_ROWS = int(os.environ.get("LLMSERVER_B200_PREFILL_WIDE_ROWS", "8192"))
WIDE_MIN_CONTEXT = int(os.environ.get("LLMSERVER_B200_PREFILL_WIDE_CONTEXT", "16384"))


def prefill_tcgen05_supported(head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int) -> bool:
    return PREFILL_KERNEL.startswith("tcgen05") and bool(
        library().llm_attention_prefill_tcgen05_supports(head_dim, n_q_heads, n_kv_heads, page_size))


FORCE_PAIRING = None     # True / False: tests set it to run both ways of handing out row tiles
_SM_COUNT = {}


def _sm_count(device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _SM_COUNT[index]


def _block_slots(device, wide: bool) -> int:
    """Blocks of a prompt kernel the GPU holds at a time (one per SM for the 256-row kernel, two for the 128-row one)."""
    return _sm_count(device) * (1 if wide else 2)


def prefill_wide_wanted(batch, group: int, head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int) -> bool:
    """Whether the prompt portions of this batch go to the 256-row kernel: when the longest of them has enough
    rows and keys, or when asked for."""
    if PREFILL_KERNEL == "tcgen05-128":
        return False
    if not library().llm_attention_prefill_wide_supports(head_dim, n_q_heads, n_kv_heads, page_size):
        return False
    if PREFILL_KERNEL == "tcgen05-256":
        return True
    length, context = max(zip(batch.q_lens, batch.context_lens))
    return length * group >= WIDE_MIN_ROWS and context >= WIDE_MIN_CONTEXT and PREFILL_TILE % group == 0


def supported(head_dim: int, n_q_heads: int, n_kv_heads: int) -> bool:
    return bool(library().llm_attention_mma_supports(head_dim, n_q_heads, n_kv_heads))


def plan(batch, group: int, n_kv_heads: int, device=None):
    """Launch shape of a batch, derived once per step from its host-side lengths (and the number of SMs: the split
    count fixes the order of the partial sums, so it is a function of the batch and the GPU model only)."""
    key = ("attention_mma", group, n_kv_heads)
    cached = batch.scratch.get(key)
    if cached is not None:
        return cached
    wave_blocks = DECODE_BLOCKS_PER_SM * _sm_count(device if device is not None else batch.context_len.device)
    singles = sum(1 for length in batch.q_lens if length == 1)
    run_decode = singles > 0
    run_portions = singles < batch.n_seqs
    tiles = sum(-(-length * group // TILE) for length in batch.q_lens if length > 1)
    split_len, max_splits = MIN_SPLIT, 1
    if run_decode:
        longest = max(context for context, length in zip(batch.context_lens, batch.q_lens) if length == 1)
        # As many equal splits of the longest context as give about one wave of blocks (two per SM); with a
        # wave's worth of (sequence, kv head) pairs already, no split at all.  Measured on the 8B head shape:
        # equal splits beat ragged ones, and one wave beats one and a half.
        pairs = singles * n_kv_heads
        splits = max(1, min(wave_blocks // pairs, -(-longest // MIN_SPLIT)))
        if CLUSTER_MERGE:
            lone_blocks = pairs * WIDE_CLUSTER_SPLITS <= wave_blocks // DECODE_BLOCKS_PER_SM
            # a cluster has up to 8 blocks, or exactly 16
            splits = WIDE_CLUSTER_SPLITS if lone_blocks and splits > 12 else min(splits, MAX_CLUSTER_SPLITS)
        if pairs > wave_blocks:
            # More than a wave of whole contexts: when the last wave would leave most SMs idle (40 sequences x 8 kv
            # heads = 1.08 waves take as long as 2), the contexts are split after all.  Measured on the 8B head shape at
            # context 3072: unsplit wins while the waves are three quarters full, else the fewest splits that fill
            # them to 0.85 (batch 40: 119 -> 100 us, batch 48: 123 -> 105, batch 80: 182 -> 170).
            def filled(count):
                blocks = pairs * count
                return blocks / (-(-blocks // wave_blocks) * wave_blocks)
            if filled(1) < 0.75:
                candidates = [count for count in (2, 3, 4) if longest // count >= 4 * TILE]
                good = [count for count in candidates if filled(count) >= 0.85]
                if good:
                    splits = good[0]
                elif candidates:
                    splits = max(candidates, key=filled)
        # every sequence is divided into this many equal parts (a negative split length says so to the kernel): the
        # longest gets the planned splits, shorter ones the same number of shorter blocks
        split_len, max_splits = -splits, splits
        forced = os.environ.get("LLMSERVER_B200_DECODE_SPLIT")
        if forced:
            split_len = int(forced)
            max_splits = -(-longest // split_len) + 1     # + 1: a window may start inside a tile
    cached = (run_portions, tiles, run_decode, split_len, max_splits)
    batch.scratch[key] = cached
    return cached


# A decode row's older keys were cached by earlier steps, which lie behind the step's batch copy; the decode kernel may
# start copying them before the kernel in front of it (which writes the newest key) has ended.  Only batches that say
# so (``keys_settled``, set where the engine packs a step) get this.
EARLY_KEYS = os.environ.get("LLMSERVER_B200_DECODE_EARLY_KEYS", "1") != "0"


def try_attention(qkv, q_stride, batch, block_tables, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim, scale, window):
    if not supported(head_dim, n_q_heads, n_kv_heads):
        return None
    check(qkv, "qkv", torch.bfloat16)
    check(k_pages, "k pages", torch.bfloat16, head_dim)
    check(v_pages, "v pages", torch.bfloat16, head_dim)
    check(block_tables, "block_tables", torch.int32)
    run_portions, tiles, run_decode, split_len, max_splits = plan(batch, n_q_heads // n_kv_heads, n_kv_heads, qkv.device)
    out = torch.empty((batch.n_tokens, n_q_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    partial_out = partial_ml = None
    if run_decode and max_splits > 1:
        # scratch of the split-KV decode, shared by every layer of the step
        key = ("attention_mma_scratch", n_q_heads, head_dim, max_splits)
        scratch = batch.scratch.get(key)
        if scratch is None:
            scratch = (torch.empty((batch.n_tokens, n_q_heads, max_splits, head_dim), dtype=torch.float32, device=qkv.device),
                       torch.empty((batch.n_tokens, n_q_heads, max_splits, 2), dtype=torch.float32, device=qkv.device))
            batch.scratch[key] = scratch
        partial_out, partial_ml = scratch
    page_size = k_pages.shape[2]
    flag = wait_error_flag(qkv.device).data_ptr()
    if run_portions and prefill_tcgen05_supported(head_dim, n_q_heads, n_kv_heads, page_size):
        # prompt portions on the tcgen05 kernel (128-row tiles); single tokens, if any, on the decode kernel
        group = n_q_heads // n_kv_heads
        wide = prefill_wide_wanted(batch, group, head_dim, n_q_heads, n_kv_heads, page_size)
        # a tile holds whole tokens: floor(128 / group) of them per 128 rows (the 256-row kernel has two such halves)
        tokens_per_tile = (PREFILL_TILE // group) * (2 if wide else 1)
        tile_counts = [-(-length // tokens_per_tile) for length in batch.q_lens if length > 1 or not run_decode]
        # A block takes a row tile and its mirror image (the light one with the heavy one), which gives every block of a
        # causal prompt the same work, or tiles go out one by one, heaviest first.  Pairs cost whole waves of double
        # blocks; single tiles fill the GPU more finely but end raggedly (about 1.3 x their mean, measured).
        paired = sum((count + 1) // 2 for count in tile_counts)
        slots = _block_slots(qkv.device, wide)
        cost_paired = 2.0 * -(-paired * n_kv_heads // slots)
        cost_single = 1.3 * max(sum(tile_counts) * n_kv_heads / slots, 1.0)
        pairing = cost_paired < cost_single if FORCE_PAIRING is None else FORCE_PAIRING
        call("llm_attention_prefill_wide" if wide else "llm_attention_prefill_tcgen05", qkv.data_ptr(), q_stride, batch.n_tokens,
             k_pages.data_ptr(), v_pages.data_ptr(),
             block_tables.data_ptr(), block_tables.shape[-1], batch.q_start.data_ptr(), batch.context_len.data_ptr(),
             out.data_ptr(), batch.n_seqs, n_q_heads, n_kv_heads, head_dim, page_size, k_pages.shape[0], float(scale), int(window),
             int(run_decode), int(pairing), paired if pairing else sum(tile_counts), flag, stream_handle())
        run_portions = False
        if not run_decode:
            return out
    call("llm_attention_mma", qkv.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), block_tables.data_ptr(),
         block_tables.shape[-1], batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(), batch.n_seqs,
         n_q_heads, n_kv_heads, head_dim, page_size, k_pages.shape[0], float(scale), int(window), int(run_portions), tiles,
         int(run_decode), split_len, max_splits, 0 if partial_out is None else partial_out.data_ptr(),
         0 if partial_ml is None else partial_ml.data_ptr(), int(EARLY_KEYS and getattr(batch, "keys_settled", False)), flag,
         stream_handle())
    return out
