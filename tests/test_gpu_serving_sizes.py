"""The kernels and launch plans that serving picks by itself at real sizes, which the tiny configurations never
reach: the 256-row prompt kernel (long portions over long contexts), the 128-row prompt kernel on thousands of
rows with both ways of handing out tiles, the decode plan with more (sequence, kv head) pairs than one wave of
blocks, and replayed decode steps of 8, 16 and 64 rows at the 8B layer sizes.

Queries are scaled so that every row's softmax is carried by a few keys at random places of the context: a key tile
that is skipped, read twice or taken from the wrong page changes the row visibly, which a flat softmax over
thousands of keys would hide."""
import numpy as np
import pytest
import torch

from helpers import tokens_for

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


class HostBatch:
    """What the attention wrapper reads of a step's batch."""

    def __init__(self, q_lens, contexts):
        self.q_lens, self.context_lens = list(q_lens), list(contexts)
        self.n_seqs, self.n_tokens = len(q_lens), sum(q_lens)
        starts = np.concatenate([[0], np.cumsum(q_lens)])
        self.q_start = torch.tensor(starts, dtype=torch.int32, device=DEVICE)
        self.context_len = torch.tensor(contexts, dtype=torch.int32, device=DEVICE)
        self.token_ids = self.q_start
        self.scratch = {}


def paged_case(seed, q_lens, contexts, heads, kv_heads, dim, page_size, sharpness=3.0):
    """Random K/V of every sequence scattered over a shuffled page pool, and the packed Q of the step's tokens."""
    generator = torch.Generator(device=DEVICE).manual_seed(seed)
    pages_per_seq = [-(-context // page_size) for context in contexts]
    n_pages = sum(pages_per_seq) + 3
    k_pages = torch.randn((n_pages, kv_heads, page_size, dim), generator=generator, device=DEVICE, dtype=torch.float32).to(torch.bfloat16)
    v_pages = torch.randn((n_pages, kv_heads, page_size, dim), generator=generator, device=DEVICE, dtype=torch.float32).to(torch.bfloat16)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    tables = torch.zeros((len(contexts), max(pages_per_seq)), dtype=torch.int32)
    for row, count in enumerate(pages_per_seq):
        tables[row, :count] = torch.tensor([order.pop() for _ in range(count)], dtype=torch.int32)
    q_stride = (heads + 2 * kv_heads) * dim
    qkv = torch.randn((sum(q_lens), q_stride), generator=generator, device=DEVICE, dtype=torch.float32)
    qkv[:, :heads * dim] *= sharpness
    return qkv.to(torch.bfloat16), q_stride, k_pages, v_pages, tables.to(DEVICE)


def plain_rows(qkv, k_pages, v_pages, table, context, first_position, rows, heads, kv_heads, dim, page_size, scale, token_offset):
    """float64 attention of the step's tokens ``rows`` (indices into the sequence's tokens of this step) over the
    sequence's keys, computed on the GPU a block of rows at a time: [len(rows), heads * dim]."""
    pages = table[:-(-context // page_size)].long()
    keys = k_pages[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, dim)[:, :context].double()      # [kv, T, D]
    values = v_pages[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, dim)[:, :context].double()
    group = heads // kv_heads
    rows = torch.as_tensor(rows, device=DEVICE)
    queries = qkv[token_offset + rows, :heads * dim].double().reshape(len(rows), kv_heads, group, dim)
    scores = torch.einsum("rkgd,ktd->rkgt", queries, keys) * scale
    positions = first_position + rows
    visible = torch.arange(context, device=DEVICE)[None, :] <= positions[:, None]
    scores = scores.masked_fill(~visible[:, None, None, :], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    return torch.einsum("rkgt,ktd->rkgd", weights, values).reshape(len(rows), heads * dim)


def relative_error(got, want):
    return ((got.double() - want).abs().max() / want.abs().max()).item()


@pytest.mark.parametrize("portion,context,wide,pairing", [
    (8192, 8192, False, True), (8192, 8192, False, False),     # a whole long prompt on the 128-row kernel
    (2048, 16384, True, None), (2048, 32768, True, True), (2048, 32768, True, False)])
def test_prompt_attention_at_the_sizes_serving_selects_it(portion, context, wide, pairing):
    """8B head shape (groups of 4 heads of 128, pages of 16) with two kv heads.  Nothing is forced but the way tiles
    are handed out: the wrapper itself must pick the 256-row kernel for a 2048-token portion at the end of 16384 and
    32768 tokens, and the 128-row kernel for the whole prompt of 8192."""
    from llmserver_b200.ops import attention_bf16
    heads, kv_heads, dim, page_size = 8, 2, 128, 16
    scale = dim ** -0.5
    batch = HostBatch([portion], [context])
    qkv, q_stride, k_pages, v_pages, tables = paged_case(context + portion, [portion], [context], heads, kv_heads, dim, page_size)
    assert attention_bf16.prefill_tcgen05_supported(dim, heads, kv_heads, page_size)
    assert attention_bf16.prefill_wide_wanted(batch, heads // kv_heads, dim, heads, kv_heads, page_size) == wide
    attention_bf16.FORCE_PAIRING = pairing
    try:
        out = attention_bf16.try_attention(qkv, q_stride, batch, tables, k_pages, v_pages, heads, kv_heads, dim, scale, 0)
    finally:
        attention_bf16.FORCE_PAIRING = None
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    # the first, a middle and the last tile of rows (a tile of the 256-row kernel holds 64 tokens of a group of 4),
    # and rows around the tile edges
    tile = 64 if wide else 32
    middle = (portion // tile // 2) * tile
    picked = sorted(set(list(range(0, tile + 2)) + list(range(middle - 2, middle + tile + 2)) +
                        list(range(portion - tile - 2, portion))))
    want = plain_rows(qkv, k_pages, v_pages, tables[0], context, context - portion, picked, heads, kv_heads, dim, page_size, scale, 0)
    error = relative_error(out[picked], want)
    assert error <= 2e-2, f"relative error {error:.3e}"
    # every row against a coarse check: the rows between the picked tiles, one in 97
    others = list(range(1, portion, 97))
    want = plain_rows(qkv, k_pages, v_pages, tables[0], context, context - portion, others, heads, kv_heads, dim, page_size, scale, 0)
    error = relative_error(out[others], want)
    assert error <= 2e-2, f"relative error {error:.3e} on the sampled rows"
    from llmserver_b200.ops.library import check_wait_errors
    check_wait_errors()


@pytest.mark.parametrize("n_seqs,expected_parts", [(40, 4), (48, 2), (64, 1), (37, 1)])
def test_decode_attention_with_more_pairs_than_a_wave(n_seqs, expected_parts):
    """8B head shape, 8 kv heads, ragged contexts from 1 to 4096 tokens: with 40, 48 and 64 sequences there are more
    (sequence, kv head) pairs than blocks in one wave, and the plan divides every context into 4, 2 and 1 parts on a
    GPU of 148 SMs (37 sequences are exactly one wave and stay whole)."""
    from llmserver_b200.ops import attention_bf16
    heads, kv_heads, dim, page_size = 32, 8, 128, 16
    scale = dim ** -0.5
    rng = np.random.default_rng(n_seqs)
    contexts = [int(value) for value in rng.integers(1, 4097, size=n_seqs)]
    contexts[0], contexts[1], contexts[2], contexts[3] = 4096, 1, 65, 1024
    batch = HostBatch([1] * n_seqs, contexts)
    qkv, q_stride, k_pages, v_pages, tables = paged_case(n_seqs, [1] * n_seqs, contexts, heads, kv_heads, dim, page_size)
    _, _, run_decode, split_len, max_splits = attention_bf16.plan(batch, heads // kv_heads, kv_heads, qkv.device)
    assert run_decode
    if torch.cuda.get_device_properties(0).multi_processor_count == 148:
        assert max_splits == expected_parts and split_len == -expected_parts
    out = attention_bf16.try_attention(qkv, q_stride, batch, tables, k_pages, v_pages, heads, kv_heads, dim, scale, 0)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    worst = 0.0
    for row, context in enumerate(contexts):
        want = plain_rows(qkv, k_pages, v_pages, tables[row], context, context - 1, [0], heads, kv_heads, dim, page_size, scale, row)
        worst = max(worst, relative_error(out[row:row + 1], want))
    assert worst <= 2e-2, f"relative error {worst:.3e}"
    from llmserver_b200.ops.library import check_wait_errors
    check_wait_errors()


def test_attention_does_not_follow_table_entries_outside_the_pool():
    """Entries past a context's end that name no page (-1, or an id beyond the pool) are read as zeros and masked;
    the result is that of a clean table, and the error flag says that such an entry was met."""
    from llmserver_b200.ops import attention_bf16
    from llmserver_b200.ops.library import wait_error_flag
    heads, kv_heads, dim, page_size = 8, 2, 128, 16
    scale = dim ** -0.5
    contexts = [100, 40, 3]            # the last 64-key tile of each reaches past the context's last page
    batch = HostBatch([1, 1, 1], contexts)
    qkv, q_stride, k_pages, v_pages, tables = paged_case(5, [1, 1, 1], contexts, heads, kv_heads, dim, page_size)
    clean = attention_bf16.try_attention(qkv, q_stride, batch, tables, k_pages, v_pages, heads, kv_heads, dim, scale, 0)
    wide_tables = torch.zeros((3, 8), dtype=torch.int32, device=DEVICE)
    wide_tables[:, :tables.shape[1]] = tables
    for row, context in enumerate(contexts):
        used = -(-context // page_size)
        wide_tables[row, used:] = torch.tensor([-1, k_pages.shape[0] + 5, 1 << 20, -7, 0, 0, 0, 0][:8 - used], dtype=torch.int32)
    flag = wait_error_flag(qkv.device)
    flag.zero_()
    batch = HostBatch([1, 1, 1], contexts)
    dirty = attention_bf16.try_attention(qkv, q_stride, batch, wide_tables, k_pages, v_pages, heads, kv_heads, dim, scale, 0)
    torch.cuda.synchronize()
    assert torch.isfinite(dirty.float()).all()
    assert torch.equal(dirty, clean)
    assert int(flag.item()) == 5
    flag.zero_()


CONFIG_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
                 intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                 rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960,
                 hidden_act="silu", attention_bias=False, use_sliding_window=False)


def test_replayed_decode_steps_give_the_logits_of_eager_steps_at_8b_sizes():
    """Two layers of the 8B sizes in bfloat16, decode steps of 8, 16 and 64 rows: the logits a captured graph leaves
    are compared with the logits of the same step launched kernel by kernel (same tokens, same cache), and the
    sampled tokens with their argmax."""
    from llmserver_b200.cache import CacheManager
    from llmserver_b200.config import Qwen3Config
    from llmserver_b200.engine.step import StepFunction
    from llmserver_b200.models import random_model
    from llmserver_b200.sampling import SamplingRow

    model = random_model(Qwen3Config.from_dict(CONFIG_8B), seed=5, dtype="bfloat16", device=DEVICE)
    vocab = 151936
    for rows in (8, 16, 64):
        cache = CacheManager(model.cache_needs(), 16, rows * 20 + 8, num_slots=rows, prefix_sharing=False)
        cache.materialize(model.runtime.device, model.runtime.dtype)
        step = StepFunction(model, cache)
        step.enable_graphs(320, rows)
        names = [f"r{index}" for index in range(rows)]
        greedy = [SamplingRow() for _ in names]
        last = []
        for index, name in enumerate(names):
            step.admit(name)
            prompt = tokens_for(vocab, 5 + (index * 37) % 230, 1000 * rows + index)
            last.append(step.run_and_sample([(name, prompt, [len(prompt) - 1])], [SamplingRow()])[0])
        compared = 0
        for _ in range(6):
            entries = [(name, [token], [0]) for name, token in zip(names, last)]
            eager_batch = step.prepare(entries, greedy)
            eager = model.step(eager_batch).float().clone()       # writes this step's keys and values; the replay rewrites them
            replayed_before = step.graph_steps
            last = step.run_and_sample(entries, greedy)
            if step.graph_steps > replayed_before:
                graph = step.graphs.graphs[rows]
                logits = graph.logits[:rows].float()
                scale = eager.abs().max(dim=-1, keepdim=True).values
                error = ((logits - eager).abs().max(dim=-1, keepdim=True).values / scale).max().item()
                assert error <= 2e-2, f"{rows} rows: replayed logits differ from eager logits by {error:.3e}"
                assert last == logits.argmax(dim=-1).tolist()
                compared += 1
        assert compared >= 3, f"{rows} rows: the graph was meant to be replayed"
        for name in names:
            step.release(name)
        step.check_errors()
        cache.check_invariants()
        del step, cache
        torch.cuda.empty_cache()
