"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory where they call it (an engine that has
given all free memory to its cache, a latency-critical loop, a C program without PyTorch's allocator);
for them ``llm_attention_decode_noalloc`` keeps the split-KV scratch in a fixed array inside the
library.  This test calls it twice in a row with different inputs, through ctypes, and compares each
result with the regular entry point's, which takes its scratch from the caller, and with plain attention
in float64.  It is collected last so that a run that stops at the first failure has already run every
other test."""
import ctypes

import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"


def make_case(seed, contexts, heads, kv_heads, dim, page_size):
    generator = torch.Generator().manual_seed(seed)
    n_seqs = len(contexts)
    pages_per_seq = [-(-c // page_size) for c in contexts]
    n_pages = sum(pages_per_seq) + 1
    k_pages = torch.randn((n_pages, kv_heads, page_size, dim), generator=generator).to(torch.bfloat16).to(DEVICE)
    v_pages = torch.randn((n_pages, kv_heads, page_size, dim), generator=generator).to(torch.bfloat16).to(DEVICE)
    order = torch.randperm(n_pages, generator=generator).tolist()
    tables = torch.zeros((n_seqs, max(pages_per_seq)), dtype=torch.int32)
    for row, count in enumerate(pages_per_seq):
        for block in range(count):
            tables[row, block] = order.pop()
    q_stride = (heads + 2 * kv_heads) * dim
    qkv = torch.randn((n_seqs, q_stride), generator=generator).to(torch.bfloat16).to(DEVICE)
    return qkv, q_stride, k_pages, v_pages, tables.to(DEVICE)


def plain_decode_attention(qkv, k_pages, v_pages, tables, contexts, heads, kv_heads, dim, page_size, scale, window):
    """float64 attention of each sequence's last position over its pages, by the plain implementation."""
    rows = []
    tables = tables.cpu()
    for row, context in enumerate(contexts):
        pages = tables[row, :-(-context // page_size)].long()
        keys = k_pages.cpu()[pages].permute(0, 2, 1, 3).reshape(-1, kv_heads, dim)[:context].double()
        values = v_pages.cpu()[pages].permute(0, 2, 1, 3).reshape(-1, kv_heads, dim)[:context].double()
        queries = torch.zeros((context, heads, dim), dtype=torch.float64)
        queries[-1] = qkv[row, :heads * dim].cpu().double().reshape(heads, dim)
        rows.append(plain_model.causal_attention(queries, keys, values, scale, window or None)[-1].reshape(-1))
    return torch.stack(rows)


class Batch:
    def __init__(self, contexts):
        self.q_lens, self.context_lens = [1] * len(contexts), list(contexts)
        self.n_seqs = self.n_tokens = len(contexts)
        self.q_start = torch.arange(len(contexts) + 1, dtype=torch.int32, device=DEVICE)
        self.context_len = torch.tensor(contexts, dtype=torch.int32, device=DEVICE)
        self.scratch = {}


def test_no_alloc_decode_attention_matches_the_regular_entry_point_twice_in_a_row():
    from llmserver_b200.ops import attention_bf16
    from llmserver_b200.ops.library import library

    lib = library()
    entry = lib.llm_attention_decode_noalloc          # the exported C symbol
    pointer, integer = ctypes.c_void_p, ctypes.c_int
    entry.argtypes = [pointer, integer, pointer, pointer, pointer, integer, pointer, pointer, pointer, integer, integer,
                      integer, integer, integer, integer, ctypes.c_float, integer, integer, integer, pointer]
    entry.restype = integer
    status_of = lib.llm_attention_decode_noalloc_status
    status_of.argtypes, status_of.restype = [pointer], integer
    heads, kv_heads, dim, page_size = 8, 2, 128, 16
    scale = dim ** -0.5
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, contexts, window) in enumerate(((1, [1500, 300, 64, 1, 777], 0), (2, [40, 1290, 513, 1024, 2], 600))):
        qkv, q_stride, k_pages, v_pages, tables = make_case(seed, contexts, heads, kv_heads, dim, page_size)
        batch = Batch(contexts)
        expected = attention_bf16.try_attention(qkv, q_stride, batch, tables, k_pages, v_pages, heads, kv_heads, dim,
                                                scale, window)
        _, _, _, split_len, max_splits = attention_bf16.plan(batch, heads // kv_heads, kv_heads, qkv.device)
        assert max_splits > 1, "the case is meant to use the scratch memory"
        out = torch.full_like(expected, float("nan"))
        status = entry(qkv.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), tables.data_ptr(),
                       tables.shape[1], batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(),
                       len(contexts), heads, kv_heads, dim, page_size, k_pages.shape[0], scale, window, split_len,
                       max_splits, stream)
        assert status == 0, lib.llm_last_error().decode()
        assert status_of(stream) == 0
        assert torch.isfinite(out.float()).all()
        error = (out.float() - expected.float()).abs().max().item() / expected.float().abs().max().item()
        assert error <= 1e-2, f"call {call}: relative error {error:.3e}"
        plain = plain_decode_attention(qkv, k_pages, v_pages, tables, contexts, heads, kv_heads, dim, page_size, scale, window)
        error = (out.cpu().double() - plain).abs().max().item() / plain.abs().max().item()
        assert error <= 1e-2, f"call {call}: relative error {error:.3e} against plain attention"
    # a request beyond the fixed array is refused with a message, not run
    status = entry(qkv.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), tables.data_ptr(), tables.shape[1],
                   batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(), len(contexts), heads,
                   kv_heads, dim, page_size, k_pages.shape[0], scale, 0, 64, 4096, stream)
    assert status == -1 and b"scratch" in lib.llm_last_error()
    # a table entry that names no page of the pool is not followed (zeros are read), and the status word says so;
    # too few splits for a context are reported too
    tables[1, 0] = k_pages.shape[0] + 7
    status = entry(qkv.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), tables.data_ptr(), tables.shape[1],
                   batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(), len(contexts), heads,
                   kv_heads, dim, page_size, k_pages.shape[0], scale, 0, split_len, max_splits, stream)
    assert status == 0 and status_of(stream) == 5
    assert torch.isfinite(out.float()).all()
    tables[1, 0] = 0
    status = entry(qkv.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), tables.data_ptr(), tables.shape[1],
                   batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(), len(contexts), heads,
                   kv_heads, dim, page_size, k_pages.shape[0], scale, 0, 256, 2, stream)
    assert status == 0 and status_of(stream) == 6
