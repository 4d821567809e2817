"""The host bookkeeping of replayed decode steps, without a GPU: the packed buffer that a captured step reads must
name every row's real pages on every step, also after a request was preempted, recomputed into other pages and put
back into the same row under the same id."""
import random
import time

import numpy as np
import torch

from llmserver_b200.engine.batch import SequenceSlice
from llmserver_b200.engine.engine import Engine
from llmserver_b200.engine.graphs import DecodeGraphs, DecodeRows
from llmserver_b200.sampling import SamplingRow
from stubs import VOCAB, StubModel, expected_generation


def tables_in(rows: DecodeRows, row: int, group: int, count: int):
    begin = rows.layout.table_offsets[group] + row * rows.layout.widths[group]
    return rows.host_view[begin:begin + count].tolist()


def test_same_id_with_other_pages_is_packed_again():
    rows = DecodeRows(batch_size=4, n_groups=1, table_width=6, vocab_size=100, null_pages=[31])
    sampling = [SamplingRow()] * 3
    a, b, c = [1, 2], [3, 4], [7, 8, 9]
    step = [SequenceSlice("A", [5], 6, [0], [a]), SequenceSlice("B", [5], 7, [0], [b]), SequenceSlice("C", [5], 9, [0], [c])]
    assert rows.fill(step, sampling) == 3 and rows.repacks == 1
    assert tables_in(rows, 2, 0, 3) == [7, 8, 9] and tables_in(rows, 3, 0, 1) == [31]
    # the same rows one token later: a page is appended to A's own list; nothing else is packed again
    a.append(12)
    step = [SequenceSlice("A", [6], 8, [0], [a]), SequenceSlice("B", [6], 8, [0], [b]), SequenceSlice("C", [6], 10, [0], [c])]
    rows.fill(step, sampling)
    assert rows.repacks == 1 and tables_in(rows, 0, 0, 3) == [1, 2, 12]
    # C was preempted and recomputed: same id, same row, same length, other pages in another list
    step[2] = SequenceSlice("C", [6], 11, [0], [[20, 21, 22]])
    rows.fill(step, sampling)
    assert rows.repacks == 2 and tables_in(rows, 2, 0, 3) == [20, 21, 22]
    # an equal list that is not the same object is not trusted either
    step[1] = SequenceSlice("B", [6], 8, [0], [list(b)])
    rows.fill(step, sampling)
    assert rows.repacks == 3
    rows.forget()
    rows.fill(step, sampling)
    assert rows.repacks == 4
    # what every step rewrites
    off = rows.layout.offsets
    assert rows.host_view[off["positions"]:off["positions"] + 4].tolist() == [8, 8, 11, 0]
    assert rows.host_view[off["context_len"]:off["context_len"] + 4].tolist() == [9, 9, 12, 1]


class HostStep:
    """Stands in for a captured step: it reads the packed buffer as the kernels would and applies the stub model's
    rule, after checking that the buffer names the pages the cache manager really gave each request."""

    def __init__(self, owner, size):
        self.owner = owner
        cache = owner.cache
        self.rows = DecodeRows(size, len(cache.groups), owner.table_width, VOCAB, owner.null_pages)
        self.layout = self.rows.layout

    def run(self, slices, sampling, phases=None):
        self.began = time.perf_counter()
        real = self.rows.fill(slices, sampling)
        off = self.layout.offsets
        host = self.rows.host_view
        for row, piece in enumerate(slices):
            for group, table in enumerate(piece.tables):
                used = -(-(piece.start + 1) // self.owner.cache.page_size)
                assert tables_in(self.rows, row, group, used) == [max(page, 0) for page in table[:used]], \
                    f"row {row} ({piece.request_id}): the buffer names other pages than the request holds"
            assert host[off["positions"] + row] == piece.start and host[off["token_ids"] + row] == piece.tokens[0]
        self.owner.checked += 1
        tokens = [(int(host[off["token_ids"] + row]) + 1 + int(host[off["positions"] + row])) % VOCAB for row in range(real)]
        return tokens + [0, 0]


class HostGraphs(DecodeGraphs):
    checked = 0

    def capture(self, size):
        return HostStep(self, size)


class DeviceStyleSampler:
    """Has ``from_batch`` like the device sampler, so the step function takes its graph path."""

    def from_batch(self, logits, batch):
        return torch.argmax(logits, dim=-1).to(torch.int32)


def test_buffer_tables_follow_the_cache_under_random_schedules_with_preemption():
    preempted_and_replayed = 0
    for seed in range(120):
        rng = random.Random(seed)
        engine = Engine(StubModel(), max_new_tokens=16, max_batch_size=4, max_num_batched_tokens=24,
                        kv_cache_num_blocks=rng.randint(9, 14), kv_cache_block_size=4, ignore_eos=True, prefix_caching=False,
                        sampler=DeviceStyleSampler(), cuda_graphs=False, max_context=64)
        graphs = HostGraphs(engine.model, engine.cache, 64, 4)
        engine.step_function.graphs = graphs
        jobs = [(rng.randint(0, 25), [rng.randrange(VOCAB) for _ in range(rng.randint(1, 12))], rng.randint(1, 16))
                for _ in range(10)]
        requests, step = {}, 0
        while len(requests) < len(jobs) or engine.scheduler.waiting or engine.scheduler.running:
            for index, (arrives, prompt, new) in enumerate(jobs):
                if index not in requests and arrives <= step:
                    requests[index] = engine.add_request(prompt_token_ids=prompt, max_new_tokens=new)
            engine.step()
            step += 1
            assert step < 2000
        for index, (_, prompt, new) in enumerate(jobs):
            assert requests[index].generated_token_ids == expected_generation(prompt, new)
        engine.cache.check_invariants()
        if engine.stats["preemptions"] and graphs.checked:
            preempted_and_replayed += 1
    assert preempted_and_replayed > 20, "the schedules were meant to preempt while steps are replayed"


def test_a_request_that_returns_to_its_row_after_being_put_out():
    """Three decoders in a bucket of four.  The youngest is put out between two replayed steps, waits at the head of
    the queue, has its cache rebuilt in other pages and comes back to the same row beside the same neighbours: the
    replayed step has to read its new pages."""
    engine = Engine(StubModel(), max_new_tokens=30, max_batch_size=4, max_num_batched_tokens=64, kv_cache_num_blocks=24,
                    kv_cache_block_size=4, ignore_eos=True, prefix_caching=False, sampler=DeviceStyleSampler(),
                    cuda_graphs=False, max_context=64)
    graphs = HostGraphs(engine.model, engine.cache, 64, 4)
    engine.step_function.graphs = graphs
    prompts = [[1, 2, 3], [4, 5, 6], [7, 8, 9, 10, 11]]
    decoders = [engine.add_request(prompt_token_ids=prompt, max_new_tokens=14) for prompt in prompts]
    for _ in range(6):
        engine.step()
    replayed_before = graphs.checked
    assert replayed_before > 0 and engine.stats["preemptions"] == 0
    old_pages = list(engine.cache.table(decoders[2].request_id))
    engine.put_out(decoders[2])
    assert engine.scheduler.waiting[0] is decoders[2] and decoders[2].replaying
    engine.step()          # the cache of the request is rebuilt beside two decode tokens
    assert decoders[2].status.value == "Decoding" and not decoders[2].replaying
    assert list(engine.cache.table(decoders[2].request_id)) != old_pages
    engine.step()
    assert graphs.checked == replayed_before + 1 and graphs.graphs[4].rows.repacks >= 2
    while engine.step():
        pass
    for prompt, request in zip(prompts, decoders):
        assert request.generated_token_ids == expected_generation(prompt, 14)
    assert decoders[2].times_put_out == 1
