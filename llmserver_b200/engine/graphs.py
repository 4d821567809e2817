"""CUDA graphs for decode steps.

A decode step launches a couple of hundred small kernels; issued one by one from Python they cost
more host time than the GPU needs to run them (the reference met the same wall and replays one graph
per batch-size bucket: utils/cuda_graph.py:3-4,11-99).  Here a step's whole input is one packed int32
buffer whose layout depends only on the batch size, so a graph is captured once per batch size over a
fixed device buffer; a replayed step is: pack on the host (pinned) -> one copy -> replay -> read the
sampled tokens (and the kernels' error flag) back in one copy.

The captured attention launch is shaped for the longest context the runner was sized for; blocks
beyond a sequence's real length exit at once.  Nothing is executed during capture, and the warm-up
that a capture needs is given by the eager steps of the same batch size that ran before it.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..ops.library import wait_error_flag
from .batch import BatchLayout, SequenceSlice, pack, views


BUCKETS = (1, 2, 4, 8, 16, 32, 48, 64, 96, 128, 192, 256)   # batch sizes graphs are captured for


class _PadRow:
    temperature, seed, step = 0.0, 0, 0


class DecodeRows:
    """Host half of a replayed decode step: the packed batch of ``batch_size`` rows in a host buffer that is
    rewritten as little as possible from step to step.

    A row is recognised by the *identity* of its block-table lists, not by its request id: the cache manager
    makes new lists when a request is admitted and drops them when it is freed, so a request that was preempted
    and recomputed into other pages comes back with other lists even under the same id in the same row.  The lists
    of the last packed step are held here, which also keeps their ``id()`` from being reused.  On a match only
    what a decode step changes is rewritten (``_update``); anything else repacks the whole buffer."""

    def __init__(self, batch_size: int, n_groups: int, table_width: int, vocab_size: int, null_pages: Sequence[int],
                 host_view: Optional[np.ndarray] = None):
        self.batch_size, self.vocab_size = batch_size, vocab_size
        self.layout = BatchLayout(batch_size, batch_size, batch_size, (table_width,) * n_groups)
        self.host_view = np.zeros(self.layout.total, dtype=np.int32) if host_view is None else host_view
        self.pad = SequenceSlice(None, [0], 0, [0], [[page] for page in null_pages], 0)
        self.row_tables: Optional[List[Sequence[Sequence[int]]]] = None
        self.table_lengths: Optional[List[List[int]]] = None
        self.repacks = 0

    def forget(self) -> None:
        """Whatever the buffer holds is not trusted any more: the next step packs all of it."""
        self.row_tables, self.table_lengths = None, None

    def _same_rows(self, slices: List[SequenceSlice]) -> bool:
        if self.row_tables is None:
            return False
        for piece, remembered, lengths in zip(slices, self.row_tables, self.table_lengths):
            if len(piece.tables) != len(remembered):
                return False
            for table, known, length in zip(piece.tables, remembered, lengths):
                if table is not known or len(table) < length:
                    return False
        return True

    def fill(self, slices: List[SequenceSlice], sampling: Sequence) -> int:
        """Brings the host buffer up to date for this step; returns the number of real rows."""
        real = len(slices)
        if real > self.batch_size:
            raise ValueError(f"{real} requests do not fit a decode step of {self.batch_size} rows")
        if real < self.batch_size:
            slices = list(slices) + [self.pad] * (self.batch_size - real)
            sampling = list(sampling) + [_PadRow] * (self.batch_size - real)
        if self._same_rows(slices):
            self._update(slices, sampling)
        else:
            pack(slices, self.layout, self.host_view, self.vocab_size, sampling)
            self.row_tables = [list(piece.tables) for piece in slices]
            self.table_lengths = [[len(table) for table in piece.tables] for piece in slices]
            self.repacks += 1
        return real

    def _update(self, slices: List[SequenceSlice], sampling: Sequence) -> None:
        """The same rows as the step before: the token, the position, the sampling inputs and block-table entries
        of pages that were added are rewritten; older table entries are already in the buffer.  (A windowed group
        marks pages it gave back in its list; the buffer keeps their old ids, which the kernels mask and never
        write to.)"""
        host, off, count = self.host_view, self.layout.offsets, len(slices)
        tokens = np.fromiter((piece.tokens[0] for piece in slices), dtype=np.int64, count=count)
        if tokens.min() < 0 or tokens.max() >= self.vocab_size:
            raise ValueError(f"a token id is outside the vocabulary of {self.vocab_size}")
        starts = np.fromiter((piece.start for piece in slices), dtype=np.int32, count=count)
        host[off["token_ids"]:off["token_ids"] + count] = tokens
        host[off["positions"]:off["positions"] + count] = starts
        host[off["context_len"]:off["context_len"] + count] = starts + 1
        host[off["temperatures"]:off["temperatures"] + count] = np.fromiter(
            (row.temperature for row in sampling), dtype=np.float32, count=count).view(np.int32)
        host[off["seeds"]:off["seeds"] + 2 * count] = np.fromiter(
            (row.seed & 0x7FFFFFFFFFFFFFFF for row in sampling), dtype=np.int64, count=count).view(np.int32)
        host[off["sample_steps"]:off["sample_steps"] + count] = np.fromiter((row.step for row in sampling), dtype=np.int32, count=count)
        host[off["error_flag"]] = 0
        for row, piece in enumerate(slices):
            lengths = self.table_lengths[row]
            for group, table in enumerate(piece.tables):
                if len(table) != lengths[group]:
                    width, begin = self.layout.widths[group], self.layout.table_offsets[group] + row * self.layout.widths[group]
                    if len(table) > width:
                        raise ValueError(f"request {piece.request_id!r} holds {len(table)} pages; the graph has room for {width}")
                    fresh = np.asarray(table[lengths[group]:], dtype=np.int32)
                    host[begin + lengths[group]:begin + len(table)] = np.maximum(fresh, 0)
                    lengths[group] = len(table)


class DecodeGraph:
    """A captured decode step for ``batch_size`` rows.  Steps with fewer requests are padded: the extra
    rows decode token 0 at position 0 of a page that belongs to no request (``null_pages``) and their
    sampled tokens are dropped, as the reference pads its buckets with copies of row 0
    (utils/cuda_graph.py:11-99)."""

    def __init__(self, model, batch_size: int, n_groups: int, table_width: int, max_context: int, vocab_size: int,
                 null_pages: Sequence[int]):
        self.model, self.vocab_size, self.batch_size = model, vocab_size, batch_size
        device = model.runtime.device
        layout = BatchLayout(batch_size, batch_size, batch_size, (table_width,) * n_groups)
        self.host = torch.zeros(layout.total, dtype=torch.int32, pin_memory=True)
        self.rows = DecodeRows(batch_size, n_groups, table_width, vocab_size, null_pages, self.host.numpy())
        self.layout = self.rows.layout
        self.buffer = torch.zeros(self.layout.total, dtype=torch.int32, device=device)
        # the static batch claims the longest context, so that launch shapes cover every later step
        shape_only = [SequenceSlice(index, [0], max_context - 1, [0], [[0] * table_width] * n_groups, 0)
                      for index in range(batch_size)]
        self.batch = views(self.buffer, self.layout, shape_only)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            logits = self.model.step(self.batch)
            self.logits = logits        # [batch_size, vocab] of the last replay (tests compare them with eager steps)
            tokens = ops.sample(logits, self.batch.temperatures, self.batch.seeds, self.batch.sample_steps)
            self.result = torch.cat([tokens, self.batch.error_flag, wait_error_flag(device)])

    def run(self, slices: List[SequenceSlice], sampling: Sequence, phases: Optional[dict] = None) -> List[int]:
        """Returns the sampled tokens of the real rows followed by the two error flags; ``phases`` receives the host
        seconds spent packing and queueing the copy, replaying, and waiting for the result."""
        clock = time.perf_counter
        self.began = clock()
        real = self.rows.fill(slices, sampling)
        self.buffer.copy_(self.host, non_blocking=True)
        packed = clock()
        self.graph.replay()
        launched = clock()
        result = self.result.tolist()
        if phases is not None:
            phases.update(pack_copy=packed - self.began, launch=launched - packed, read_back=clock() - launched)
        return result[:real] + result[-2:]


class DecodeGraphs:
    """One graph per batch-size bucket, captured the third time the bucket is needed (the two eager steps
    before it warm the kernels up and let the matrix products choose their variants)."""

    WARM_STEPS = 2

    def __init__(self, model, cache, max_context: int, max_batch: int = 256):
        self.model, self.cache = model, cache
        self.max_context, self.max_batch = max_context, max_batch
        self.table_width = -(-max_context // cache.page_size)
        self.graphs: Dict[int, DecodeGraph] = {}
        self.seen: Dict[int, int] = {}
        # every mixer has to say that it can be captured; and rows that only pad a batch would have to own a state
        # slot, which the slot allocator does not set aside
        mixers = [getattr(layer, "mixer", None) for layer in getattr(model, "layers", [])]
        self.failed = bool(cache.state_entries) or any(not getattr(mixer, "capturable", True) for mixer in mixers)
        self.null_pages = None

    def forget_rows(self) -> None:
        """Called when a request gives its pages back: no graph may go on trusting the block tables in its buffer."""
        for graph in self.graphs.values():
            graph.rows.forget()

    def bucket_for(self, size: int) -> int:
        for bucket in BUCKETS:
            if size <= bucket and (bucket <= self.max_batch or bucket == size):
                return bucket
        return size

    def ready_for(self, slices: List[SequenceSlice]):
        """The graph that can run this step, or None (then the step runs eagerly)."""
        if self.failed or len(slices) > self.max_batch:
            return None
        for piece in slices:
            if len(piece.tokens) != 1 or len(piece.want) != 1 or piece.start + 1 > self.max_context:
                return None
        size = self.bucket_for(len(slices))
        graph = self.graphs.get(size)
        if graph is not None:
            return graph
        self.seen[size] = self.seen.get(size, 0) + 1
        if self.seen[size] <= self.WARM_STEPS:
            return None
        if self.null_pages is None:
            try:
                self.null_pages = self.cache.reserve_null_pages()
            except BufferError:          # no page to spare: go on without graphs
                self.failed = True
                return None
        self.graphs[size] = self.capture(size)
        return self.graphs[size]

    def capture(self, size: int):
        """Makes the replayable step for ``size`` rows (tests without a GPU put a host-side stand-in here)."""
        return DecodeGraph(self.model, size, len(self.cache.groups), self.table_width, self.max_context,
                           self.model.spec.vocab_size, self.null_pages)
