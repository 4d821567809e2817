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

from typing import Dict, List, Sequence

import numpy as np
import torch

from .. import ops
from ..ops.library import wait_error_flag
from .batch import BatchLayout, SequenceSlice, pack, views


BUCKETS = (1, 2, 4, 8, 16, 32, 48, 64, 96, 128, 192, 256)   # batch sizes graphs are captured for


class _PadRow:
    temperature, seed, step = 0.0, 0, 0


class DecodeGraph:
    """A captured decode step for ``batch_size`` rows.  Steps with fewer requests are padded: the extra
    rows decode token 0 at position 0 of a page that belongs to no request (``null_pages``) and their
    sampled tokens are dropped, as the reference pads its buckets with copies of row 0
    (utils/cuda_graph.py:11-99)."""

    def __init__(self, model, batch_size: int, n_groups: int, table_width: int, max_context: int, vocab_size: int,
                 null_pages: Sequence[int]):
        self.model, self.vocab_size, self.batch_size = model, vocab_size, batch_size
        self.layout = BatchLayout(batch_size, batch_size, batch_size, (table_width,) * n_groups)
        device = model.runtime.device
        self.host = torch.zeros(self.layout.total, dtype=torch.int32, pin_memory=True)
        self.host_view = self.host.numpy()
        self.buffer = torch.zeros(self.layout.total, dtype=torch.int32, device=device)
        self.pad = SequenceSlice(None, [0], 0, [0], [[page] for page in null_pages], 0)
        # the static batch claims the longest context, so that launch shapes cover every later step
        shape_only = [SequenceSlice(index, [0], max_context - 1, [0], [[0] * table_width] * n_groups, 0)
                      for index in range(batch_size)]
        self.batch = views(self.buffer, self.layout, shape_only)
        self.row_ids, self.table_lengths = None, None
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            logits = self.model.step(self.batch)
            tokens = ops.sample(logits, self.batch.temperatures, self.batch.seeds, self.batch.sample_steps)
            self.result = torch.cat([tokens, self.batch.error_flag, wait_error_flag(device)])

    def run(self, slices: List[SequenceSlice], sampling: Sequence) -> List[int]:
        """Returns the sampled tokens of the real rows followed by the two error flags."""
        real = len(slices)
        if real < self.batch_size:
            slices = list(slices) + [self.pad] * (self.batch_size - real)
            sampling = list(sampling) + [_PadRow] * (self.batch_size - real)
        ids = [piece.request_id for piece in slices]
        if ids != self.row_ids:
            pack(slices, self.layout, self.host_view, self.vocab_size, sampling)
            self.row_ids = ids
            self.table_lengths = [[len(table) for table in piece.tables] for piece in slices]
        else:
            self._update(slices, sampling)
        self.buffer.copy_(self.host, non_blocking=True)
        self.graph.replay()
        result = self.result.tolist()
        return result[:real] + result[-2:]

    def _update(self, slices: List[SequenceSlice], sampling: Sequence) -> None:
        """The same requests in the same rows as the step before: only what a decode step changes is
        rewritten (the token, the position, the sampling step, and block-table entries of pages that were
        added); temperatures, seeds and older table entries are already in the pinned buffer."""
        host, off, count = self.host_view, self.layout.offsets, len(slices)
        tokens = np.fromiter((piece.tokens[0] for piece in slices), dtype=np.int64, count=count)
        if tokens.min() < 0 or tokens.max() >= self.vocab_size:
            raise ValueError(f"a token id is outside the vocabulary of {self.vocab_size}")
        starts = np.fromiter((piece.start for piece in slices), dtype=np.int32, count=count)
        host[off["token_ids"]:off["token_ids"] + count] = tokens
        host[off["positions"]:off["positions"] + count] = starts
        host[off["context_len"]:off["context_len"] + count] = starts + 1
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
        # a mixer that keeps state per request runs host code per row: nothing to capture, and padding rows
        # would have to own a state slot
        self.failed = bool(cache.state_entries)
        self.null_pages = None

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
        self.graphs[size] = DecodeGraph(self.model, size, len(self.cache.groups), self.table_width, self.max_context,
                                        self.model.spec.vocab_size, self.null_pages)
        return self.graphs[size]
