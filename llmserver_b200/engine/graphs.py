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

import torch

from .. import ops
from ..ops.library import wait_error_flag
from .batch import BatchLayout, SequenceSlice, pack, views


class DecodeGraph:
    def __init__(self, model, batch_size: int, n_groups: int, table_width: int, max_context: int, vocab_size: int):
        self.model, self.vocab_size = model, vocab_size
        self.layout = BatchLayout(batch_size, batch_size, batch_size, (table_width,) * n_groups)
        device = model.runtime.device
        self.host = torch.zeros(self.layout.total, dtype=torch.int32, pin_memory=True)
        self.host_view = self.host.numpy()
        self.buffer = torch.zeros(self.layout.total, dtype=torch.int32, device=device)
        # the static batch claims the longest context, so that launch shapes cover every later step
        shape_only = [SequenceSlice(index, [0], max_context - 1, [0], [[0] * table_width] * n_groups, 0)
                      for index in range(batch_size)]
        self.batch = views(self.buffer, self.layout, shape_only)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            logits = self.model.step(self.batch)
            tokens = ops.sample(logits, self.batch.temperatures, self.batch.seeds, self.batch.sample_steps)
            self.result = torch.cat([tokens, self.batch.error_flag, wait_error_flag(device)])

    def run(self, slices: List[SequenceSlice], sampling: Sequence) -> List[int]:
        pack(slices, self.layout, self.host_view, self.vocab_size, sampling)
        self.buffer.copy_(self.host, non_blocking=True)
        self.graph.replay()
        return self.result.tolist()


class DecodeGraphs:
    """One graph per batch size, captured the third time that batch size is seen."""

    WARM_STEPS = 2

    def __init__(self, model, n_groups: int, page_size: int, max_context: int, max_batch: int = 256):
        self.model, self.n_groups = model, n_groups
        self.max_context, self.max_batch = max_context, max_batch
        self.table_width = -(-max_context // page_size)
        self.graphs: Dict[int, DecodeGraph] = {}
        self.seen: Dict[int, int] = {}
        self.failed = False

    def ready_for(self, slices: List[SequenceSlice]):
        """The graph that can run this step, or None (then the step runs eagerly)."""
        if self.failed or len(slices) > self.max_batch:
            return None
        for piece in slices:
            if len(piece.tokens) != 1 or len(piece.want) != 1 or piece.start + 1 > self.max_context:
                return None
        size = len(slices)
        graph = self.graphs.get(size)
        if graph is not None:
            return graph
        self.seen[size] = self.seen.get(size, 0) + 1
        if self.seen[size] <= self.WARM_STEPS:
            return None
        self.graphs[size] = DecodeGraph(self.model, size, self.n_groups, self.table_width, self.max_context,
                                        self.model.spec.vocab_size)
        return self.graphs[size]
