"""The step function: one batch of (request, its next tokens) through the model and the cache.

It runs only the tokens it is given, as one flat batch, reading what earlier steps left in the
cache, and returns float32 logits at the wanted places.  Pages are allocated before the forward, so
the forward itself allocates nothing (the reference allocates blocks lazily inside the forward,
utils/kv_cache.py:220-277,335-338).  Generation, the scheduler and trace replay all go through this
one function.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..cache import CacheManager, KVCacheExhaustedError
from ..ops.library import check_wait_errors, wait_error_flag
from ..sampling import Sampler, SamplingRow
from .batch import SequenceSlice, StepBatch, build_batch

StepEntry = Tuple[object, Sequence[int], Sequence[int]]  # (request id, next tokens, wanted places)


class StepFunction:
    def __init__(self, model, cache: CacheManager):
        self.model, self.cache = model, cache
        self.device = model.runtime.device
        self.computed = {}          # request -> tokens already in the cache
        model.bind_cache(cache)
        self.pending_flags: List[torch.Tensor] = []
        self.steps_run = 0
        self.last_batch_bytes = 0   # size of the last step's host-to-device copy
        self.graphs = None
        self.graph_steps = 0
        self.sampler = Sampler(self.device)
        self.last_phases = {"pack_copy": 0.0, "launch": 0.0, "read_back": 0.0}

    # ------------------------------------------------------------------ request lifetime
    def admit(self, request_id, prompt: Sequence[int] = None) -> int:
        """Registers a request with the cache; with ``prompt`` given, cached pages of a known prefix
        are taken over.  Returns the number of prompt tokens that need no computing."""
        self.cache.admit(request_id)
        covered = self.cache.share_prefix(request_id, prompt) if prompt is not None else 0
        self.computed[request_id] = covered
        return covered

    def release(self, request_id) -> None:
        self.cache.free(request_id)
        del self.computed[request_id]
        if self.graphs is not None:
            self.graphs.forget_rows()

    def num_computed(self, request_id) -> int:
        return self.computed[request_id]

    # ------------------------------------------------------------------ the step
    def enable_graphs(self, max_context: int, max_batch: int = 256) -> None:
        """Decode-only steps of up to ``max_context`` tokens per request run as CUDA graphs from now on."""
        from .graphs import DecodeGraphs
        self.graphs = DecodeGraphs(self.model, self.cache, max_context, max_batch)

    def slices_for(self, entries: List[StepEntry]) -> List[SequenceSlice]:
        """Allocates the pages the step needs (all or nothing) and describes each request's share."""
        seen = set()
        for request_id, tokens, _ in entries:
            if request_id in seen:
                raise ValueError(f"request {request_id!r} appears twice in one step")
            seen.add(request_id)
            if request_id not in self.computed:
                raise KeyError(f"request {request_id!r} was not admitted")
        # check the whole step against what is available before allocating anything (entries that stay inside
        # their last page, as most decode tokens do, need nothing)
        growing = [entry for entry in entries
                   if not self.cache.has_room(entry[0], self.computed[entry[0]] + len(entry[1]))]
        if growing:
            totals = [0] * len(self.cache.groups)
            for request_id, tokens, _ in growing:
                needed = self.cache.pages_needed(request_id, self.computed[request_id] + len(tokens))
                totals = [a + b for a, b in zip(totals, needed)]
            for group, (total, available) in enumerate(zip(totals, self.cache.available())):
                if total > available:
                    raise KVCacheExhaustedError(f"the step needs {total} pages in cache group {group}, {available} are available")
            for request_id, tokens, _ in growing:
                self.cache.ensure(request_id, self.computed[request_id] + len(tokens))
        limit = self.model.spec.max_positions
        slices = []
        for request_id, tokens, want in entries:
            start = self.computed[request_id]
            if limit is not None and start + len(tokens) > limit:
                raise ValueError(f"request {request_id!r} would reach {start + len(tokens)} tokens; "
                                 f"the model's max_position_embeddings is {limit}")
            slices.append(SequenceSlice(request_id, tokens, start, want,
                                        [self.cache.table(request_id, group) for group in range(len(self.cache.groups))],
                                        self.cache.slot_of(request_id)))
        return slices

    def prepare(self, entries: List[StepEntry], sampling: Optional[Sequence] = None) -> StepBatch:
        batch = build_batch(self.slices_for(entries), len(self.cache.groups), self.device, self.model.spec.vocab_size,
                            sampling=sampling)
        self.last_batch_bytes = batch.host_bytes
        return batch

    def _advance(self, entries: List[StepEntry]) -> None:
        windows = self.cache.has_windows
        for request_id, tokens, _ in entries:
            self.computed[request_id] += len(tokens)
            if windows:
                self.cache.advance(request_id, self.computed[request_id])
        self.steps_run += 1

    def run(self, entries: List[StepEntry]) -> torch.Tensor:
        """Runs one step; returns logits [wanted, vocab] (float32) in the order of the entries and of
        their wanted places."""
        batch = self.prepare(entries)
        logits = self.model.step(batch)
        self.pending_flags.append(batch.error_flag)
        self._advance(entries)
        return logits

    def run_and_sample(self, entries: List[StepEntry], sampling: Sequence, sampler=None) -> List[int]:
        """Runs one step and samples one token per wanted place (``sampling``: one row per wanted place
        with ``temperature``, ``seed``, ``step``).  Returns the tokens on the host: the step's only
        device-to-host read, which also brings the kernels' error flag.  ``last_phases`` then holds the host
        seconds of the step's phases: ``pack_copy``, ``launch``, ``read_back``."""
        if sampler is not None and not hasattr(sampler, "from_batch"):
            logits = self.run(entries)       # a sampler of the caller's own (tests use one on the CPU)
            return sampler(logits, sampling) if sampling else []
        clock = time.perf_counter
        began = clock()
        slices = self.slices_for(entries)
        graph = self.graphs.ready_for(slices) if self.graphs is not None and sampling else None
        if graph is not None:
            result = graph.run(slices, sampling, self.last_phases)
            self.last_phases["pack_copy"] += graph.began - began
            self.last_batch_bytes = graph.layout.total * 4
            self.graph_steps += 1
        else:
            batch = build_batch(slices, len(self.cache.groups), self.device, self.model.spec.vocab_size, sampling=sampling)
            packed = clock()
            self.last_batch_bytes = batch.host_bytes
            logits = self.model.step(batch)
            if not sampling:
                self.pending_flags.append(batch.error_flag)
                self._advance(entries)
                self.last_phases.update(pack_copy=packed - began, launch=clock() - packed, read_back=0.0)
                return []
            tokens = (sampler or self.sampler).from_batch(logits, batch)
            flags = torch.cat([tokens, batch.error_flag, wait_error_flag(self.device)])
            launched = clock()
            result = flags.tolist()
            self.last_phases.update(pack_copy=packed - began, launch=launched - packed, read_back=clock() - launched)
        self._advance(entries)
        if result[-2] != 0:
            raise RuntimeError("a kernel met a block-table entry outside the page pool; the cache bookkeeping is corrupt")
        if result[-1] != 0:
            check_wait_errors()      # raises with the code and clears the flag
        return result[:-2]

    # ------------------------------------------------------------------ warm-up
    def warmup(self, max_batch: int, batch_sizes: Optional[Sequence[int]] = None) -> dict:
        """Runs throw-away steps on an idle cache so that later steps neither tune a matrix product nor capture a
        graph: one prompt portion per row bucket of the small-row product kernel, then decode steps of every
        batch-size bucket up to ``max_batch`` (or of ``batch_sizes``) until that bucket's graph exists.  The dummy
        requests hold a page each while their step runs and give it back."""
        from ..ops import gemm_bf16
        from .graphs import BUCKETS
        if self.computed:
            raise RuntimeError("warmup needs an idle step function: requests are admitted")
        began = time.perf_counter()
        tuned_before = gemm_bf16.tunings()
        vocab = self.model.spec.vocab_size
        greedy = [SamplingRow()]
        limit = self.model.spec.max_positions
        page_room = min(self.cache.capacity()) * self.cache.page_size if self.cache.groups else 1 << 30
        portions = []
        if self.model.runtime.dtype == torch.bfloat16:
            portions = [rows for rows in gemm_bf16.ROW_BUCKETS if rows > 1 and rows <= page_room and (limit is None or rows <= limit)]
        for rows in portions:
            self.admit("warm-up")
            try:
                self.run_and_sample([("warm-up", [index % vocab for index in range(rows)], [rows - 1])], greedy)
            finally:
                self.release("warm-up")
        if batch_sizes is None:
            batch_sizes = [size for size in BUCKETS if size <= max_batch]
            if max_batch not in batch_sizes and self.graphs is not None and self.graphs.bucket_for(max_batch) == max_batch:
                batch_sizes.append(max_batch)
        captured = []
        for size in batch_sizes:
            if (self.cache.groups and size > min(self.cache.capacity())) or size > self.cache.slots.num_slots:
                continue
            names = [f"warm-up-{row}" for row in range(size)]
            for name in names:
                self.admit(name)
            try:
                rounds = 1 if self.graphs is None or self.graphs.failed else self.graphs.WARM_STEPS + 1
                for round_index in range(rounds):
                    if limit is not None and round_index + 1 > limit:
                        break
                    self.run_and_sample([(name, [0], [0]) for name in names], greedy * size)
            finally:
                for name in names:
                    self.release(name)
            if self.graphs is not None and size in self.graphs.graphs:
                captured.append(size)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        return {"graphs": captured, "products_tuned": gemm_bf16.tunings() - tuned_before,
                "seconds": time.perf_counter() - began}

    def check_errors(self) -> None:
        """Reads the kernels' error flags of the steps run since the last check (synchronises)."""
        check_wait_errors()
        flags, self.pending_flags = self.pending_flags, []
        if flags and int(torch.stack([flag.reshape(()) for flag in flags]).max().item()) != 0:
            raise RuntimeError("a kernel met a block-table entry outside the page pool; the cache bookkeeping is corrupt")
