"""Continuous batching under a token budget.

Policy of the reference's scheduler (utils/scheduler.py:24-65): every decoding request gets one
token, counted first against the budget; running prefills get min(remaining prompt, chunk size,
tokens left); then waiting requests are admitted first-in first-out while request slots, tokens and
cache pages last, keeping one page of headroom per running request, and admission stops at the first
request that gets nothing.  ``plan`` changes nothing; ``commit`` applies it.

Unlike the reference, whose engine runs decode rows and prompt chunks as separate forwards
(utils/engine.py:437-443), one plan becomes ONE mixed step.  Pages are counted per cache group, so a
plan fits only if it fits every group.
"""
from __future__ import annotations

from collections import deque
from typing import List

from ..cache import KVCacheExhaustedError
from .request import Request, RequestStatus


class SchedulerOutput:
    def __init__(self):
        self.num_admitted_requests = 0
        self.prefill_requests: List[Request] = []
        self.prefill_token_counts: List[int] = []
        self.decode_requests: List[Request] = []
        self.num_scheduled_tokens = 0
        self.pages_needed: List[int] = []     # per cache group

    @property
    def empty(self) -> bool:
        return not self.prefill_requests and not self.decode_requests


class PageBudget:
    """What the scheduler asks of the cache: pages available per group, pages a request would need
    to hold ``total`` tokens, and the page size.  ``CacheManager`` fits as it is; tests use a stub."""

    def __init__(self, cache):
        self.cache = cache
        self.page_size = cache.page_size

    def available(self) -> List[int]:
        return list(self.cache.available())

    def needed(self, request: Request, total_tokens: int) -> List[int]:
        return list(self.cache.pages_needed(request.request_id, total_tokens))


class Scheduler:
    def __init__(self, max_batch_size: int, max_num_batched_tokens: int, prefill_chunk_size: int = None):
        if max_batch_size <= 0:
            raise ValueError(f"max_batch_size must be positive: {max_batch_size}")
        if max_num_batched_tokens <= 0:
            raise ValueError(f"max_num_batched_tokens must be positive: {max_num_batched_tokens}")
        if max_num_batched_tokens < max_batch_size:
            raise ValueError(f"max_num_batched_tokens must be >= max_batch_size: max_num_batched_tokens: {max_num_batched_tokens}, max_batch_size: {max_batch_size}")
        if prefill_chunk_size is None:
            prefill_chunk_size = max_num_batched_tokens
        if prefill_chunk_size <= 0:
            raise ValueError(f"prefill_chunk_size must be positive: {prefill_chunk_size}")
        self.max_batch_size = max_batch_size
        self.max_num_batched_tokens = max_num_batched_tokens
        self.prefill_chunk_size = prefill_chunk_size
        self.waiting: deque = deque()
        self.running: List[Request] = []

    def plan(self, budget: PageBudget) -> SchedulerOutput:
        out = SchedulerOutput()
        page_size = budget.page_size
        free = budget.available()
        n_groups = len(free)
        needed_total = [0] * n_groups
        available_slots = self.max_batch_size - len(self.running)
        out.decode_requests = [request for request in self.running if request.status == RequestStatus.DECODING]
        remaining_tokens = self.max_num_batched_tokens - len(out.decode_requests)
        for request in self.running:
            needed = [0] * n_groups
            if request.status == RequestStatus.PREFILL:
                chunk = min(request.remaining_prefill, self.prefill_chunk_size, remaining_tokens)
                if chunk > 0:
                    needed = budget.needed(request, request.num_computed_tokens + chunk)
                    out.prefill_requests.append(request)
                    out.prefill_token_counts.append(chunk)
                    remaining_tokens -= chunk
            elif request.status == RequestStatus.DECODING:
                needed = budget.needed(request, request.num_computed_tokens + 1)
            free = [a - b for a, b in zip(free, needed)]
            needed_total = [a + b for a, b in zip(needed_total, needed)]
        reserved = len(self.running)   # one page of headroom per running request (utils/scheduler.py:43,50)
        index = 0
        while index < len(self.waiting) and available_slots > 0 and remaining_tokens > 0:
            request = self.waiting[index]
            if request.remaining_prefill <= 0:
                raise ValueError(f"No prompt tokens remain to prefill: request_id: {request.request_id}, num_computed_tokens: {request.num_computed_tokens}")
            spare = min(free) - reserved if free else 1 << 30
            # pages a shared prefix already covers cost nothing; count only what lies beyond it
            covered_pages = request.num_computed_tokens // page_size
            fitting = max(0, spare - request.prefix_idle_pages) * page_size - (request.num_computed_tokens - covered_pages * page_size)
            chunk = min(request.remaining_prefill, self.prefill_chunk_size, remaining_tokens, max(0, fitting))
            if chunk == 0:
                break
            # cached pages that are idle now stop being available once the request takes them
            pages = -(-(request.num_computed_tokens + chunk) // page_size) - covered_pages + request.prefix_idle_pages
            out.prefill_requests.append(request)
            out.prefill_token_counts.append(chunk)
            free = [a - pages for a in free]
            needed_total = [a + pages for a in needed_total]
            available_slots -= 1
            remaining_tokens -= chunk
            index += 1
        out.num_admitted_requests = index
        out.num_scheduled_tokens = self.max_num_batched_tokens - remaining_tokens
        out.pages_needed = needed_total
        if self.waiting and out.empty:
            raise KVCacheExhaustedError("No request can fit into the KV cache")
        return out

    def commit(self, out: SchedulerOutput) -> List[Request]:
        """Moves the admitted requests from waiting to running; returns them."""
        admitted = []
        for _ in range(out.num_admitted_requests):
            request = self.waiting.popleft()
            request.start_prefill()
            self.running.append(request)
            admitted.append(request)
        for request in self.waiting:
            request.waiting_steps += 1
        return admitted
