"""Continuous batching: who runs how many tokens in the next step.

A step has a budget of tokens, a number of rows (requests in flight) and the cache's pages.  The order of claims is
the reference's (utils/scheduler.py:24-65): every decoding request first, one token each; then requests that are in
the middle of their prompt, a portion each; then newcomers from the queue, first come first served, and the first
newcomer that cannot be given anything ends the admission, so nobody overtakes.  ``plan`` only reads; ``commit``
moves the newcomers into the batch.

What is this engine's own:

* a plan is ONE step: decode tokens and prompt portions run in the same forward (the reference runs two,
  utils/engine.py:437-443);
* pages are counted per cache group, and a plan must fit every group;
* a newcomer is taken only if the pages of *everything it still has to feed* are available beyond one spare page
  per request in flight, although it may then be fed in portions.  A request that is let in on a part of its prompt
  and cannot go on holds pages that older requests need, is put out, comes back and is put out again; asking for
  the whole prompt's pages at the door avoids most of that.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List

from ..cache import KVCacheExhaustedError
from .request import Request, RequestStatus


@dataclass
class Share:
    """One request's part of a step."""
    request: Request
    tokens: int              # how many of its tokens the step runs
    decode: bool = False     # the one token is the request's last sampled token; else a portion of what it has to feed
    newcomer: bool = False   # comes from the queue with this plan


@dataclass
class StepPlan:
    shares: List[Share] = field(default_factory=list)
    pages: List[int] = field(default_factory=list)     # per cache group: pages the step has to allocate
    tokens: int = 0

    @property
    def decoding(self) -> List[Share]:
        return [share for share in self.shares if share.decode]

    @property
    def prompts(self) -> List[Share]:
        return [share for share in self.shares if not share.decode]

    @property
    def newcomers(self) -> int:
        return sum(1 for share in self.shares if share.newcomer)


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
        if max_batch_size < 1:
            raise ValueError(f"a batch needs at least one row (max_batch_size={max_batch_size})")
        if max_num_batched_tokens < max_batch_size:
            raise ValueError(f"a step of {max_num_batched_tokens} tokens cannot give each of {max_batch_size} rows its "
                             "decode token; raise max_num_batched_tokens or lower max_batch_size")
        portion = max_num_batched_tokens if prefill_chunk_size is None else prefill_chunk_size
        if portion < 1:
            raise ValueError(f"prompt portions need at least one token (prefill_chunk_size={prefill_chunk_size})")
        self.max_batch_size, self.max_num_batched_tokens, self.prefill_chunk_size = max_batch_size, max_num_batched_tokens, portion
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []      # in the order they were let in: the last is the youngest

    def plan(self, budget: PageBudget) -> StepPlan:
        plan = StepPlan()
        left = budget.available()
        plan.pages = [0] * len(left)
        tokens_left = self.max_num_batched_tokens

        def claim(share: Share, pages: List[int]) -> None:
            nonlocal tokens_left
            plan.shares.append(share)
            tokens_left -= share.tokens
            for group, count in enumerate(pages):
                left[group] -= count
                plan.pages[group] += count

        # 1. requests in flight: decode tokens are set apart first, then the prompts go on
        in_prompt = []
        for request in self.running:
            if request.status is RequestStatus.DECODING:
                claim(Share(request, 1, decode=True), budget.needed(request, request.num_computed_tokens + 1))
            elif request.status is RequestStatus.PREFILL:
                in_prompt.append(request)
        page = budget.page_size
        promised = 0       # pages that prompts in flight will still ask for after this step
        for request in in_prompt:
            portion = min(request.pending, self.prefill_chunk_size, tokens_left)
            if portion > 0:
                claim(Share(request, portion), budget.needed(request, request.num_computed_tokens + portion))
            promised += -(-len(request.feed) // page) - -(-(request.num_computed_tokens + portion) // page)

        # 2. the queue, in order, while rows, tokens and pages last
        rows_left = self.max_batch_size - len(self.running)
        spare_kept = len(self.running)        # a page per request in flight stays free for its next tokens
        for request in self.waiting:
            if rows_left == 0 or tokens_left == 0:
                break
            if request.pending < 1:
                raise ValueError(f"request {request.request_id!r} waits with nothing left to feed")
            # pages of a shared prefix cost nothing, except those that are idle now and stop being available
            covered = request.num_computed_tokens // page
            whole = -(-len(request.feed) // page) - covered + request.prefix_idle_pages
            if left and whole > min(left) - promised - spare_kept:
                break
            portion = min(request.pending, self.prefill_chunk_size, tokens_left)
            now = -(-(request.num_computed_tokens + portion) // page) - covered + request.prefix_idle_pages
            claim(Share(request, portion, newcomer=True), [now] * len(left))
            promised += whole - now
            rows_left -= 1
            spare_kept += 1
        plan.tokens = self.max_num_batched_tokens - tokens_left
        if not plan.shares and self.waiting:
            raise KVCacheExhaustedError(f"the cache cannot hold request {self.waiting[0].request_id!r} "
                                        f"({len(self.waiting[0].feed)} tokens to feed) even with nothing else in flight")
        return plan

    def commit(self, plan: StepPlan) -> List[Request]:
        """Lets the plan's newcomers in (they leave the queue in order); returns them."""
        let_in = []
        for share in plan.shares:
            if share.newcomer:
                request = self.waiting.popleft()
                if request is not share.request:
                    raise RuntimeError("the queue changed between plan and commit")
                request.admit()
                self.running.append(request)
                let_in.append(request)
        for request in self.waiting:
            request.steps_queued += 1
        return let_in

    def put_back(self, request: Request) -> None:
        """A request that was put out returns to the head of the queue: it is older than anything that waits."""
        self.running.remove(request)
        request.put_out()
        self.waiting.appendleft(request)
