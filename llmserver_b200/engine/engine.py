"""The engine: request intake, scheduling, the mixed step, sampling, stopping and freeing.

Python entry point in the manner of the reference's ``Engine`` (utils/engine.py:46-475): the same
constructor names where they apply (``max_new_tokens``, ``max_batch_size``, ``max_num_batched_tokens``,
``prefill_chunk_size``, ``kv_cache_num_blocks``, ``kv_cache_block_size``, ``ignore_eos``,
``cuda_graphs``), ``add_request`` / ``step`` / ``cancel_request``, requests that carry
``generated_token_ids``.  It is a token-id engine: prompts come as ids, nothing is tokenised.

What differs by design: one step is ONE forward over decode tokens and prompt portions together
(the reference runs them as separate forwards, utils/engine.py:437-443); sampling is a kernel that
does greedy and seeded temperature sampling (the reference: argmax only, utils/engine.py:295-297).

When pages run out (decided in ``schedule_step``): the plan is checked against the pages available
in every cache group; if it does not fit, the youngest request in flight is put out (its pages
freed, itself at the head of the queue, its cache to be rebuilt later) and planning is repeated; a
lone request that does not fit raises ``KVCacheExhaustedError``.
"""
from __future__ import annotations

import itertools
import time
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from ..cache import CacheManager, KVCacheExhaustedError
from ..sampling import Sampler, SamplingRow
from .request import Request, RequestFinishReason, RequestStatus
from .scheduler import PageBudget, Scheduler, StepPlan
from .step import StepFunction


class Engine:
    def __init__(self, model, max_new_tokens: int = 128, max_batch_size: int = 8, max_num_batched_tokens: int = 8192,
                 prefill_chunk_size: Optional[int] = None, kv_cache_num_blocks: Optional[int] = None,
                 kv_cache_block_size: int = 16, ignore_eos: bool = False, cuda_graphs: Optional[bool] = None,
                 prefix_caching: bool = True, eos_token_ids: Optional[Iterable[int]] = None, dtype="bfloat16",
                 device="cuda:0", max_context: Optional[int] = None, cache: Optional[CacheManager] = None,
                 step_function: Optional[StepFunction] = None, sampler=None):
        """``model``: a model folder (config.json + model.safetensors) or a loaded ``DecoderModel``.

        ``kv_cache_num_blocks`` defaults to the reference benchmark's sizing rule
        (benchmark_cuda.py:107-111): max_batch_size * ceil(max_context / block_size) + 8 pages."""
        if isinstance(model, str):
            from ..models import load_model
            model = load_model(model, dtype, device)
        if max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens is <= 0: {max_new_tokens}")
        self.model = model
        self.device, self.dtype = model.runtime.device, model.runtime.dtype
        self.max_new_tokens = max_new_tokens
        self.ignore_eos = ignore_eos
        self.block_size = kv_cache_block_size
        self.scheduler = Scheduler(max_batch_size, max_num_batched_tokens, prefill_chunk_size)
        if max_context is None:
            max_context = model.spec.max_positions or 4096
        if kv_cache_num_blocks is None:
            kv_cache_num_blocks = max_batch_size * -(-max_context // kv_cache_block_size) + 8
        if cache is None:
            cache = CacheManager(model.cache_needs(), kv_cache_block_size, kv_cache_num_blocks,
                                 num_slots=max_batch_size, prefix_sharing=prefix_caching,
                                 model_identity=model.spec.architecture)
            cache.materialize(self.device, self.dtype)
        # a cache (and step function) that already live on the device may be handed in and shared
        self.cache = cache
        self.block_size = cache.page_size
        self.num_blocks = cache.groups[0].pool.num_pages if cache.groups else 0
        self.step_function = step_function or StepFunction(model, self.cache)
        self.budget = PageBudget(self.cache)
        self.sampler = sampler or Sampler(self.device)
        self.eos_token_ids = set(model.spec.eos_token_ids if eos_token_ids is None else eos_token_ids)
        self.active_requests: Dict[str, Request] = {}
        self.finished_requests: Dict[str, Request] = {}
        self._ids = itertools.count()
        # decode steps replay CUDA graphs unless told otherwise (the reference: utils/engine.py:126-148)
        self.cuda_graphs = (self.device.type == "cuda") if cuda_graphs is None else bool(cuda_graphs)
        if self.cuda_graphs and self.step_function.graphs is None:
            self.step_function.enable_graphs(min(max_context, self.num_blocks * self.block_size), max_batch_size)
        # with ``record_steps`` set, every step leaves (decode rows, prompt tokens, logits rows, cached tokens the step
        # reads, (query, key) pairs its attention covers) in ``step_log``: what a benchmark needs to count bytes and FLOPs
        self.record_steps, self.step_log = False, []
        self.stats = {"steps": 0, "preemptions": 0, "tokens": 0, "prefill_tokens": 0, "decode_tokens": 0, "prefix_tokens": 0,
                      "schedule_s": 0.0, "pack_copy_s": 0.0, "launch_s": 0.0, "read_back_s": 0.0, "accept_s": 0.0, "step_s": 0.0}

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt=None, prompt_token_ids: Optional[Sequence[int]] = None,
                    max_new_tokens: Optional[int] = None, temperature: float = 0.0, seed: Optional[int] = None,
                    ignore_eos: Optional[bool] = None) -> Request:
        """Queues a request.  ``prompt`` exists for signature parity with the reference
        (utils/engine.py:210) and must be None or a sequence of ids: text needs a tokenizer, which
        this engine does not have."""
        if prompt_token_ids is None:
            if prompt is None or isinstance(prompt, str):
                raise ValueError("pass prompt_token_ids: this engine takes token ids, not text")
            prompt_token_ids = prompt
        prompt_token_ids = [int(token) for token in prompt_token_ids]
        if not prompt_token_ids:
            raise ValueError("prompt_token_ids must not be empty")
        vocab = self.model.spec.vocab_size
        for token in prompt_token_ids:
            if not 0 <= token < vocab:
                raise ValueError(f"token id {token} is outside the vocabulary of {vocab}")
        limit = self.model.spec.max_positions
        budget = max_new_tokens or self.max_new_tokens
        if limit is not None and len(prompt_token_ids) + budget > limit + 1:
            raise ValueError(f"prompt of {len(prompt_token_ids)} tokens plus {budget} new tokens exceeds max_position_embeddings {limit}")
        index = next(self._ids)
        request = Request(f"req-{index}", prompt_token_ids, budget, temperature,
                          seed if seed is not None else index, self.ignore_eos if ignore_eos is None else ignore_eos)
        self.active_requests[request.request_id] = request
        self.scheduler.waiting.append(request)
        return request

    def cancel_request(self, request_id: str) -> bool:
        request = self.active_requests.get(request_id)
        if request is None or request.status in (RequestStatus.FINISHED, RequestStatus.CANCELLED):
            return False
        if request in self.scheduler.waiting:
            self.scheduler.waiting.remove(request)
        if request in self.scheduler.running:
            self.scheduler.running.remove(request)
        request.cancel()
        self._release(request)
        self._archive(request)
        return True

    def _release(self, request: Request) -> None:
        if self.cache.is_admitted(request.request_id):
            self.step_function.release(request.request_id)

    def _archive(self, request: Request) -> None:
        self.active_requests.pop(request.request_id, None)
        self.finished_requests[request.request_id] = request
        while len(self.finished_requests) > 1000:   # utils/engine.py:47 max_completed_requests
            self.finished_requests.pop(next(iter(self.finished_requests)))

    # ------------------------------------------------------------------ scheduling
    def _probe_waiting_prefixes(self) -> None:
        """Sets ``num_computed_tokens`` of waiting requests to what a shared prefix would cover, so the
        plan counts only the tokens that need computing (the reference looks prefixes up when the
        request is added, utils/engine.py:197-208,226; here it happens as late as possible)."""
        if not self.cache.prefix_sharing:
            return
        for request in itertools.islice(self.scheduler.waiting, self.scheduler.max_batch_size):
            request.num_computed_tokens, request.prefix_idle_pages = self.cache.probe_prefix(request.feed)

    def put_out(self, request: Request) -> None:
        """Takes a request out of the batch to free its pages; it waits at the head of the queue."""
        self._release(request)
        self.scheduler.put_back(request)
        self.stats["preemptions"] += 1

    def schedule_step(self) -> StepPlan:
        """Plans until the plan fits the cache.  When it does not, the youngest request in flight (the one let in
        last) gives its pages back and waits at the head of the queue; the oldest is never put out while another
        runs, so it always finishes and the engine cannot turn in circles.  The reference instead picks the request
        that was put out least and waited least and queues it at the back (utils/engine.py:412-435); with four
        requests that need most of a small cache each, that rotation puts one request out every step and none of
        them ever ends."""
        while True:
            self._probe_waiting_prefixes()
            plan = self.scheduler.plan(self.budget)
            have = self.cache.available()
            if all(need <= got for need, got in zip(plan.pages, have)):
                for request in self.scheduler.commit(plan):
                    covered = self.step_function.admit(request.request_id, request.feed)
                    request.num_computed_tokens = covered
                    self.stats["prefix_tokens"] += covered
                return plan
            holders = [request for request in self.scheduler.running
                       if any(self.cache.table(request.request_id, group) for group in range(len(self.cache.groups)))]
            if len(self.scheduler.running) < 2 or not holders:
                raise KVCacheExhaustedError(f"the step needs {plan.pages} pages per cache group, {have} are available, "
                                            "and no other request is left to put out")
            self.put_out(holders[-1])

    # ------------------------------------------------------------------ the step
    def step(self) -> bool:
        """Plans and runs one mixed step; returns whether work is left."""
        if not (self.scheduler.waiting or self.scheduler.running):
            return False
        clock = time.perf_counter
        began = clock()
        plan = self.schedule_step()
        entries, sampled = [], []     # sampled: requests that get a token from this step, in row order
        for share in plan.shares:
            request = share.request
            if share.decode:
                entries.append((request.request_id, request.generated_token_ids[-1:], [0]))
                sampled.append(request)
                continue
            first = request.num_computed_tokens
            last_portion = share.tokens == request.pending
            # the end of a rebuilt cache samples nothing: its next token is known (utils/engine.py:380)
            wants = last_portion and not request.replaying
            entries.append((request.request_id, request.feed[first:first + share.tokens], [share.tokens - 1] if wants else []))
            if wants:
                sampled.append(request)
        rows = [SamplingRow(request.temperature, request.seed, len(request.generated_token_ids)) for request in sampled]
        if self.record_steps:
            held = [(share.request.num_computed_tokens, share.tokens) for share in plan.shares]
            self.step_log.append((len(plan.decoding), sum(share.tokens for share in plan.prompts), len(sampled),
                                  sum(start + count for start, count in held),
                                  sum(count * start + count * (count + 1) // 2 for start, count in held)))
        planned = clock()
        tokens = self.step_function.run_and_sample(entries, rows, self.sampler)
        ran = clock()
        for share in plan.shares:
            request = share.request
            before = request.num_computed_tokens
            request.ran(share.tokens)
            if not share.decode:
                self.cache.register_prefix(request.request_id, request.prompt_token_ids, before, request.num_computed_tokens)
        for request, token in zip(sampled, tokens):
            self._accept(request, token)
        self.scheduler.running[:] = [request for request in self.scheduler.running
                                     if request.status not in (RequestStatus.FINISHED, RequestStatus.CANCELLED)]
        stats, phases = self.stats, self.step_function.last_phases
        stats["steps"] += 1
        stats["decode_tokens"] += len(plan.decoding)
        stats["prefill_tokens"] += sum(share.tokens for share in plan.prompts)
        done = clock()
        stats["schedule_s"] += planned - began
        stats["pack_copy_s"] += phases.get("pack_copy", 0.0)
        stats["launch_s"] += phases.get("launch", 0.0)
        stats["read_back_s"] += phases.get("read_back", 0.0)
        stats["accept_s"] += done - ran
        stats["step_s"] += done - began
        return bool(self.scheduler.waiting or self.scheduler.running)

    def step_profile(self) -> Dict[str, float]:
        """Mean host time per step, in milliseconds, by phase (the reference keeps such a record in
        ``Engine.step_profile``, utils/engine.py:69,446-475): ``schedule`` planning and building the step's
        entries; ``pack_copy`` page allocation, packing the batch and queueing its copy; ``launch`` issuing the
        kernels or the graph replay; ``read_back`` waiting for the device and reading the tokens; ``accept``
        bookkeeping after the step; ``step`` all of it."""
        steps = max(1, self.stats["steps"])
        return {name[:-2]: 1e3 * self.stats[name] / steps
                for name in ("schedule_s", "pack_copy_s", "launch_s", "read_back_s", "accept_s", "step_s")}

    def _accept(self, request: Request, token: int) -> None:
        request.take(token)
        self.stats["tokens"] += 1
        if token in self.eos_token_ids and not request.ignore_eos:
            request.finish(RequestFinishReason.EOS)
        elif len(request.generated_token_ids) >= request.max_new_tokens:
            request.finish(RequestFinishReason.LENGTH)
        else:
            return
        self._release(request)
        self._archive(request)

    # ------------------------------------------------------------------ warm-up
    def warmup(self, batch_sizes: Optional[Sequence[int]] = None) -> Dict[str, object]:
        """Before the first request: chooses the variant of every matrix product of a decode step and captures the
        decode graph of every batch-size bucket up to ``max_batch_size`` (or of the given sizes), so that no later
        ``step()`` tunes or captures.  The engine must be idle.  The reference's counterpart is
        ``Engine.warmup_graphs`` (utils/engine.py:150-161)."""
        if self.scheduler.waiting or self.scheduler.running or self.cache.requests:
            raise RuntimeError("warmup() needs an idle engine: requests are queued or in flight")
        return self.step_function.warmup(self.scheduler.max_batch_size, batch_sizes)

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: Optional[int] = None, temperature: float = 0.0,
                 seed: Optional[int] = None, ignore_eos: Optional[bool] = None) -> List[List[int]]:
        """Runs the given prompts (lists of token ids) to completion; returns the generated ids."""
        requests = [self.add_request(prompt_token_ids=prompt, max_new_tokens=max_new_tokens, temperature=temperature,
                                     seed=None if seed is None else seed + index, ignore_eos=ignore_eos)
                    for index, prompt in enumerate(prompts)]
        while self.step():
            pass
        return [request.generated_token_ids for request in requests]
