"""The scheduler's decisions and the engine's handling of a full cache, with a stub model (no GPU)."""
import pytest

from llmserver_b200.cache import CacheManager, KVCacheExhaustedError, KVPagesNeed
from llmserver_b200.engine.engine import Engine
from llmserver_b200.engine.request import Request, RequestFinishReason, RequestStateError, RequestStatus
from llmserver_b200.engine.scheduler import PageBudget, Scheduler
from stubs import ArgmaxSampler, StubModel, expected_generation


def make_request(name, length, max_new=4):
    return Request(name, list(range(1, length + 1)), max_new)


def budget(pages=100, page_size=4):
    return PageBudget(CacheManager([KVPagesNeed(1, 2, None)], page_size, pages, num_slots=16, prefix_sharing=False))


def test_constructor_checks():
    with pytest.raises(ValueError):
        Scheduler(0, 8)
    with pytest.raises(ValueError):
        Scheduler(4, 2)            # fewer tokens than rows
    with pytest.raises(ValueError):
        Scheduler(2, 8, prefill_chunk_size=0)
    assert Scheduler(2, 8).prefill_chunk_size == 8


def test_admission_is_fifo_under_the_token_budget_and_plan_is_pure():
    scheduler = Scheduler(max_batch_size=3, max_num_batched_tokens=10, prefill_chunk_size=6)
    a, b, c = make_request("a", 5), make_request("b", 9), make_request("c", 2)
    scheduler.waiting.extend([a, b, c])
    pages = budget()
    out = scheduler.plan(pages)
    assert [r.request_id for r in out.prefill_requests] == ["a", "b"] and out.prefill_token_counts == [5, 5]
    assert out.num_admitted_requests == 2 and out.num_scheduled_tokens == 10
    assert len(scheduler.waiting) == 3 and not scheduler.running      # nothing changed yet
    assert scheduler.plan(pages).prefill_token_counts == [5, 5]
    admitted = scheduler.commit(out)
    assert [r.request_id for r in admitted] == ["a", "b"] and c.waiting_steps == 1
    assert a.status == RequestStatus.PREFILL and list(scheduler.waiting) == [c]


def test_decode_tokens_are_counted_first_and_running_prefills_go_on():
    scheduler = Scheduler(max_batch_size=4, max_num_batched_tokens=8, prefill_chunk_size=8)
    pages = budget()
    decoding, prefilling = make_request("d", 3), make_request("p", 20)
    for request in (decoding, prefilling):
        pages.cache.admit(request.request_id)
        request.start_prefill()
    decoding.advance_prefill(3)
    decoding.complete_prefill()
    decoding.append_generated_token(7)
    prefilling.advance_prefill(6)
    scheduler.running.extend([decoding, prefilling])
    scheduler.waiting.append(make_request("w", 9))
    out = scheduler.plan(pages)
    assert out.decode_requests == [decoding]
    assert out.prefill_requests[0] is prefilling and out.prefill_token_counts[0] == 7     # 8 - 1 decode token
    assert out.num_admitted_requests == 0                                                  # no tokens left
    assert out.pages_needed == [1 + 4]     # decode: position 3 opens page 0; prefill to 13 tokens: 4 pages


def test_admission_respects_free_pages_with_headroom_and_stops_at_the_first_misfit():
    scheduler = Scheduler(max_batch_size=4, max_num_batched_tokens=64)
    pages = budget(pages=6, page_size=4)
    running = make_request("r", 4)
    pages.cache.admit("r")
    pages.cache.ensure("r", 4)
    running.start_prefill()
    running.advance_prefill(4)
    running.complete_prefill()
    running.append_generated_token(1)
    scheduler.running.append(running)
    big, small = make_request("big", 30), make_request("small", 2)
    scheduler.waiting.extend([big, small])
    out = scheduler.plan(pages)
    # 5 pages free, the decode takes 1, one is kept as headroom for the running request: 3 pages = 12 tokens
    assert out.prefill_requests == [big] and out.prefill_token_counts == [12]
    # nothing fits: a request behind the first misfit is not taken ahead of it
    pages = budget(pages=2, page_size=4)
    pages.cache.admit("r")
    pages.cache.ensure("r", 4)
    out = scheduler.plan(pages)
    assert out.prefill_requests == [] and out.decode_requests == [running]


def test_nothing_schedulable_raises():
    scheduler = Scheduler(2, 8)
    scheduler.waiting.append(make_request("a", 5))
    pages = budget(pages=1, page_size=4)
    pages.cache.admit("x")
    pages.cache.ensure("x", 4)
    with pytest.raises(KVCacheExhaustedError):
        scheduler.plan(pages)


def test_request_state_machine():
    request = make_request("a", 3, max_new=2)
    with pytest.raises(RequestStateError):
        request.advance_prefill(1)
    request.start_prefill()
    with pytest.raises(ValueError):
        request.advance_prefill(4)
    request.advance_prefill(2)
    with pytest.raises(RequestStateError):
        request.complete_prefill()
    request.advance_prefill(1)
    request.complete_prefill()
    request.append_generated_token(9)
    request.complete_decode()
    request.append_generated_token(8)
    request.preempt_for_compute()
    assert request.status == RequestStatus.WAITING and request.needs_decode_resume and request.num_computed_tokens == 0
    assert request.prefill_token_ids == [1, 2, 3, 9]          # the last generated token is fed by the next decode
    request.start_prefill()
    request.advance_prefill(4)
    request.complete_prefill()
    assert not request.needs_decode_resume
    request.finish(RequestFinishReason.LENGTH)
    with pytest.raises(RequestStateError):
        request.finish(RequestFinishReason.EOS)
    with pytest.raises(ValueError):
        Request("b", [], 1)


def engine_with(pages, page_size=4, **kwargs):
    options = dict(max_new_tokens=6, max_batch_size=4, max_num_batched_tokens=16, kv_cache_num_blocks=pages,
                   kv_cache_block_size=page_size, ignore_eos=True, prefix_caching=False, sampler=ArgmaxSampler())
    options.update(kwargs)
    return Engine(StubModel(eos=options.pop("eos", ())), **options)


def test_engine_mixes_prompt_portions_and_decode_tokens_in_one_step():
    engine = engine_with(pages=64, prefill_chunk_size=5)
    prompts = [[3, 4, 5], list(range(10, 23)), [7]]
    outputs = engine.generate(prompts)
    assert outputs == [expected_generation(prompt, 6) for prompt in prompts]
    mixed = [batch for batch in engine.model.batches if not batch.decode_only and 1 in batch.q_lens and batch.max_q_len > 1]
    assert mixed, "no step held a prompt portion beside a decode token"
    assert all(batch.n_tokens <= 16 for batch in engine.model.batches)
    engine.cache.check_invariants()
    assert engine.cache.available() == [64] and not engine.cache.requests


def test_engine_preempts_when_pages_run_out_and_resumes_without_duplicate_tokens():
    # 5 pages of 4 tokens: three requests that grow to 5 + 12 tokens each cannot all stay
    engine = engine_with(pages=7, max_new_tokens=12, max_batch_size=3)
    prompts = [[1, 2, 3, 4, 5], [9, 8, 7, 6, 5], [20, 21, 22, 23, 24]]
    outputs = engine.generate(prompts)
    assert engine.stats["preemptions"] > 0
    assert outputs == [expected_generation(prompt, 12) for prompt in prompts]
    engine.cache.check_invariants()
    assert engine.cache.available() == [7]


def test_a_lone_request_that_does_not_fit_raises():
    engine = engine_with(pages=2, max_new_tokens=20, max_batch_size=2)
    engine.add_request(prompt_token_ids=[1, 2, 3, 4, 5, 6])
    with pytest.raises(KVCacheExhaustedError):
        while engine.step():
            pass


def test_stopping_cancelling_and_validation():
    engine = engine_with(pages=32, eos=(9,), ignore_eos=False, max_new_tokens=10)
    stops = engine.add_request(prompt_token_ids=[5, 6])            # 6 + 1 + 1 = 8, then 8 + 1 + 2 = 11 ...
    runs = engine.add_request(prompt_token_ids=[1], ignore_eos=True, max_new_tokens=3)
    cancelled = engine.add_request(prompt_token_ids=[2, 2, 2])
    engine.step()
    assert engine.cancel_request(cancelled.request_id) and not engine.cancel_request(cancelled.request_id)
    while engine.step():
        pass
    assert runs.finish_reason == RequestFinishReason.LENGTH and len(runs.generated_token_ids) == 3
    assert cancelled.status == RequestStatus.CANCELLED
    assert stops.status == RequestStatus.FINISHED
    if 9 in stops.generated_token_ids:
        assert stops.finish_reason == RequestFinishReason.EOS and stops.generated_token_ids[-1] == 9
    assert engine.cache.available() == [32]
    with pytest.raises(ValueError):
        engine.add_request(prompt_token_ids=[])
    with pytest.raises(ValueError):
        engine.add_request(prompt_token_ids=[1000])
    with pytest.raises(ValueError):
        engine.add_request(prompt="some text")


def test_shared_prefix_is_not_recomputed():
    engine = engine_with(pages=32, prefix_caching=True, max_batch_size=1)
    prompt = list(range(1, 12))
    first = engine.generate([prompt])
    fed_before = sum(batch.n_tokens for batch in engine.model.batches)
    second = engine.generate([prompt])
    fed = sum(batch.n_tokens for batch in engine.model.batches) - fed_before
    assert first == second == [expected_generation(prompt, 6)]
    assert fed == (11 - 8) + 5      # two complete blocks of 4 came from the cache
    engine.cache.check_invariants()
