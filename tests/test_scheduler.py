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


def names(shares):
    return [share.request.request_id for share in shares]


def test_admission_is_fifo_under_the_token_budget_and_plan_is_pure():
    scheduler = Scheduler(max_batch_size=3, max_num_batched_tokens=10, prefill_chunk_size=6)
    a, b, c = make_request("a", 5), make_request("b", 9), make_request("c", 2)
    scheduler.waiting.extend([a, b, c])
    pages = budget()
    plan = scheduler.plan(pages)
    assert names(plan.prompts) == ["a", "b"] and [share.tokens for share in plan.shares] == [5, 5]
    assert plan.newcomers == 2 and plan.tokens == 10 and not plan.decoding
    assert len(scheduler.waiting) == 3 and not scheduler.running      # nothing changed yet
    assert [share.tokens for share in scheduler.plan(pages).shares] == [5, 5]
    admitted = scheduler.commit(plan)
    assert [r.request_id for r in admitted] == ["a", "b"] and c.steps_queued == 1
    assert a.status == RequestStatus.PREFILL and list(scheduler.waiting) == [c]


def test_decode_tokens_are_counted_first_and_running_prefills_go_on():
    scheduler = Scheduler(max_batch_size=4, max_num_batched_tokens=8, prefill_chunk_size=8)
    pages = budget()
    prefilling, decoding = make_request("p", 20), make_request("d", 3)
    for request in (prefilling, decoding):
        pages.cache.admit(request.request_id)
        request.admit()
    decoding.ran(3)
    decoding.take(7)
    prefilling.ran(6)
    scheduler.running.extend([prefilling, decoding])     # the prompt is older, the decode token still comes first
    scheduler.waiting.append(make_request("w", 9))
    plan = scheduler.plan(pages)
    assert names(plan.shares) == ["d", "p"] and plan.shares[0].decode and not plan.shares[1].decode
    assert plan.shares[1].tokens == 7                       # 8 - 1 decode token
    assert plan.newcomers == 0                              # no tokens left
    assert plan.pages == [1 + 4]     # decode: position 3 opens page 0; prefill to 13 tokens: 4 pages


def running_decoder(pages, name="r", length=4):
    request = make_request(name, length)
    pages.cache.admit(name)
    pages.cache.ensure(name, length)
    request.admit()
    request.ran(length)
    request.take(1)
    return request


def test_a_newcomer_needs_room_for_its_whole_prompt_and_nobody_overtakes():
    scheduler = Scheduler(max_batch_size=4, max_num_batched_tokens=64, prefill_chunk_size=8)
    pages = budget(pages=8, page_size=4)
    scheduler.running.append(running_decoder(pages))
    big, small = make_request("big", 30), make_request("small", 2)
    scheduler.waiting.extend([big, small])
    # 7 pages free, the decode takes 1, one stays spare for the running request: 5 pages, the prompt needs 8
    plan = scheduler.plan(pages)
    assert names(plan.shares) == ["r"] and plan.newcomers == 0      # "small" would fit but does not overtake
    # with room for all of it, the prompt is let in and fed in portions
    scheduler.waiting.popleft()
    fits = make_request("fits", 20)
    scheduler.waiting.appendleft(fits)
    plan = scheduler.plan(pages)
    assert names(plan.shares) == ["r", "fits"] and plan.shares[1].tokens == 8 and plan.shares[1].newcomer
    assert plan.pages == [1 + 2]          # only the first portion's pages are taken now
    # "small" is not taken: after "fits" two requests are in flight, and 6 - 5 pages do not leave a spare one each
    assert plan.newcomers == 1


def test_nothing_schedulable_raises():
    scheduler = Scheduler(2, 8)
    scheduler.waiting.append(make_request("a", 5))
    pages = budget(pages=1, page_size=4)
    with pytest.raises(KVCacheExhaustedError):
        scheduler.plan(pages)


def test_put_back_queues_at_the_head():
    scheduler = Scheduler(4, 16)
    pages = budget()
    old, young = running_decoder(pages, "old"), running_decoder(pages, "young")
    scheduler.running.extend([old, young])
    scheduler.waiting.append(make_request("w", 3))
    scheduler.put_back(young)
    assert names([type("S", (), {"request": r}) for r in scheduler.waiting]) == ["young", "w"]
    assert scheduler.running == [old] and young.status == RequestStatus.WAITING and young.replaying


def test_request_state_machine():
    request = make_request("a", 3, max_new=2)
    with pytest.raises(RequestStateError):
        request.ran(1)
    request.admit()
    with pytest.raises(RequestStateError):
        request.admit()
    with pytest.raises(ValueError):
        request.ran(4)
    request.ran(2)
    assert request.status == RequestStatus.PREFILL and request.pending == 1
    with pytest.raises(RequestStateError):
        request.take(9)
    request.ran(1)
    assert request.status == RequestStatus.DECODING
    request.take(9)
    request.ran(1)
    with pytest.raises(ValueError):
        request.ran(2)
    request.take(8)
    request.put_out()
    assert request.status == RequestStatus.WAITING and request.replaying and request.num_computed_tokens == 0
    assert request.feed == [1, 2, 3, 9]          # the last generated token is fed by the next decode
    request.admit()
    request.ran(4)
    assert request.status == RequestStatus.DECODING and not request.replaying
    request.finish(RequestFinishReason.LENGTH)
    with pytest.raises(RequestStateError):
        request.finish(RequestFinishReason.EOS)
    with pytest.raises(ValueError):
        Request("b", [], 1)
    # put out in the middle of its prompt: nothing was sampled, nothing is replayed
    early = make_request("e", 6)
    early.admit()
    early.ran(4)
    early.put_out()
    assert not early.replaying and early.feed == early.prompt_token_ids and early.pending == 6


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
    # 7 pages of 4 tokens: three requests that grow to 5 + 12 tokens each cannot all stay
    engine = engine_with(pages=7, max_new_tokens=12, max_batch_size=3)
    prompts = [[1, 2, 3, 4, 5], [9, 8, 7, 6, 5], [20, 21, 22, 23, 24]]
    requests = [engine.add_request(prompt_token_ids=prompt) for prompt in prompts]
    while engine.step():
        pass
    assert engine.stats["preemptions"] > 0
    assert [request.generated_token_ids for request in requests] == [expected_generation(prompt, 12) for prompt in prompts]
    # the oldest request is never the one that is put out, and finishes first
    assert requests[0].times_put_out == 0 and requests[1].times_put_out + requests[2].times_put_out > 0
    assert requests[0].finished_at <= requests[1].finished_at <= requests[2].finished_at
    engine.cache.check_invariants()
    assert engine.cache.available() == [7]


def test_requests_that_each_need_most_of_the_cache_all_finish():
    """Four requests that need 7 of 8 pages each: only one can be in its last tokens at a time.  A policy that takes
    turns in putting requests out (fewest times put out first) ends none of them; putting out the youngest ends them
    one after the other."""
    engine = engine_with(pages=8, max_new_tokens=16, max_batch_size=4, max_num_batched_tokens=24)
    prompts = [[index + 1] * 11 for index in range(4)]
    requests = [engine.add_request(prompt_token_ids=prompt) for prompt in prompts]
    steps = 0
    while engine.step():
        steps += 1
        assert steps < 400, "the engine turns in circles"
    assert [request.generated_token_ids for request in requests] == [expected_generation(prompt, 16) for prompt in prompts]
    assert engine.stats["tokens"] == 64
    engine.cache.check_invariants()


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
