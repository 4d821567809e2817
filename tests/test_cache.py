"""The cache manager without a GPU: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; groups are independent; shared prefixes; state slots."""
import random

import pytest

from llmserver_b200.cache import (CacheManager, KVCacheExhaustedError, KVCacheStateError, KVPagesNeed, PagePool,
                                  RELEASED, StateNeed)

FULL = KVPagesNeed(2, 16, None)
WINDOWED = KVPagesNeed(2, 16, 10)


def test_pool_allocates_in_fifo_order_and_reuses_freed_pages():
    pool = PagePool(3)
    assert [pool.allocate() for _ in range(3)] == [0, 1, 2]
    with pytest.raises(KVCacheExhaustedError):
        pool.allocate()
    pool.release(1)
    pool.release(0)
    assert pool.allocate() == 1 and pool.allocate() == 0    # given back first, used again first
    pool.check_invariants()


def test_pool_rejects_double_free_and_bad_ids():
    pool = PagePool(2)
    page = pool.allocate()
    pool.release(page)
    with pytest.raises(KVCacheStateError):
        pool.release(page)
    with pytest.raises(KVCacheStateError):
        pool.retain(page)
    with pytest.raises(ValueError):
        pool.release(7)
    pool.check_invariants()


def test_reference_counts_and_idle_pages():
    pool = PagePool(2)
    page = pool.allocate()
    pool.retain(page)
    pool.release(page)
    assert pool.num_free == 1 and page in pool.references
    pool.register_digest(page, "d1")
    pool.release(page)
    assert pool.num_idle == 1 and pool.num_available == 2      # idle pages count as available
    table = []
    assert pool.share("d1", table) == page and table == [page] and pool.num_idle == 0
    with pytest.raises(ValueError):
        pool.share("d1", table)                                # once per table
    pool.release(page)
    other = pool.allocate()                                    # the free page first ...
    assert other != page and pool.lookup("d1") == page
    evicted = pool.allocate()                                  # ... then the idle one is evicted
    assert evicted == page and pool.lookup("d1") is None and pool.evictions == 1
    pool.check_invariants()


def make(needs=(FULL, FULL), pages=8, page_size=4, slots=4, sharing=False):
    return CacheManager(list(needs), page_size, pages, num_slots=slots, prefix_sharing=sharing)


def test_groups_follow_the_needs():
    cache = make([FULL, WINDOWED, FULL, None, WINDOWED, StateNeed((3, 2))])
    assert [group.entries for group in cache.groups] == [[0, 2], [1, 4]]
    assert cache.group_of_entry == {0: (0, 0), 2: (0, 1), 1: (1, 0), 4: (1, 1)}
    assert list(cache.state_entries) == [5]
    cache.materialize("cpu", __import__("torch").float32)
    assert cache.groups[0].storage.shape == (2, 2, 8, 2, 4, 16)
    k_pages, v_pages, group = cache.pages_of_entry(4)
    assert k_pages.shape == (8, 2, 4, 16) and group == 1
    assert cache.state_of_entry(5).shape == (4, 3, 2)


def test_ensure_allocates_all_or_nothing_and_free_gives_everything_back():
    cache = make(pages=5)
    cache.admit("a")
    cache.admit("b")
    assert cache.pages_needed("a", 9) == [3]
    cache.ensure("a", 9)
    assert len(cache.table("a")) == 3 and cache.available() == [2]
    cache.ensure("a", 10)                      # same page
    assert len(cache.table("a")) == 3
    with pytest.raises(KVCacheExhaustedError):
        cache.ensure("b", 12)                  # needs 3, 2 left: nothing is taken
    assert cache.table("b") == [] and cache.available() == [2]
    cache.ensure("b", 8)
    cache.check_invariants()
    cache.free("a")
    assert cache.available() == [3]
    with pytest.raises(KVCacheStateError):
        cache.free("a")
    with pytest.raises(KVCacheStateError):
        cache.ensure("zzz", 1)
    cache.free("b")
    assert cache.available() == [5]
    cache.check_invariants()


def test_a_corrupt_table_frees_nothing():
    cache = make(pages=6)
    cache.admit("a")
    cache.ensure("a", 12)
    cache.table("a").append(cache.table("a")[0])          # the same page twice
    with pytest.raises(KVCacheStateError):
        cache.free("a")
    assert cache.available() == [3]
    cache.table("a").pop()
    cache.table("a")[1] = 5                               # a page that is not allocated
    with pytest.raises(KVCacheStateError):
        cache.free("a")
    assert cache.available() == [3]


def test_a_window_gives_pages_back_as_it_passes_them():
    cache = make([FULL, WINDOWED], pages=16, page_size=4)
    cache.admit("a")
    cache.ensure("a", 30)
    assert [len(cache.table("a", g)) for g in (0, 1)] == [8, 8]
    # 30 tokens done, window 10: the next query (position 30) reads keys 21..30 -> pages 0..4 are passed
    assert cache.advance("a", 30) == 5
    assert cache.table("a", 1)[:6] == [RELEASED] * 5 + [cache.table("a", 1)[5]]
    assert cache.available() == [8, 13]
    assert cache.advance("a", 30) == 0                    # nothing is released twice
    cache.ensure("a", 34)                                 # growing goes on behind released pages
    assert len(cache.table("a", 1)) == 9 and cache.pages_needed("a", 36) == [0, 0]
    cache.check_invariants()
    cache.free("a")
    assert cache.available() == [16, 16]
    cache.check_invariants()


def test_state_slots_are_zeroed_on_admission_and_limited():
    import torch
    cache = make([FULL, StateNeed((5,))], slots=2)
    cache.materialize("cpu", torch.float32)
    first = cache.admit("a")
    cache.state_of_entry(1)[first] = 7.0
    cache.admit("b")
    with pytest.raises(KVCacheExhaustedError):
        cache.admit("c")
    cache.free("a")
    again = cache.admit("c")
    assert again == first and torch.all(cache.state_of_entry(1)[again] == 0)
    with pytest.raises(KVCacheStateError):
        cache.admit("c")
    cache.check_invariants()


def test_shared_prefix_blocks():
    cache = make([FULL], pages=8, page_size=4, sharing=True)
    prompt = list(range(10))
    cache.admit("a")
    assert cache.share_prefix("a", prompt) == 0
    cache.ensure("a", 10)
    cache.register_prefix("a", prompt, 0, 10)              # blocks 0 and 1 are complete, block 2 is not
    assert len(cache.groups[0].pool.digest_of) == 2
    cache.admit("b")
    assert cache.probe_prefix(prompt + [99]) == (8, 0)
    assert cache.share_prefix("b", prompt + [99]) == 8
    assert cache.table("b") == cache.table("a")[:2]
    cache.admit("c")
    assert cache.share_prefix("c", prompt[:8]) == 4        # at least one token is left to compute
    other = [0, 1, 2, 3, 9, 9, 9, 9, 9]
    cache.admit("d")
    assert cache.share_prefix("d", other) == 4             # the chain breaks at the first different block
    cache.check_invariants()
    for name in "abcd":
        cache.free(name)
    assert cache.available() == [8] and cache.groups[0].pool.num_idle == 2
    assert cache.probe_prefix(prompt) == (8, 2)            # the cached blocks are idle now
    cache.check_invariants()
    # sharing is off when a group has a window or a mixer keeps state
    assert not make([FULL, WINDOWED], sharing=True).prefix_sharing
    assert not make([FULL, StateNeed((1,))], sharing=True).prefix_sharing


def test_shared_prefix_across_two_groups_of_full_attention():
    """Two groups that keep every key (other head sizes): each keeps its own digest chain; a prefix is taken over only
    as far as both still hold it."""
    other_shape = KVPagesNeed(1, 8, None)
    cache = make([FULL, other_shape, FULL], pages=6, page_size=4, sharing=True)
    assert cache.prefix_sharing and len(cache.groups) == 2
    prompt = list(range(13))
    cache.admit("a")
    cache.ensure("a", 13)
    cache.register_prefix("a", prompt, 0, 13)              # three complete blocks in both groups
    assert [len(group.pool.digest_of) for group in cache.groups] == [3, 3]
    cache.admit("b")
    assert cache.probe_prefix(prompt) == (12, 0)
    assert cache.share_prefix("b", prompt) == 12
    assert [cache.table("b", group) == cache.table("a", group)[:3] for group in (0, 1)] == [True, True]
    cache.free("a")
    cache.free("b")
    assert cache.probe_prefix(prompt) == (12, 3)
    # the second group loses its cached blocks (another request takes every page there); the first still has them:
    # nothing can be skipped, since the second group's layers would have no keys for the prefix
    pool = cache.groups[1].pool
    held = [pool.allocate() for _ in range(pool.num_available)]
    assert cache.probe_prefix(prompt) == (0, 0)
    cache.admit("c")
    assert cache.share_prefix("c", prompt) == 0 and cache.table("c", 0) == []
    for page in held:
        pool.release(page)
    cache.free("c")
    cache.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_duplicate_a_page(seed):
    rng = random.Random(seed)
    cache = make([FULL, WINDOWED, FULL], pages=24, page_size=4, slots=5)
    live = {}
    for turn in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            name = f"r{turn}"
            cache.admit(name)
            live[name] = 0
        elif action < 0.8 and live:
            name = rng.choice(list(live))
            total = live[name] + rng.choice([1, 1, 2, 5, 13])
            try:
                cache.ensure(name, total)
                live[name] = total
                cache.advance(name, total)
            except KVCacheExhaustedError:
                before = cache.available()
                assert cache.available() == before
        elif live:
            name = rng.choice(list(live))
            cache.free(name)
            del live[name]
        cache.check_invariants()
        for group in cache.groups:
            held = sum(1 for table in group.tables.values() for page in table if page != RELEASED)
            assert held + group.pool.num_available == group.pool.num_pages
    for name in list(live):
        cache.free(name)
    assert cache.available() == [24, 24]
