"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""
from __future__ import annotations

import numpy as np
import pytest

from pylon_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from pylon_b200.parts.base import CacheNeed, KVNeed, StateNeed


def manager(num_pages=8, page_size=4, max_requests=4, window=None, runs=3):
    needs = [CacheNeed(kv=KVNeed(2, 8, window)) for _ in range(runs)]
    return CacheManager(needs, [None] * runs, page_size=page_size, num_pages=num_pages, max_requests=max_requests)


def test_pool_lifo_reuse_and_double_free():
    pool = PagePool(4)
    first = pool.acquire(3)
    assert first == [0, 1, 2] and pool.free_count == 1
    pool.release([1])
    assert pool.acquire(1) == [1]            # the page given back last is used again first
    with pytest.raises(OutOfPages):
        pool.acquire(2)
    pool.release([0])
    with pytest.raises(CacheError, match="freed twice"):
        pool.release([0])
    with pytest.raises(CacheError, match="does not exist"):
        pool.release([9])


def test_pages_follow_the_token_count_and_come_back():
    cache = manager()
    a = cache.open("a", 20)
    cache.prepare([(a, 4)])
    assert len(a.tables[0]) == 1 and a.pending == 4 and a.length == 0
    cache.commit(a)
    assert a.length == 4
    cache.prepare([(a, 1)])                  # crosses the page edge
    cache.commit(a)
    assert len(a.tables[0]) == 2 and cache.free_pages() == [6]
    cache.check()
    cache.close(a)
    assert cache.free_pages() == [8] and cache.free_slots() == 4
    with pytest.raises(CacheError, match="closed twice"):
        cache.close(a)


def test_a_step_is_all_or_nothing():
    cache = manager(num_pages=3)
    a, b = cache.open("a", 12), cache.open("b", 12)
    with pytest.raises(OutOfPages):
        cache.prepare([(a, 8), (b, 8)])      # 2 + 2 pages wanted, 3 free
    assert cache.free_pages() == [3] and a.tables[0] == [] and b.tables[0] == [] and a.pending == 0
    cache.prepare([(a, 8), (b, 4)])
    cache.commit(a)
    cache.commit(b)
    cache.check()


def test_rules_of_use():
    cache = manager()
    a = cache.open("a", 6)
    with pytest.raises(CacheError, match="open already"):
        cache.open("a", 6)
    with pytest.raises(CacheError, match="capacity"):
        cache.prepare([(a, 7)])
    with pytest.raises(CacheError, match="twice in one step"):
        cache.prepare([(a, 1), (a, 1)])
    cache.prepare([(a, 2)])
    with pytest.raises(CacheError, match="uncommitted"):
        cache.prepare([(a, 1)])
    cache.rollback(a)
    assert a.tables[0] == [] and cache.free_pages() == [8]
    for name in "bcd":
        cache.open(name, 4)
    with pytest.raises(CacheError, match="slot"):
        cache.open("e", 4)


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    needs = [CacheNeed(kv=KVNeed(2, 8)), CacheNeed(kv=KVNeed(2, 8, window=6)), CacheNeed(kv=KVNeed(2, 8)), None]
    cache = CacheManager(needs, [None, None, None, 1], page_size=4, num_pages=10, max_requests=2)
    assert len(cache.groups) == 2 and cache.groups[0].runs == [0, 2] and cache.groups[1].runs == [1]
    a = cache.open("a", 40)
    for _ in range(5):
        cache.prepare([(a, 4)])
        cache.commit(a)
    assert a.length == 20
    assert len(a.held(0)) == 5                       # all keys
    # window 6: the next token (position 20) reads keys 15..20, so pages 0..2 (positions 0..11) are gone
    assert a.tables[1][:3] == [-1, -1, -1] and len(a.held(1)) == 2
    assert cache.free_pages() == [5, 8]
    cache.check()
    table = cache.block_table([a], 1)
    assert table.dtype == np.int32 and table.shape == (1, 5) and list(table[0][:3]) == [-1, -1, -1]
    assert cache.lifetime_pages(40, 4) == [10, 4]     # window + a step's tokens, not page aligned
    cache.close(a)
    assert cache.free_pages() == [10, 10]


def test_each_group_gets_the_pages_it_needs():
    from pylon_b200.cache.manager import group_page_counts

    full, windowed, latent = KVNeed(2, 8), KVNeed(2, 8, window=6), KVNeed(1, 24, value_dim=0)
    needs = [CacheNeed(kv=full), CacheNeed(kv=windowed), CacheNeed(kv=full), None, CacheNeed(kv=latent), CacheNeed(state=StateNeed((4,)))]
    # a pool of 400 tokens in pages of 4; three requests of up to 64 tokens, steps of up to 8 tokens
    counts = group_page_counts(needs, page_size=4, pool_tokens=400, max_requests=3, longest_request=64, max_step_tokens=8)
    # window 6 and a step of 8 tokens span 13 positions: 4 pages and one for the misalignment, per request
    assert counts == {full: 100, windowed: 3 * 5, latent: 100}
    cache = CacheManager(needs, [None, None, None, 1, None, None], page_size=4, num_pages=counts, max_requests=3)
    assert [group.pool.num_pages for group in cache.groups] == [100, 15, 100]
    assert cache.lifetime_pages(64, 8) == [16, 5, 16]
    # three requests at once never need more of the windowed group than it has
    live = [cache.open(name, 64) for name in "abc"]
    for _ in range(8):
        cache.prepare([(request, 8) for request in live])
        for request in live:
            cache.commit(request)
        cache.check()
    assert all(request.length == 64 for request in live)
    # a pool that is small anyway is not made larger for a window
    assert group_page_counts(needs, 4, 40, 3, 64, 8)[windowed] == 10


def test_rows_without_values_and_rows_of_other_widths_count_their_bytes():
    needs = [CacheNeed(kv=KVNeed(2, 8)), CacheNeed(kv=KVNeed(1, 24, value_dim=0)), CacheNeed(kv=KVNeed(2, 8, value_dim=4))]
    cache = CacheManager(needs, [None, None, None], page_size=4, num_pages=3, max_requests=1)
    assert [group.need.value_width for group in cache.groups] == [8, 0, 4]
    assert [group.bytes_per_token(2) for group in cache.groups] == [2 * (8 + 8) * 2, 24 * 2, 2 * (8 + 4) * 2]


def test_state_slots_without_pages():
    needs = [CacheNeed(state=StateNeed((3, 5))), CacheNeed(kv=KVNeed(1, 4))]
    cache = CacheManager(needs, [None, None], page_size=4, num_pages=2, max_requests=2)
    assert len(cache.groups) == 1 and cache.state_bytes_per_request() == 3 * 5 * 4
    a, b = cache.open("a", 4), cache.open("b", 4)
    assert {a.slot, b.slot} == {0, 1}
    cache.close(a)
    c = cache.open("c", 4)
    assert c.slot == a.slot
    cache.check()


def test_qwen3_has_no_state():
    from conftest import TINY_CONFIGS
    from pylon_b200.config import Qwen3Config
    from pylon_b200.models.decoder import DecoderModel
    from pylon_b200.models.qwen3 import qwen3_spec

    model = DecoderModel(qwen3_spec(Qwen3Config(**TINY_CONFIGS["tinyA"]), 64))
    needs = model.cache_needs()
    cache = CacheManager(needs, [None, None], page_size=16, num_pages=4, max_requests=2)
    assert len(cache.groups) == 1 and cache.state_bytes_per_request() == 0 and all(need.state is None for need in needs)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 9])
def test_random_orders_of_requests_keep_the_books(seed, window):
    rng = np.random.default_rng(seed)
    cache = manager(num_pages=12, page_size=4, max_requests=4, window=window)
    live = {}
    opened = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            live[opened] = cache.open(opened, int(rng.integers(1, 40)))
            opened += 1
        elif action < 0.85 and live:
            chosen = [live[k] for k in rng.permutation(list(live))[: int(rng.integers(1, len(live) + 1))]]
            batch = [(r, int(rng.integers(1, min(9, r.capacity - r.length) + 1))) for r in chosen if r.length < r.capacity]
            if not batch:
                continue
            free_before = cache.free_pages()
            try:
                cache.prepare(batch)
            except OutOfPages:
                assert cache.free_pages() == free_before and all(r.pending == 0 for r, _ in batch)
            else:
                if rng.random() < 0.1:
                    for r, _ in batch:
                        cache.rollback(r)
                else:
                    for r, _ in batch:
                        cache.commit(r)
        elif live:
            key = int(rng.choice(list(live)))
            cache.close(live.pop(key))
        cache.check()
        for r in live.values():
            for g, group in enumerate(cache.groups):
                assert len(r.tables[g]) == group.pages_for(r.length)
                if window is None:
                    assert all(page >= 0 for page in r.tables[g])
                else:   # every key a later token reads still has its page
                    for position in range(max(0, r.length - window + 1), r.length):
                        assert r.tables[g][position // 4] >= 0
    for r in list(live.values()):
        cache.close(r)
    cache.check()
    assert cache.free_pages() == [12] and cache.free_slots() == 4
