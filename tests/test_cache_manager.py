"""Cache manager: pages are never lost, held twice or freed twice, under random orders of
requests; windows give pages back; published prefixes are found again and evicted only
under pressure; state slots."""
import random

import pytest

from vosti_b200.cache import (RELEASED, CacheManager, OutOfPages, OutOfSlots, PageAccountingError, PagePool,
                              chain_hash)
from vosti_b200.parts import PagedCacheSpec, StateSpec

FULL = PagedCacheSpec(2, 2, 16)
WINDOWED = PagedCacheSpec(2, 2, 16, window=10)


def test_pool_order_and_double_free():
    pool = PagePool(4)
    assert pool.allocate(2) == [0, 1]
    pool.release(0)
    assert pool.allocate(1) == [0]                 # a freed page is the next one used
    with pytest.raises(OutOfPages):
        pool.allocate(3)
    pool.release(1)
    with pytest.raises(PageAccountingError):
        pool.release(1)
    with pytest.raises(PageAccountingError):
        pool.acquire(1)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_accounts(seed):
    rng = random.Random(seed)
    prefix_reuse = seed % 2 == 0
    specs = [FULL, FULL] if prefix_reuse else [FULL, WINDOWED, FULL]
    cache = CacheManager(specs, [None] * len(specs), num_pages=24, page_size=4, max_requests=5,
                         prefix_reuse=prefix_reuse)
    assert cache.prefix_reuse == prefix_reuse
    live, tokens_of, next_id = [], {}, 0
    shared = [rng.randrange(50) for _ in range(12)]
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            prompt = (shared if rng.random() < 0.5 else []) + [rng.randrange(50) for _ in range(rng.randrange(1, 9))]
            cache.begin(next_id, prompt)
            tokens_of[next_id] = prompt
            live.append(next_id)
            next_id += 1
        elif action < 0.8 and live:
            rid = rng.choice(live)
            known, have = tokens_of[rid], cache.length(rid)
            if have >= len(known):
                known.append(rng.randrange(50))
            count = rng.randrange(1, len(known) - have + 1)
            if cache.can_extend(rid, count):
                before = cache.length(rid)
                slots = cache.extend(rid, count)
                assert len(slots) == len(cache.groups) and all(len(s) == count for s in slots)
                for g, group_slots in enumerate(slots):
                    row = cache.block_row(rid, g)
                    for i, slot in enumerate(group_slots):
                        pos = before + i
                        assert slot == row[pos // 4] * 4 + pos % 4 and row[pos // 4] != RELEASED
                cache.publish(rid, known[:cache.length(rid)])
                cache.trim(rid)
            else:
                with pytest.raises(OutOfPages):
                    cache.extend(rid, count)
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            cache.finish(rid)
        cache.check()
        # slots of different live requests never collide unless the page is shared on purpose
        if not prefix_reuse:
            for g in range(len(cache.groups)):
                held = [p for r in live for p in cache.block_row(r, g) if p != RELEASED]
                assert len(held) == len(set(held))
    for rid in live:
        cache.finish(rid)
    cache.check()
    assert all(g.pool.available() == 24 for g in cache.groups)


def test_window_gives_pages_back_and_keeps_what_is_read():
    cache = CacheManager([FULL, WINDOWED], [None, None], num_pages=16, page_size=4, max_requests=2)
    assert [g.window for g in cache.groups] == [0, 10] and not cache.prefix_reuse
    cache.begin("r")
    cache.extend("r", 30)
    cache.trim("r")
    full, win = cache.block_row("r", 0), cache.block_row("r", 1)
    assert RELEASED not in full and len(full) == 8
    # next query sits at position 30 and reads keys 21..30: pages 0..4 (positions < 20) are gone
    assert [p == RELEASED for p in win] == [True] * 5 + [False] * 3
    assert cache.groups[1].pool.available() == 16 - 3 and cache.groups[0].pool.available() == 8
    cache.extend("r", 1)
    cache.trim("r")
    assert cache.block_row("r", 1)[5] != RELEASED      # position 22 is still inside the window of 31
    cache.finish("r")
    cache.check()
    assert cache.groups[1].pool.available() == 16


def test_prefix_pages_are_found_and_evicted_only_under_pressure():
    cache = CacheManager([FULL], [None], num_pages=6, page_size=4, max_requests=3)
    prompt = list(range(100, 111))                     # 11 tokens: two full pages and a tail
    cache.begin("a", prompt)
    cache.extend("a", 11)
    assert cache.publish("a", prompt) == 2
    pages_a = list(cache.block_row("a", 0))
    cache.begin("b", prompt[:8] + [7, 7, 7])           # same two pages, other tail
    assert cache.block_row("b", 0) == pages_a[:2] and cache.length("b") == 8
    assert cache.live["b"].cached_prefix_pages == 2
    cache.begin("c", prompt[:8])                       # never the page with the last token
    assert cache.length("c") == 4
    cache.check()
    for rid in "abc":
        cache.finish(rid)
    cache.check()
    pool = cache.groups[0].pool
    assert len(pool.evictable) == 2 and pool.available() == 6
    cache.begin("d", [1, 2, 3])
    cache.extend("d", 4 * 4)                           # fits into the vacant pages: nothing evicted
    assert pool.evictions == 0 and len(pool.evictable) == 2
    cache.extend("d", 4)                               # now a published page has to go: the leaf first
    assert pool.evictions == 1 and pages_a[1] in cache.block_row("d", 0)
    cache.begin("e", prompt)
    assert cache.length("e") == 4                      # the chain is found up to the evicted page
    cache.finish("d"), cache.finish("e")
    cache.check()


def test_match_checks_tokens_not_only_hashes():
    pool = PagePool(4)
    page = pool.allocate(1)[0]
    h, _ = pool.publish(page, [1, 2, 3, 4], 0, 1, -1)
    assert h == chain_hash(0, [1, 2, 3, 4])
    pool._set_published_tokens(page, [9, 9, 9, 9])     # as if another prompt hashed the same
    assert pool.match([1, 2, 3, 4, 5], 4) == []


def test_state_slots():
    cache = CacheManager([None, FULL], [StateSpec((3,)), None], num_pages=4, page_size=4, max_requests=2)
    assert not cache.prefix_reuse                      # a state cannot be rebuilt from pages
    a, b = cache.begin("a"), cache.begin("b")
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(OutOfSlots):
        cache.begin("c")
    cache.finish("a")
    assert cache.begin("c").slot == a.slot
    with pytest.raises(ValueError):
        cache.begin("c")
    cache.check()
