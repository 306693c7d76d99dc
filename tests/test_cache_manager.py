"""The cache manager's accounting (no GPU): no page lost, held twice or freed twice."""
import random

import pytest

from safetyraise_lmengine_b200.cache.manager import (FIXED_STATE, PAGED_ALL, PAGED_WINDOW, CacheGroupSpec,
                                                     CacheManager)
from safetyraise_lmengine_b200.errors import ResourceExhausted

ALL = CacheGroupSpec("all", PAGED_ALL, (0, 1), kv_heads=2, head_dim=16)
WIN = CacheGroupSpec("win", PAGED_WINDOW, (2,), kv_heads=1, head_dim=16, window=10)
STATE = CacheGroupSpec("st", FIXED_STATE, (3,), state_shape=(4,))


def test_reserve_commit_close():
    m = CacheManager([ALL], page_size=4, num_pages=8, max_requests=3)
    s = m.open_request()
    assert m.reserve(s, 9) and m.table("all", s) == [0, 1, 2] and m.free_pages("all") == 5
    m.commit(s, 9)
    assert m.length(s) == 9
    assert m.reserve(s, 12) and m.table("all", s) == [0, 1, 2]        # still inside the third page
    assert m.reserve(s, 13) and len(m.table("all", s)) == 4
    m.truncate(s, 9)                                                    # the step failed: give the page back
    assert len(m.table("all", s)) == 3 and m.length(s) == 9 and m.free_pages("all") == 5
    m.close_request(s)
    assert m.free_pages("all") == 8 and m.audit() == 0
    with pytest.raises(ValueError):
        m.close_request(s)                                              # closed twice


def test_all_or_nothing_and_lifo_reuse():
    m = CacheManager([ALL], page_size=4, num_pages=4, max_requests=2)
    a, b = m.open_request(), m.open_request()
    assert m.reserve(a, 12)                     # 3 pages
    assert not m.reserve(b, 8)                  # needs 2, only 1 free: nothing taken
    assert m.free_pages("all") == 1 and m.table("all", b) == []
    assert m.fit_tokens(b, 8) == 4
    pages_a = m.table("all", a)
    m.close_request(a)
    assert m.reserve(b, 8)
    assert m.table("all", b)[0] == pages_a[-1]  # the page freed last is used next
    taken, reused = m.reuse_counts()
    assert taken == 5 and reused == 2 and m.audit() == 0
    with pytest.raises(ResourceExhausted):
        m.open_request(), m.open_request()


def test_window_group_gives_pages_back():
    m = CacheManager([ALL, WIN], page_size=4, num_pages=16, max_requests=2)
    s = m.open_request()
    for new_len in (6, 14, 30, 31):
        assert m.reserve(s, new_len)
        m.commit(s, new_len)
    # the group that keeps every key holds one page for every 4 tokens, each a different one, none given back
    held = m.table("all", s)
    assert len(held) == 8 and len(set(held)) == 8 and all(0 <= p < 16 for p in held)
    assert m.free_pages("all") == 16 - 8
    win = m.table("win", s)
    # after 31 tokens the next query (position >= 31) sees keys >= 22: pages 0..4 are passed
    assert win[:5] == [-1] * 5 and all(p >= 0 for p in win[5:])
    assert m.free_pages("win") == 16 - 3 and m.audit() == 0
    with pytest.raises(ValueError):
        m.truncate(s, 10)                        # the window group no longer holds those keys
    m.close_request(s)
    assert m.free_pages("win") == 16 and m.free_pages("all") == 16


def test_state_slots_without_pages():
    m = CacheManager([STATE], page_size=4, num_pages=1, max_requests=2)
    a, b = m.open_request(), m.open_request()
    assert {a, b} == {0, 1}
    assert m.reserve(a, 1000)                    # a fixed-size state needs no pages
    m.commit(a, 1000)
    m.close_request(a)
    assert m.open_request() == a and m.generation(a) == 2 and m.audit() == 0


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    groups = [ALL, WIN] if seed % 2 else [ALL]
    m = CacheManager(groups, page_size=rng.choice([1, 4, 16]), num_pages=rng.choice([5, 23, 64]),
                     max_requests=4)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.15 and len(live) < 4:
            live[m.open_request()] = 0
        elif op < 0.3 and live:
            s = rng.choice(list(live))
            m.close_request(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            want = live[s] + rng.randint(1, 40)
            if m.reserve(s, want):
                if rng.random() < 0.8:
                    m.commit(s, want)
                    live[s] = want
                else:
                    m.truncate(s, live[s])
            else:
                fit = m.fit_tokens(s, want)
                assert live[s] <= fit < want
                if fit > live[s]:
                    assert m.reserve(s, fit)
                    m.commit(s, fit)
                    live[s] = fit
        assert m.audit() == 0
        for s, n in live.items():
            assert m.length(s) == n
            tab = m.table("all", s)
            assert len(tab) >= (n + m.page_size - 1) // m.page_size and len(set(tab)) == len(tab)
    for s in list(live):
        m.close_request(s)
    assert m.audit() == 0 and all(m.free_pages(g.name) == m.num_pages for g in m.paged_groups)
