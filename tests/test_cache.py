"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from ultima_b200.cache import Cache, CacheError, PageAllocator, SlotBook, PAGE
from ultima_b200.parts import KVNeed, StateNeed


def test_page_allocator_hands_each_page_to_one_owner():
    a = PageAllocator(8)
    x, y = a.take(3), a.take(5)
    assert sorted(x + y) == list(range(8)) and a.n_free == 0
    with pytest.raises(CacheError, match="full"):
        a.take(1)
    a.give_back(x)
    with pytest.raises(CacheError, match="not held"):
        a.give_back(x[:1])
    assert a.n_free == 3 and sorted(a.take(3)) == sorted(x)


def test_slot_book_double_release_and_unknown_slot():
    b = SlotBook(2)
    s0, s1 = b.acquire(), b.acquire()
    assert {s0, s1} == {0, 1}
    with pytest.raises(CacheError, match="no free slot"):
        b.acquire()
    b.release(s0)
    with pytest.raises(CacheError, match="not held"):
        b.release(s0)
    with pytest.raises(CacheError, match="does not exist"):
        b.release(5)
    assert b.acquire() == s0


def _cache(**kw):
    needs = [KVNeed(2, 16), KVNeed(2, 16, window=20), KVNeed(2, 16), (KVNeed(2, 16, window=20), StateNeed((3, 4)))]
    args = dict(max_tokens=8 * PAGE, max_context=512, n_slots=4, step_chunk=64)
    args.update(kw)
    return Cache(needs, [None] * 4, dtype=torch.float32, device="cpu", **args)


def test_groups_have_storage_of_their_own():
    c = _cache()
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    full = [g for g in c.kv_groups if g.need.window is None][0]
    win = [g for g in c.kv_groups if g.need.window is not None][0]
    assert full.runs == [0, 2] and win.runs == [1, 3]
    assert full.k.shape == (2, 8, 2, PAGE, 16) and full.k.data_ptr() != win.k.data_ptr()
    # a window of 20 with steps of up to 64 new tokens spans 83 positions: two pages
    assert win.ring_pages == 2 and win.k.shape[1] == min(8, 4 * 2)
    assert c.state_groups[0].data.shape == (1, 4, 3, 4)


def test_pages_follow_length_and_come_back():
    c = _cache()
    s = c.acquire()
    c.reserve(s, 1)
    c.commit(s, 1)
    assert c.pages_held() == 2
    c.reserve(s, 65)
    c.commit(s, 64)
    assert c.length(s) == 65 and c.pages_held() == 4
    c.reserve(s, 300)                       # the window group stays at its two pages
    assert [len(g.pages_of[s]) for g in c.kv_groups] == [5, 2]
    t = c.tables([s])
    assert t[0].shape == (1, 8) and t[1].shape == (1, 2) and t[0].dtype.name == "int32"
    c.release(s)
    assert c.pages_held() == 0 and all(g.pool.n_free == g.n_pages for g in c.kv_groups)
    with pytest.raises(CacheError, match="not held"):
        c.release(s)
    with pytest.raises(CacheError, match="not held"):
        c.reserve(s, 3)


def test_full_cache_is_an_error_before_anything_changes():
    c = _cache(max_tokens=4 * PAGE)
    a, b = c.acquire(), c.acquire()
    c.reserve(a, 3 * PAGE)
    with pytest.raises(CacheError, match="cache is full"):
        c.can_hold({b: 2 * PAGE})
    c.can_hold({b: PAGE})
    with pytest.raises(CacheError, match="limit"):
        c.reserve(b, 513)


def test_state_is_zero_for_a_new_sequence():
    c = _cache()
    s = c.acquire()
    c.state_groups[0].data[:, s] = 7.0
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(c.state_groups[0].data[:, s2].abs().sum()) == 0.0


def test_reader_runs_share_the_owner_s_storage():
    needs = [KVNeed(1, 16), KVNeed(1, 16), KVNeed(1, 16)]
    c = Cache(needs, [None, 0, None], max_tokens=4 * PAGE, max_context=128, n_slots=2, step_chunk=64,
              dtype=torch.float32, device="cpu")
    assert c.kv_groups[0].runs == [0, 2]
    tabs = [torch.zeros(1, 2, dtype=torch.int32)]
    own, rd = c.run_cache(0, tabs), c.run_cache(1, tabs)
    assert rd.kv.k.data_ptr() == own.kv.k.data_ptr() and own.kv.owner and not rd.kv.owner
    with pytest.raises(CacheError, match="earlier run"):
        Cache(needs, [None, 2, None], 256, 128, 2, 64, device="cpu")


def test_random_churn_never_loses_or_doubles_a_page():
    rng = random.Random(0)
    c = _cache(max_tokens=16 * PAGE, n_slots=6)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and c.slots.n_free:
            live[c.acquire()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = live[s] + rng.randint(1, 90)
            try:
                c.can_hold({s: n})
            except CacheError:
                continue
            if n > c.max_context:
                continue
            c.reserve(s, n)
            c.commit(s, n - live[s])
            live[s] = n
        elif live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        for g in c.kv_groups:
            held = [p for s in range(c.n_slots) for p in g.pages_of[s]]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + g.pool.n_free == g.n_pages, "a page is lost"
            for s, n in live.items():
                assert len(g.pages_of[s]) == g.pages_needed(n)
        assert sorted(live) == [s for s in range(c.n_slots) if c.slots.in_use[s]]


def test_truncate_gives_pages_back_and_refuses_what_cannot_go_back():
    c = Cache([KVNeed(2, 16)], [None], max_tokens=8 * PAGE, max_context=512, n_slots=2, step_chunk=64,
              dtype=torch.float32, device="cpu")
    s = c.acquire()
    c.reserve(s, 200)
    c.commit(s, 200)
    assert c.pages_held() == 4
    c.truncate(s, 70)
    assert c.length(s) == 70 and c.pages_held() == 2
    with pytest.raises(CacheError, match="cannot truncate"):
        c.truncate(s, 71)
    c.truncate(s, 0)
    assert c.pages_held() == 0 and c.kv_groups[0].pool.n_free == 8
    w = _cache()
    s = w.acquire()
    w.reserve(s, 100)
    w.commit(s, 100)
    with pytest.raises(CacheError, match="only be truncated to its start"):
        w.truncate(s, 50)
    w.truncate(s, 0)
    assert w.pages_held() == 0
