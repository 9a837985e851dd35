"""The cache's bookkeeping: slots, pages, lengths, groups, state (no device)."""
import random

import pytest
import torch

from picolm_b200.cache import CacheFull, CacheSpec, IndexPool, SequenceCache, PAGE_TOKENS


def test_pool_never_loses_or_doubles():
    p = IndexPool(5, first=1, what="page")
    got = [p.take() for _ in range(5)]
    assert sorted(got) == [1, 2, 3, 4, 5]
    with pytest.raises(CacheFull):
        p.take()
    p.give_back(3)
    with pytest.raises(RuntimeError, match="freed twice"):
        p.give_back(3)
    with pytest.raises(RuntimeError, match="does not belong"):
        p.give_back(17)
    assert p.take() == 3
    p.check()


def _cache(**kw):
    specs = [CacheSpec.kv(2, 16), CacheSpec.kv(2, 16), CacheSpec.kv(2, 16, window=100), CacheSpec.state((3, 4)), None]
    args = dict(max_tokens=640, max_seqs=4, kv_dtype=torch.float32, device="cpu")
    args.update(kw)
    return SequenceCache(specs, **args)


def test_groups_have_storage_of_their_own():
    c = _cache()
    assert len(c.kv_groups) == 2
    assert c.kv_groups[0].layers == [0, 1] and c.kv_groups[1].layers == [2]
    assert c.kv_groups[0].k.shape == (2, 11, 2, PAGE_TOKENS, 16)           # 10 pages + the null page
    assert c.kv_groups[1].k.shape == (1, 11, 2, PAGE_TOKENS, 16)
    assert c.kv_groups[0].k.data_ptr() != c.kv_groups[1].k.data_ptr()
    assert c.state[3].shape == (5, 3, 4) and 4 not in c.layer_group and 4 not in c.state     # 4 slots + the null slot
    assert c.null_slot == 4 and not c.slots.holds(c.null_slot)


def test_lengths_pages_and_release():
    c = _cache()
    a, b = c.allocate(), c.allocate()
    c.reserve([(a, 70), (b, 5)])
    assert [len(c.kv_groups[0].pages[s]) for s in (a, b)] == [2, 1]
    assert 0 not in c.kv_groups[0].pages[a]                                   # the null page is never handed out
    c.advance(a, 70), c.advance(b, 5)
    assert c.length(a) == 70 and c.length(b) == 5
    c.reserve([(a, 1), (b, 1)])
    assert [len(c.kv_groups[0].pages[s]) for s in (a, b)] == [2, 1]          # still room on the last pages
    c.advance(a, 1), c.advance(b, 1)
    c.check()
    c.release(b)
    with pytest.raises(RuntimeError, match="freed twice|not in use"):
        c.release(b)
    with pytest.raises(RuntimeError, match="not in use"):
        c.reserve([(b, 1)])
    c.check()
    assert c.kv_groups[0].pool.used == 2
    b2 = c.allocate()
    assert b2 == b and c.length(b2) == 0                                       # the slot is used again, empty


def test_reserve_is_all_or_nothing():
    c = _cache()
    s = [c.allocate() for _ in range(3)]
    c.reserve([(s[0], 300)])
    c.advance(s[0], 300)
    free_before = c.kv_groups[0].pool.free
    with pytest.raises(CacheFull):
        c.reserve([(s[1], 200), (s[2], 200)])                                  # 5 + 4 + 4 pages > 10
    assert c.kv_groups[0].pool.free == free_before and c.kv_groups[0].pages[s[1]] == []
    with pytest.raises(RuntimeError, match="twice"):
        c.reserve([(s[1], 1), (s[1], 1)])
    c.check()


def test_longest_sequence_is_enforced():
    c = _cache(max_seq_tokens=100)
    s = c.allocate()
    with pytest.raises(CacheFull, match="longest sequence"):
        c.reserve([(s, 101)])
    c.reserve([(s, 100)])


def test_window_group_gives_pages_back():
    c = _cache()
    s = c.allocate()
    c.reserve([(s, 300)])
    c.advance(s, 300)
    full, win = c.kv_groups[0], c.kv_groups[1]
    assert sum(1 for p in full.pages[s] if p) == 5
    # next query is position 300 and reads from 201: blocks 0..2 (positions < 192) are gone
    assert [bool(p) for p in win.pages[s]] == [False, False, False, True, True]
    c.check()
    c.release(s)
    c.check()
    assert win.pool.used == 0 and full.pool.used == 0


def test_state_is_zeroed_when_a_slot_is_handed_out():
    c = _cache()
    s = c.allocate()
    c.state[3][s] += 5.0
    c.release(s)
    s2 = c.allocate()
    assert s2 == s and torch.count_nonzero(c.state[3][s2]) == 0


def test_random_traffic_keeps_the_books(seed=3):
    rnd = random.Random(seed)
    c = _cache(max_tokens=64 * 40, max_seqs=6)
    live = {}
    for _ in range(400):
        r = rnd.random()
        if r < 0.3 and c.slots.free:
            live[c.allocate()] = 0
        elif r < 0.8 and live:
            s = rnd.choice(list(live))
            n = rnd.choice([1, 1, 1, 7, 64, 130])
            try:
                c.reserve([(s, n)])
                c.advance(s, n)
                live[s] += n
            except CacheFull:
                pass
        elif live:
            s = rnd.choice(list(live))
            c.release(s)
            del live[s]
        c.check()
        assert {s: c.length(s) for s in live} == live
    for s in list(live):
        c.release(s)
    c.check()
    assert all(g.pool.used == 0 for g in c.kv_groups) and c.slots.used == 0
