"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

KvNeed = None


@pytest.fixture(scope="module")
def C(llogos):
    return llogos.cache


@pytest.fixture(scope="module")
def P(llogos):
    return llogos.parts


def make(C, P, *, max_tokens=64 * 10, max_seq_len=64 * 6, n_slots=4, window=0, extra_state=False):
    needs = {0: P.KvNeed(2, 16, 0), 1: P.KvNeed(2, 16, window), 2: P.KvNeed(2, 16, 0)}
    if extra_state:
        needs[3] = P.StateNeed((3, 5))
    return C.SequenceCache(needs, max_tokens=max_tokens, max_seq_len=max_seq_len, n_slots=n_slots,
                           dtype=torch.float32, device=torch.device("cpu"))


def test_free_list(C):
    f = C.FreeList(3, "page")
    a = f.take(2)
    assert a == [0, 1] and f.free_count == 1
    with pytest.raises(C.CacheError, match="out of pages"):
        f.take(2)
    f.give([0])
    with pytest.raises(C.CacheError, match="not held"):
        f.give([0])
    with pytest.raises(C.CacheError, match="not held"):
        f.give([2])
    with pytest.raises(C.CacheError):
        f.give([1, 1])
    assert f.take(2) == [0, 2]


def test_slots_are_reused_and_never_double_freed(C, P):
    c = make(C, P)
    slots = [c.acquire() for _ in range(4)]
    assert sorted(slots) == [0, 1, 2, 3]
    with pytest.raises(C.CacheError, match="out of slots"):
        c.acquire()
    c.release(slots[1])
    with pytest.raises(C.CacheError, match="not in use"):
        c.release(slots[1])
    assert c.acquire() == slots[1]
    with pytest.raises(C.CacheError, match="not in use"):
        c.length(17)


def test_groups_by_need(C, P):
    c = make(C, P, window=100)
    assert len(c.kv_groups) == 2
    full = [g for g in c.kv_groups if g.window == 0][0]
    ring = [g for g in c.kv_groups if g.window == 100][0]
    assert full.units == [0, 2] and ring.units == [1]
    assert full.ring_pages == 6 and ring.ring_pages == 3          # ceil(100 / 64) + 1
    # one page and one table row more than sequences can get: the padding slot's
    assert full.k[0].shape == (11, 2, 64, 16) and ring.page_table.shape == (5, 3)
    assert c.pad_slot == 4 and ring.page_table[4].tolist() == [10, 10, 10]
    assert c.view(1).window == 100 and c.view(0).ring_pages == 6


def test_pages_follow_lengths(C, P):
    c = make(C, P, window=100)
    full = [g for g in c.kv_groups if g.window == 0][0]
    ring = [g for g in c.kv_groups if g.window == 100][0]
    s = c.acquire()
    c.check_room([(s, 130)])
    ups = dict((id(g), u) for g, u in c.grow([(s, 130)]))
    c.commit([(s, 130)])
    assert c.length(s) == 130 and len(full.pages_of[s]) == 3 and len(ring.pages_of[s]) == 3
    assert [i for i, _ in ups[id(full)]] == [s * 6 + 0, s * 6 + 1, s * 6 + 2]
    c.grow([(s, 200)])
    c.commit([(s, 200)])
    assert len(full.pages_of[s]) == 6 and len(ring.pages_of[s]) == 3    # the ring does not grow
    with pytest.raises(C.CacheError, match="longest sequence"):
        c.check_room([(s, 64 * 6 - 330 + 1)])
    c.audit()
    c.release(s)
    assert full.pool.free_count == 10 and ring.pool.free_count == 10
    c.audit()


def test_step_checks(C, P):
    c = make(C, P)
    a, b = c.acquire(), c.acquire()
    with pytest.raises(C.CacheError, match="twice"):
        c.check_room([(a, 1), (a, 1)])
    with pytest.raises(C.CacheError, match="at least one"):
        c.check_room([(a, 0)])
    with pytest.raises(C.CacheError, match="not in use"):
        c.check_room([(3, 1)])
    c.grow([(a, 64 * 6)])
    c.commit([(a, 64 * 6)])
    with pytest.raises(C.CacheError, match="cache full"):
        c.check_room([(b, 64 * 4 + 1)])
    c.check_room([(b, 64 * 4)])


def test_state_is_zeroed_for_a_new_sequence(C, P):
    c = make(C, P, extra_state=True)
    s = c.acquire()
    v = c.view(3)
    assert v.state.shape == (5, 3, 5)
    v.state[s] += 7
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(c.view(3).state[s2].abs().sum()) == 0


def test_random_traffic_keeps_the_books(C, P):
    rng = random.Random(0)
    c = make(C, P, max_tokens=64 * 40, max_seq_len=64 * 12, n_slots=8, window=70)
    live = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.3 and c.slots.free_count:
            live[c.acquire()] = 0
        elif r < 0.5 and live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        elif live:
            batch = rng.sample(list(live), rng.randint(1, len(live)))
            growth = [(s, rng.choice([1, 1, 1, 5, 64, 130])) for s in batch]
            try:
                c.check_room(growth)
            except C.CacheError:
                continue
            c.grow(growth)
            c.commit(growth)
            for s, a in growth:
                live[s] += a
        c.audit()
        assert {s: c.length(s) for s in live} == live
        for g in c.kv_groups:
            for s, n in live.items():
                assert len(g.pages_of.get(s, [])) == g.pages_needed(n)
    for s in list(live):
        c.release(s)
    c.audit()
    assert all(g.pool.free_count == g.pool.n for g in c.kv_groups) and c.slots.free_count == 8


def test_truncate_gives_pages_back_and_refuses_what_is_lost(C, P):
    c = make(C, P, window=100)
    full = [g for g in c.kv_groups if g.window == 0][0]
    ring = [g for g in c.kv_groups if g.window == 100][0]
    s = c.acquire()

    def add(n):
        c.check_room([(s, n)])
        c.grow([(s, n)])
        c.commit([(s, n)])

    add(190)                                       # 3 pages everywhere; the ring (3 pages) has not gone round
    c.truncate(s, 100)
    assert c.length(s) == 100 and len(full.pages_of[s]) == 2 and len(ring.pages_of[s]) == 2
    assert full.pool.free_count == 8 and ring.pool.free_count == 8
    c.audit()
    add(250)                                       # 350 tokens: the ring has gone round (pages 3, 4, 5 are kept)
    assert len(full.pages_of[s]) == 6 and len(ring.pages_of[s]) == 3
    c.truncate(s, 300)                             # position 300 looks back to 201: page 3 is still there
    assert c.length(s) == 300 and len(full.pages_of[s]) == 5 and len(ring.pages_of[s]) == 3
    with pytest.raises(C.CacheError, match="overwritten"):
        c.truncate(s, 250)                         # would need keys from 151 on: page 2 is gone
    assert c.length(s) == 300 and len(full.pages_of[s]) == 5
    with pytest.raises(C.CacheError, match="cannot truncate"):
        c.truncate(s, 301)
    c.truncate(s, 300)                             # no change
    c.audit()
    c.release(s)
    assert full.pool.free_count == 10 and ring.pool.free_count == 10
    c2 = make(C, P, extra_state=True)
    s2 = c2.acquire()
    c2.check_room([(s2, 5)]); c2.grow([(s2, 5)]); c2.commit([(s2, 5)])
    with pytest.raises(C.CacheError, match="state"):
        c2.truncate(s2, 2)
