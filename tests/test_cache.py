"""Slots and pages of the cache: nothing lost, held twice or freed twice (no GPU)."""
import random

import pytest

from airframe_b200.cache import CacheFull, ContextOverflow, IndexPool, PoolError, SequenceCache, pages_for
from airframe_b200.parts import KVNeed, StateNeed

PAGE = 64


def test_pool_gives_each_index_once_and_lowest_first():
    p = IndexPool(4, "slot")
    got = [p.take() for _ in range(4)]
    assert got == [0, 1, 2, 3] and p.n_free == 0
    with pytest.raises(CacheFull, match="no free slot"):
        p.take()
    p.give_back(2)
    p.give_back(0)
    assert p.take() == 0 and p.take() == 2
    with pytest.raises(PoolError, match="not held"):
        p.give_back(7)
    p.give_back(1)
    with pytest.raises(PoolError, match="freed twice"):
        p.give_back(1)


def _needs():
    # run 0: window 100 (ring of 128 rows); run 1: all keys; run 2: reads run 1; run 3: state only
    return [(KVNeed(2, 16, 100), None, None), (KVNeed(2, 16, None), None, None),
            (KVNeed(2, 16, None), None, 1), (None, StateNeed((3, 5)), None)]


def test_groups_and_views():
    c = SequenceCache(_needs(), max_tokens=640, max_context=512)
    assert c.total_pages == 10 and c.n_slots == 10
    assert len(c.groups) == 2
    ring = c.groups[KVNeed(2, 16, 100)]
    full = c.groups[KVNeed(2, 16, None)]
    assert ring.ring_rows == 128 and ring.pages_per_seq == 2 and full.ring_rows == 0 and full.pages_per_seq == 8
    assert full.run_ids == [1]                                # run 2 keeps no storage of its own
    v = c.views
    assert (v[0].writes, v[1].writes, v[2].writes) == (True, True, False)
    assert v[2].cache_id == 1 and v[1].keep_step_kv and not v[0].keep_step_kv
    assert v[3].kv is None


def test_pages_follow_lengths_and_come_back():
    c = SequenceCache(_needs(), max_tokens=640, max_context=512)
    ring = c.groups[KVNeed(2, 16, 100)]
    full = c.groups[KVNeed(2, 16, None)]
    a, b = c.take_slot(), c.take_slot()
    c.reserve({a: 65, b: 300})
    c.commit({a: 65, b: 300})
    assert len(full.held[a]) == 2 and len(full.held[b]) == 5
    assert len(ring.held[a]) == 2 and len(ring.held[b]) == 2       # a ring never holds more than its rows
    assert c.length(a) == 65 and c.length(b) == 300
    held = set(full.held[a]) | set(full.held[b])
    assert len(held) == 7                                           # no page held twice
    assert list(full.table_host[a, :2]) == full.held[a] and int(full.table_host[a, 2]) == -1
    c.reserve({a: 66})
    assert len(full.held[a]) == 2                                   # same page
    c.reserve({a: 129})
    assert len(full.held[a]) == 3
    with pytest.raises(CacheFull):
        c.reserve({a: 384})                                         # 3 more pages wanted, 2 free
    assert len(full.held[a]) == 3 and full.pages.n_free == 2        # a failed reserve changes nothing
    with pytest.raises(ContextOverflow):
        c.reserve({a: 513})
    c.free_slot(b)
    assert full.pages.n_free == 7 and ring.pages.n_free == ring.n_pages - 2
    with pytest.raises(PoolError, match="not held"):
        c.free_slot(b)
    with pytest.raises(PoolError):
        c.length(b)
    assert c.take_slot() == b and c.length(b) == 0                  # the slot is used again, empty
    assert int(full.table_host[b, 0]) == -1


def test_random_traffic_never_loses_or_doubles_anything():
    rng = random.Random(5)
    c = SequenceCache(_needs(), max_tokens=64 * 40, max_context=1024, max_sequences=12)
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.3 and c.slots.n_free:
            s = c.take_slot()
            assert s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            new = live[s] + (rng.randrange(1, 200) if live[s] == 0 else 1)
            try:
                c.reserve({s: new})
                c.commit({s: new})
                live[s] = new
            except (CacheFull, ContextOverflow):
                pass
        elif live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        assert c.slots.n_held == len(live) and c.slots.n_held + c.slots.n_free == c.n_slots
        for g in c.groups.values():
            pages = [p for s in range(c.n_slots) for p in g.held[s]]
            assert len(pages) == len(set(pages)) == g.pages.n_held
            assert g.pages.n_held + g.pages.n_free == g.n_pages
            for s in range(c.n_slots):
                want = pages_for(g.rows_held(live[s])) if s in live else 0
                assert len(g.held[s]) == want
    for s in list(live):
        c.free_slot(s)
    assert all(g.pages.n_held == 0 for g in c.groups.values()) and c.slots.n_held == 0


def test_slot_count_and_ring_pool_are_bounded():
    c = SequenceCache(_needs(), max_tokens=64 * 100, max_context=4096, max_sequences=4)
    assert c.n_slots == 4
    assert c.groups[KVNeed(2, 16, 100)].n_pages == 8               # 4 sequences x 2 ring pages
    assert c.groups[KVNeed(2, 16, None)].n_pages == 100


def test_reading_a_cache_with_other_head_sizes_is_refused():
    with pytest.raises(ValueError, match="other head sizes"):
        SequenceCache([(KVNeed(2, 16, None), None, None), (KVNeed(4, 16, None), None, 0)], 640, 512)


def test_a_group_with_a_window_has_storage_of_its_own_size():
    """With the most sequences named, the ring's group holds slots x ring pages, fewer than the group that
    keeps all keys; ``fits`` answers for every group."""
    c = SequenceCache(_needs(), max_tokens=64 * 40, max_context=1024, max_sequences=4)
    ring, full = c.groups[KVNeed(2, 16, 100)], c.groups[KVNeed(2, 16, None)]
    assert full.n_pages == 40 and ring.n_pages == 4 * 2
    assert c.fits([640, 640, 640, 640])                   # 40 pages of all keys, 8 of the ring
    assert not c.fits([640, 640, 640, 641])               # a 41st page of all keys
    assert not c.fits([64] * 5)                           # a fifth slot
    # without the most sequences there are as many slots as pages and the ring's group saves nothing
    c = SequenceCache(_needs(), max_tokens=64 * 40, max_context=1024)
    assert c.groups[KVNeed(2, 16, 100)].n_pages == 40
