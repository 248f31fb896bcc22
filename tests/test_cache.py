import random

import pytest
import torch

from brolm_b200.cache import Cache, CacheError, CacheFull, KVSpec, PagePool, SlotTable, StateSpec


def test_page_pool_never_loses_or_doubles_a_page():
    pool = PagePool(10)
    held = []
    rng = random.Random(0)
    for _ in range(500):
        if held and rng.random() < 0.5:
            k = rng.randrange(1, len(held) + 1)
            rng.shuffle(held)
            pool.free(held[:k])
            held = held[k:]
        else:
            k = rng.randrange(0, 4)
            if k <= pool.free_pages:
                got = pool.alloc(k)
                assert not set(got) & set(held)
                held += got
            else:
                with pytest.raises(CacheFull):
                    pool.alloc(k)
        assert pool.free_pages + len(held) == 10 and len(set(held)) == len(held)
    pool.free(held)
    assert pool.free_pages == 10 and sorted(pool.alloc(10)) == list(range(10))


def test_double_free_and_foreign_pages_raise():
    pool = PagePool(4)
    a = pool.alloc(2)
    pool.free(a)
    with pytest.raises(CacheError):
        pool.free(a[:1])
    with pytest.raises(CacheError):
        pool.free([7])
    slots = SlotTable(2)
    s = slots.alloc()
    slots.free(s)
    with pytest.raises(CacheError):
        slots.free(s)
    slots.alloc(), slots.alloc()
    with pytest.raises(CacheFull):
        slots.alloc()


def specs():
    full, win = KVSpec(2, 16, None), KVSpec(2, 16, 100)
    return [win, full, win, None, StateSpec((3, 5), torch.float32)]


def test_groups_have_storage_of_their_own():
    c = Cache(specs(), max_tokens=1000, dtype=torch.float32, device="cpu", max_slots=3)
    assert c.num_pages == 16 and c.max_tokens == 1024
    win, full = c.kv_groups
    assert win.entries == [0, 2] and full.entries == [1] and win.ring == 128 and full.ring is None
    assert tuple(win.k.shape) == (2, 6, 2, 64, 16)          # 3 slots x 2 ring pages is all it can ever need
    assert tuple(full.k.shape) == (1, 16, 2, 64, 16)
    assert tuple(c.state_groups[0].data.shape) == (1, 3 + 1, 3, 5)      # a spare row for a step's padding rows
    assert c.padding_slot == 3
    assert c.entries[3] is None and c.entry(2).index == 1 and c.entry(1).k.shape[0] == 16
    with pytest.raises(CacheError):
        c.entry(3)


def test_sequences_grow_by_pages_and_the_ring_stops_growing():
    c = Cache(specs(), max_tokens=1024, dtype=torch.float32, device="cpu", max_slots=3)
    win, full = c.kv_groups
    s = c.alloc_slot()
    for n, (pw, pf) in [(1, (1, 1)), (64, (1, 1)), (65, (2, 2)), (128, (2, 2)), (129, (2, 3)), (500, (2, 8))]:
        c.reserve({s: n})
        c.commit({s: n})
        assert (len(win.pages[s]), len(full.pages[s])) == (pw, pf) and c.length(s) == n
    t = c.page_table(1, [s, -1], width=10, rows=3)
    assert t.shape == (3, 10) and t[0, :8].tolist() == full.pages[s] and t[1:].abs().sum() == 0
    with pytest.raises(CacheError):
        c.reserve({s: 10})                                   # cannot shrink
    c.free_slot(s)
    assert win.pool.held_pages == 0 and full.pool.held_pages == 0
    with pytest.raises(CacheError):
        c.free_slot(s)
    with pytest.raises(CacheError):
        c.length(s)


def test_reserve_is_all_or_nothing():
    c = Cache([KVSpec(1, 16, None)], max_tokens=256, dtype=torch.float32, device="cpu")
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve({a: 100})
    with pytest.raises(CacheFull, match="sized for 256"):
        c.reserve({a: 130, b: 100})                          # needs 1 + 2 pages, 2 are free
    assert c.kv_groups[0].pool.free_pages == 2 and len(c.kv_groups[0].pages[b]) == 0


def test_slots_come_back_and_state_starts_at_zero():
    c = Cache(specs(), max_tokens=640, dtype=torch.float32, device="cpu", max_slots=2)
    rng = random.Random(1)
    live = {}
    for _ in range(300):
        if live and (rng.random() < 0.4 or c.slots.free_slots == 0):
            s = rng.choice(list(live))
            c.state_groups[0].data[:, s] = 7.0
            c.free_slot(s)
            del live[s]
        else:
            s = c.alloc_slot()
            assert s not in live and float(c.state_groups[0].data[:, s].abs().sum()) == 0.0
            n = rng.randrange(1, 300)
            c.reserve({s: n})
            c.commit({s: n})
            live[s] = n
        for g in c.kv_groups:
            owned = [p for s in live for p in g.pages[s]]
            assert len(owned) == len(set(owned)) == g.pool.held_pages
        assert c.live_slots == len(live)
    with pytest.raises(CacheFull):
        for _ in range(3):
            c.alloc_slot()


def test_write_rows_follow_the_pages_and_skip_what_the_ring_drops():
    c = Cache([KVSpec(1, 16, None), KVSpec(1, 16, 100)], max_tokens=1024, dtype=torch.float32, device="cpu")
    full, win = c.kv_groups
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve({a: 300, b: 3})
    rows = c.write_rows(0, [a, b], [0, 0], [300, 3])
    assert rows.shape == (303,) and rows[0] == full.pages[a][0] * 64 and rows[299] == full.pages[a][4] * 64 + 43
    assert rows[300] == full.pages[b][0] * 64
    rows = c.write_rows(1, [a, b], [0, 0], [300, 3])                 # ring of 128: the first 172 are dropped
    assert (rows[:172] == -1).all() and (rows[172:300] >= 0).all() and len(set(rows[172:300].tolist())) == 128
    assert rows[172] == win.pages[a][(172 % 128) // 64] * 64 + 172 % 64
    c.commit({a: 300, b: 3})
    c.reserve({a: 301, b: 4})
    rows = c.write_rows(1, [a, -1, b], [300, 0, 3], [301, 1, 4])       # a decode step with a padding row
    assert rows.tolist() == [win.pages[a][(300 % 128) // 64] * 64 + 300 % 64, -1, win.pages[b][0] * 64 + 3]


def test_decode_rows_equal_write_rows_for_one_token():
    """The decode step's scalar form of write_rows: the same places, through the ring's wrap as well."""
    cache = Cache([KVSpec(2, 16, None), KVSpec(2, 16, 96)], max_tokens=64 * 12, dtype=torch.float32, device="cpu",
                  max_slots=3)
    slots = [cache.alloc_slot() for _ in range(3)]
    lengths = [0, 0, 0]
    rng = random.Random(3)
    first = [5, 70, 130]
    cache.reserve(dict(zip(slots, first)))
    cache.commit(dict(zip(slots, first)))
    lengths = list(first)
    for _ in range(150):
        new = [n + 1 for n in lengths]
        cache.reserve(dict(zip(slots, new)))
        for g in range(2):
            want = cache.write_rows(g, slots + [-1], lengths + [0], new + [1]).tolist()
            assert cache.decode_rows(g, slots + [-1], lengths + [0]) == want
        cache.commit(dict(zip(slots, new)))
        lengths = new


def test_pages_signature_changes_with_the_table():
    cache = Cache([KVSpec(1, 16, None)], max_tokens=64 * 8, dtype=torch.float32, device="cpu", max_slots=2)
    a = cache.alloc_slot()
    cache.reserve({a: 10})
    cache.commit({a: 10})
    sig = cache.pages_signature(0, [a, -1])
    cache.reserve({a: 64})
    assert cache.pages_signature(0, [a, -1]) == sig            # same page
    cache.reserve({a: 65})
    assert cache.pages_signature(0, [a, -1]) != sig            # a page was added
    sig = cache.pages_signature(0, [a])
    pages = list(cache.kv_groups[0].pages[a])
    cache.free_slot(a)
    b = cache.alloc_slot()
    cache.reserve({b: 65})
    assert b == a and len(cache.kv_groups[0].pages[b]) == len(pages)
    assert cache.pages_signature(0, [b]) != sig                # the same slot, another tenant
