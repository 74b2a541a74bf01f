"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from rustyllm_b200.cache.allocators import CacheFull, CacheMisuse, FreeList
from rustyllm_b200.cache.sequence_cache import KVNeed, SequenceCache, StateNeed

PAGE = 64


def test_free_list_hands_out_each_id_once_and_lowest_first():
    fl = FreeList(5, "slot")
    assert fl.take(3) == [0, 1, 2]
    fl.give_back([1])
    assert fl.take(1) == [1]            # reused at once
    assert fl.take(2) == [3, 4]
    with pytest.raises(CacheFull):
        fl.take(1)
    fl.check()


def test_free_list_refuses_double_free_and_foreign_ids():
    fl = FreeList(3, "page")
    (a,) = fl.take(1)
    fl.give_back([a])
    with pytest.raises(CacheMisuse, match="freed twice"):
        fl.give_back([a])
    with pytest.raises(CacheMisuse, match="does not exist"):
        fl.give_back([7])
    fl.check()


def _cache(max_tokens=64 * 8, window=None, state=0, **kw):
    kv = [KVNeed(2, 16, None), KVNeed(2, 16, None), KVNeed(1, 32, window)]
    st = [None, StateNeed(state) if state else None, None]
    return SequenceCache(kv, st, max_tokens, torch.float32, "cpu", **kw)


def test_layers_with_equal_needs_share_a_group():
    c = _cache()
    assert len(c.groups) == 2
    assert c.entry_group == [(0, 0), (0, 1), (1, 0)]
    assert c.groups[0].keys.shape == (2, 8, 2, PAGE, 16) and c.groups[0].values.shape == (2, 8, 2, PAGE, 16)
    assert c.groups[1].keys.shape == (1, 8, 1, PAGE, 32)


def test_value_heads_of_another_width_get_storage_of_their_own():
    kv = [KVNeed(2, 16, None), KVNeed(2, 16, None, value_dim=8), KVNeed(2, 16, None, value_dim=8), KVNeed(2, 16, None, value_dim=16)]
    c = SequenceCache(kv, [None] * 4, 64 * 4, torch.float32, "cpu")
    assert len(c.groups) == 2 and c.entry_group[3][0] == c.entry_group[0][0]    # value_dim = head_dim is the plain need
    wide = c.groups[c.entry_group[1][0]]
    assert c.entry_group[1][0] == c.entry_group[2][0] != c.entry_group[0][0]
    assert wide.keys.shape == (2, 4, 2, PAGE, 16) and wide.values.shape == (2, 4, 2, PAGE, 8)
    assert wide.bytes_per_token() == 2 * 2 * (16 + 8) * 4
    assert c.memory_bytes() >= wide.keys.numel() * 4 + wide.values.numel() * 4


def test_pages_follow_lengths_and_come_back():
    c = _cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a, b], [65, 3]); c.commit([a, b], [65, 3])
    assert c.length(a) == 65 and c.length(b) == 3
    g = c.groups[0]
    assert len(g.slot_pages[a]) == 2 and len(g.slot_pages[b]) == 1
    assert g.page_table_host[a, :2].tolist() == g.slot_pages[a]
    assert c.free_pages == 5
    for _ in range(61):
        c.prepare([b], [1]); c.commit([b], [1])
    assert c.length(b) == 64 and len(g.slot_pages[b]) == 1
    c.prepare([b], [1]); c.commit([b], [1])
    assert len(g.slot_pages[b]) == 2
    c.check()
    c.free_slot(a)
    assert c.free_pages == 6
    c.check()
    with pytest.raises(CacheMisuse):
        c.free_slot(a)
    with pytest.raises(CacheMisuse):
        c.prepare([a], [1])
    a2 = c.alloc_slot()
    assert a2 == a and c.length(a2) == 0       # the slot is used again, empty


def test_prepare_is_all_or_nothing():
    c = _cache(max_tokens=64 * 4)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a], [128]); c.commit([a], [128])
    with pytest.raises(CacheFull):
        c.prepare([a, b], [64, 65])            # needs 1 + 2 pages, 2 free
    assert c.free_pages == 2 and len(c.groups[0].slot_pages[b]) == 0
    c.prepare([a, b], [64, 64]); c.commit([a, b], [64, 64])
    assert c.free_pages == 0
    c.check()
    with pytest.raises(CacheMisuse, match="twice"):
        c.prepare([a, a], [1, 1])


def test_longest_sequence_is_enforced():
    c = _cache(max_tokens=64 * 8, max_seq_len=100)
    a = c.alloc_slot()
    c.prepare([a], [100]); c.commit([a], [100])
    with pytest.raises(CacheFull, match="longest"):
        c.prepare([a], [1])


def test_window_group_gives_pages_back_behind_the_window():
    c = _cache(max_tokens=64 * 8, window=70)
    a = c.alloc_slot()
    c.prepare([a], [200]); c.commit([a], [200])
    full, win = c.groups[0], c.groups[1]
    assert sum(p >= 0 for p in full.slot_pages[a]) == 4
    # next query at position 200 reads positions >= 131: pages 0 and 1 are dead
    assert [p >= 0 for p in win.slot_pages[a]] == [False, False, True, True]
    c.check()
    c.free_slot(a)
    assert win.pages.free_count == win.num_pages
    c.check()


def test_state_area_is_zeroed_when_a_slot_is_handed_out():
    c = _cache(state=40)
    assert c.state_bytes == 256 and c.state_entry(0) is None
    a = c.alloc_slot()
    view = c.state_entry(1)
    assert view.shape == (c.max_slots, 40)
    view[a].fill_(7)
    c.free_slot(a)
    assert c.alloc_slot() == a
    assert int(c.state_entry(1)[a].sum()) == 0


def test_random_traffic_keeps_the_invariants():
    rng = random.Random(0)
    c = _cache(max_tokens=64 * 32, window=100, max_slots=6)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            live[c.alloc_slot()] = 0
        elif op < 0.4 and live:
            s = rng.choice(list(live))
            c.free_slot(s); del live[s]
        elif live:
            ss = rng.sample(list(live), rng.randint(1, len(live)))
            ns = [rng.choice([1, 1, 1, 5, 64, 130]) for _ in ss]
            try:
                c.prepare(ss, ns)
            except CacheFull:
                continue
            c.commit(ss, ns)
            for s, n in zip(ss, ns):
                live[s] += n
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert all(g.pages.free_count == g.num_pages for g in c.groups)
    assert c.slots.free_count == 6
