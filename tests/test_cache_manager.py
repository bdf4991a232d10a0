"""The cache manager on the host: no page lost, held twice or freed twice, under random orders
of requests; windows give pages back; state slots are reused (no GPU)."""
import random

import pytest

from lightllm_b200.cache import (CacheError, CacheLayout, CacheManager, CacheSpec, KVSpec, OutOfPages, PagePool,
                                 StateSpec)


def layout(window=None, state=False):
    specs = [CacheSpec(kv=KVSpec(2, 16)), CacheSpec(kv=KVSpec(2, 16, window), state=StateSpec((4,)) if state else None),
             CacheSpec(kv=KVSpec(2, 16))]
    return CacheLayout.build(specs, [None, None, None])


def test_layout_groups_planes_by_need():
    lo = layout(window=8, state=True)
    assert lo.groups == [KVSpec(2, 16), KVSpec(2, 16, 8)] and lo.planes_per_group == [2, 1]
    assert [(r.group, r.plane) for r in lo.refs] == [(0, 0), (1, 0), (0, 1)]
    assert lo.refs[1].state_plane == 0 and len(lo.state_planes) == 1
    shared = CacheLayout.build([CacheSpec(kv=KVSpec(1, 8)), CacheSpec(kv=KVSpec(1, 8))], [None, 0])
    assert shared.planes_per_group == [1] and not shared.refs[1].owns and shared.refs[1].plane == 0
    with pytest.raises(ValueError, match="does not fit"):
        CacheLayout.build([CacheSpec(kv=KVSpec(1, 8)), CacheSpec(kv=KVSpec(2, 8))], [None, 0])
    with pytest.raises(ValueError, match="window"):
        CacheLayout.build([CacheSpec(kv=KVSpec(1, 8, 4)), CacheSpec(kv=KVSpec(1, 8))], [None, 0])


def test_pool_refuses_double_free_and_foreign_free():
    p = PagePool(3)
    a = p.take("x")
    with pytest.raises(CacheError, match="belongs to"):
        p.give(a, "y")
    p.give(a, "x")
    with pytest.raises(CacheError, match="freed twice"):
        p.give(a, "x")
    assert p.take("z") == a            # a page just given back is the next one handed out
    p.take("z"), p.take("z")
    with pytest.raises(OutOfPages):
        p.take("z")
    p.check()


def test_reserve_is_all_or_nothing_and_advance_needs_pages():
    m = CacheManager(layout(), page_size=4, num_pages=5, max_seqs=2, max_seq_len=64)
    m.open("a"), m.open("b")
    m.reserve("a", 9)                   # 3 pages
    assert m.free_pages() == 2
    with pytest.raises(OutOfPages):
        m.reserve("b", 12)
    assert m.free_pages() == 2 and m.block_table("b", 0) == []
    m.advance("a", 9)
    assert not m.can_reserve_all([("a", 4), ("b", 8)]) and m.can_reserve_all([("a", 3), ("b", 8)])
    with pytest.raises(OutOfPages):
        m.reserve_all([("a", 4), ("b", 8)])
    assert m.free_pages() == 2
    with pytest.raises(CacheError, match="without pages"):
        m.advance("b", 1)
    assert m.slot_mapping("a", 0, 7, 2) == [m.block_table("a", 0)[1] * 4 + 3, m.block_table("a", 0)[2] * 4]
    with pytest.raises(OutOfPages, match="request slots"):
        m.open("c")
    m.close("a")
    with pytest.raises(CacheError, match="not open"):
        m.close("a")
    assert m.free_pages() == 5
    m.check()


def test_window_gives_pages_back_and_they_are_reused():
    m = CacheManager(layout(window=6), page_size=4, num_pages=[10, 6], max_seqs=2, max_seq_len=200)
    m.open("a")
    used_windowed = []
    for _ in range(40):
        m.reserve("a", 1)
        m.advance("a", 1)
        used_windowed.append(m.used_pages(1))
        m.check()
    # the windowed group never holds more than ceil((window-1)/page)+1 pages; the full group grows
    assert max(used_windowed) <= 3
    assert m.used_pages(0) == 10
    t = m.block_table("a", 1)
    assert t[0] == -1 and t[-1] >= 0 and len(t) == 10
    live = [p for p in t if p >= 0]
    assert len(set(live)) == len(live)
    with pytest.raises(CacheError, match="given back"):
        m.slot_mapping("a", 1, 0, 1)
    m.close("a")
    assert m.free_pages(0) == 10 and m.free_pages(1) == 6


def test_full_group_limits_a_long_request_not_the_windowed_one():
    m = CacheManager(layout(window=6), page_size=4, num_pages=[4, 3], max_seqs=1, max_seq_len=200)
    m.open("a")
    n = 0
    while m.can_reserve("a", 1):
        m.reserve("a", 1)
        m.advance("a", 1)
        n += 1
    assert n == 16                     # 4 pages of the full group
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = CacheManager(layout(window=10, state=True), page_size=4, num_pages=[24, 9], max_seqs=4, max_seq_len=60)
    live, next_id, slots_seen = {}, 0, set()
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            seq = m.open(next_id)
            slots_seen.add(seq.slot)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 16])
            if m.can_reserve(rid, n):
                m.reserve(rid, n)
                if rng.random() < 0.9:          # sometimes reserved pages stay unused for a while
                    m.advance(rid, n)
                    live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.get(rid).length == n
    for rid in list(live):
        m.close(rid)
    m.check()
    assert m.free_pages(0) == 24 and m.free_pages(1) == 9 and m.free_slots == 4
    assert slots_seen <= {0, 1, 2, 3} and next_id > 4          # slots were used again


def test_pages_taken_in_one_slice_come_in_the_order_of_single_takes():
    a, b = PagePool(10), PagePool(10)
    a.take("w"), b.take("w")
    singles = [a.take("x") for _ in range(4)]
    assert b.take_many("x", 4) == singles and b.take_many("x", 0) == []
    assert a.free_count == b.free_count == 5
    with pytest.raises(OutOfPages):
        b.take_many("y", 6)
    assert b.free_count == 5                       # nothing was taken
    for page in singles:
        b.give(page, "x")
    b.check()
