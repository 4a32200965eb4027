"""The host-side cache manager: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots."""

import random

import pytest

from qwen3_runtime_b200.cache import FREED, CacheError, CacheManager, GroupSpec, PageAllocator
from qwen3_runtime_b200.cache.layout import CacheLayout, KVLayerSpec, StateLayerSpec


def test_span_allocation_grows_tables_in_place():
    m = CacheManager([GroupSpec("full")], page_size=4, num_pages=8, num_slots=2)
    a = m.open("a")
    m.reserve(a, 3)
    assert a.tables == [[0]]
    m.commit(a, 3)
    m.reserve(a, 1)  # still inside page 0
    assert a.tables == [[0]]
    m.commit(a, 1)
    m.reserve(a, 1)  # crosses into a second page
    assert a.tables == [[0, 1]]
    m.commit(a, 1)
    assert a.num_computed == 5 and m.num_free_pages == [6]
    m.close(a)
    assert m.num_free_pages == [8]
    m.check_invariants()


def test_new_pages_needed_says_what_reserve_will_take():
    """What the engine asks before it runs ahead: the pages a span would take from each pool."""
    m = CacheManager([GroupSpec("full"), GroupSpec("window", window=6)], page_size=4, num_pages=[8, 8], num_slots=2)
    a = m.open("a")
    assert m.new_pages_needed(a, 1) == [1, 1] and m.new_pages_needed(a, 9) == [3, 3]
    for _ in range(14):
        need = m.new_pages_needed(a, 1)
        free = m.num_free_pages
        m.reserve(a, 1)
        after = m.num_free_pages
        assert [f - g for f, g in zip(free, after)] == need, "exactly what reserve took"
        m.commit(a, 1)  # a window gives pages back here, never in reserve
    assert m.new_pages_needed(a, 0) == [0, 0]
    m.close(a)
    m.check_invariants()


def test_fifo_reuse_and_capacity_queries():
    m = CacheManager([GroupSpec("full")], page_size=4, num_pages=4, num_slots=4)
    a, b = m.open("a"), m.open("b")
    m.reserve(a, 8)
    m.commit(a, 8)
    assert m.max_reservable(b, 100) == 8 and m.can_reserve(b, 8) and not m.can_reserve(b, 9)
    assert m.max_reservable(a, 100) == 8  # two held pages are full, two free ones remain
    m.close(a)
    m.reserve(b, 16)
    assert b.tables == [[2, 3, 0, 1]]  # freed pages go to the back of the queue
    with pytest.raises(CacheError, match="exhausted"):
        m.reserve(m.open("c"), 1)
    assert m.fits_at_all(16) and not m.fits_at_all(17)


def test_misuse_is_reported():
    m = CacheManager([GroupSpec("full")], 4, 4, 1)
    a = m.open("a")
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    with pytest.raises(CacheError, match="no free state slot"):
        m.open("b")
    m.reserve(a, 4)
    with pytest.raises(CacheError, match="beyond the reserved"):
        m.commit(a, 5)
    m.close(a)
    with pytest.raises(CacheError, match="not open"):
        m.close(a)
    with pytest.raises(CacheError, match="not open"):
        m.reserve(a, 1)
    alloc = PageAllocator(2)
    p = alloc.allocate()
    alloc.release(p)
    with pytest.raises(CacheError, match="not held"):
        alloc.release(p)


def test_window_group_returns_pages_it_has_passed():
    m = CacheManager([GroupSpec("full"), GroupSpec("window", 6)], page_size=4, num_pages=[16, 4], num_slots=2)
    a = m.open("a")
    for _ in range(40):  # decode 40 tokens one at a time: the window group never needs more than 3 pages
        m.reserve(a, 1)
        m.commit(a, 1)
        m.check_invariants()
        live = [p for p in a.tables[1] if p != FREED]
        assert len(live) <= 3
        # the keys the next query reads are all still there
        first_needed = max(0, a.num_computed - 6 + 1)
        assert m.first_live_token(a, 1) <= first_needed
    assert len([p for p in a.tables[0] if p != FREED]) == 10  # the full group keeps everything
    assert a.tables[1][:7] == [FREED] * 7
    m.close(a)
    assert m.num_free_pages == [16, 4]


def test_reset_for_preemption_keeps_slot_and_clears_progress():
    m = CacheManager([GroupSpec("full"), GroupSpec("state")], 4, 8, 2)
    a = m.open("a")
    a.needs_state_reset = False
    m.reserve(a, 9)
    m.commit(a, 9)
    slot = a.slot
    m.reset(a)
    assert a.num_computed == 0 and a.tables == [[]] and a.slot == slot and a.needs_state_reset
    assert m.num_free_pages == [8]


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rnd = random.Random(seed)
    groups = [GroupSpec("full"), GroupSpec("window", rnd.choice([3, 8, 17])), GroupSpec("state")]
    ps = rnd.choice([1, 4, 16])
    m = CacheManager(groups, ps, [rnd.randint(6, 24), rnd.randint(6, 24)], num_slots=4)
    live, next_id = {}, 0
    for _ in range(600):
        action = rnd.random()
        if action < 0.25 and m.slots.num_free:
            live[next_id] = m.open(next_id)
            next_id += 1
        elif action < 0.75 and live:
            rc = rnd.choice(list(live.values()))
            n = m.max_reservable(rc, rnd.randint(1, 3 * ps + 2))
            if n:
                m.reserve(rc, n)
                m.commit(rc, rnd.randint(0, n) if rnd.random() < 0.2 else n)
        elif action < 0.85 and live:
            m.reset(rnd.choice(list(live.values())))
        elif live:
            rid = rnd.choice(list(live))
            m.close(live.pop(rid))
        m.check_invariants()
    for rc in live.values():
        m.close(rc)
    m.check_invariants()
    assert m.num_free_pages == m.num_pages and m.slots.num_free == 4


def test_layout_groups_layers_by_need():
    kv = KVLayerSpec(2, 16)
    layout = CacheLayout({0: kv, 1: KVLayerSpec(2, 16, window=8), 2: kv, 3: StateLayerSpec((5,)), 4: None})
    assert [g.spec.kind for g in layout.groups] == ["full", "window", "state"]
    assert layout.groups[0].cache_ids == (0, 2) and layout.where[2] == (0, 1)
    assert layout.paged_groups == [0, 1]
    assert layout.page_bytes(4, 2) == [2 * 2 * 2 * 16 * 4 * 2, 1 * 2 * 2 * 16 * 4 * 2]
    assert layout.token_bytes(2) == 3 * 2 * 2 * 16 * 2
    equal = 10_000 // sum(layout.page_bytes(4, 2))
    assert layout.pages_for_budget(10_000, 4, 2) == [equal, equal]
    # a window group is capped at what its requests can hold; the rest goes to the full group
    full_b, win_b = layout.page_bytes(4, 2)
    counts = layout.pages_for_budget(100_000, 4, 2, max_num_seqs=2, max_step_tokens=8)
    cap = 2 * (-(-(8 + 8) // 4) + 2)
    assert counts[1] == cap and counts[0] == (100_000 - cap * win_b) // full_b
    assert counts[0] * full_b + counts[1] * win_b <= 100_000 and counts[0] > 100_000 // (full_b + win_b)
