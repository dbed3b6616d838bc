"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice, under
random orders of requests; window groups give pages back as the window passes them."""
import random

import pytest

from tinyserve_b200.cache import CacheError, CacheManager, GroupSpec


def full(pages=9, page=4, slots=4):
    return CacheManager([GroupSpec("full")], pages, page, slots)


def test_allocate_is_all_or_nothing_and_frees_on_end():
    m = full(pages=5)            # 4 usable pages of 4 tokens
    m.begin("a")
    assert m.allocate("a", 9)    # 3 pages
    assert m.num_free_pages() == 1
    m.begin("b")
    assert not m.allocate("b", 5)          # needs 2, only 1 free: nothing taken
    assert m.num_free_pages() == 1 and m.block_table("b", 0) == []
    assert m.allocate("b", 4)
    m.commit("a", 9)
    assert m.num_computed("a") == 9 and not m.is_fresh("a")
    assert m.allocate("a", 3)              # 12 tokens still fit in 3 pages
    assert not m.allocate("a", 4)          # a 4th page is not there
    m.free("b")
    assert m.allocate("a", 4)
    m.check_invariants()
    m.free("a")
    assert m.num_free_pages() == 4
    m.check_invariants()


def test_null_page_and_reuse_order():
    m = full(pages=6)
    m.begin("a"); m.allocate("a", 8)
    m.begin("b"); m.allocate("b", 4)
    first = list(m.block_table("a", 0)) + list(m.block_table("b", 0))
    assert 0 not in first and len(set(first)) == 3
    m.free("a")
    m.begin("c"); m.allocate("c", 16)      # takes the 2 never-used pages first, then a's
    pages = m.block_table("c", 0)
    assert set(pages[2:]) == set(first[:2]), "freed pages are handed out again"
    assert 0 not in pages
    m.check_invariants()


def test_errors():
    m = full(slots=1)
    m.begin("a")
    with pytest.raises(CacheError):
        m.begin("a")
    with pytest.raises(CacheError):
        m.begin("b")                       # no slot
    m.free("a")
    with pytest.raises(CacheError):
        m.free("a")                        # freed twice
    m.begin("b")
    m.allocate("b", 4)
    with pytest.raises(CacheError):
        m.commit("b", 5)                   # ran past its pages
    with pytest.raises(CacheError):
        m.pools[0].give_back(0, "b")
    with pytest.raises(CacheError):
        CacheManager([GroupSpec("full")], 1, 4, 1)
    with pytest.raises(CacheError):
        CacheManager([GroupSpec("full")], 4, 6, 1)


def test_slots_are_unique_and_come_back():
    m = full(pages=20, slots=3)
    slots = [m.begin(r) for r in "abc"]
    assert sorted(slots) == [0, 1, 2] and not m.can_begin()
    m.free("b")
    assert m.can_begin() and m.begin("d") == slots[1]
    m.check_invariants()


def test_window_group_gives_pages_back():
    page, window = 4, 6
    m = CacheManager([GroupSpec("full"), GroupSpec("window", window)], [40, 6], page, 2)
    m.begin("a")
    total = 0
    for n in (5, 3, 9, 1, 1, 1, 7, 2):
        assert m.allocate("a", n), (total, n)
        # every key that a query of this portion can see is on a live page
        for q in range(total, total + n):
            for j in range(max(0, q - window + 1), q + 1):
                assert m.block_table("a", 1)[j // page] != 0
                m.slot_of_position("a", 1, j)
        m.commit("a", n)
        total += n
        table = m.block_table("a", 1)
        live = [i for i, p in enumerate(table) if p]
        lowest_visible = max(0, total - window + 1)
        assert live and live[0] == lowest_visible // page, "pages behind the window are given back"
        assert all(p == 0 for p in table[:live[0]])
        assert len(m.block_table("a", 0)) == len(table) and 0 not in m.block_table("a", 0)
        m.check_invariants()
    # 29 tokens would need 8 pages of 4; the window pool has 5 usable
    assert total == 29 and m.pools[1].num_usable == 5
    with pytest.raises(CacheError):
        m.slot_of_position("a", 1, 0)
    m.free("a")
    m.check_invariants()
    assert m.num_free_pages(1) == 5 and m.num_free_pages(0) == 39


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    groups = [GroupSpec("full"), GroupSpec("window", rng.choice([3, 8, 17]))]
    m = CacheManager(groups, [rng.randint(6, 30), rng.randint(6, 30)], page, 5)
    live, counter = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.can_begin():
            rid = f"r{counter}"; counter += 1
            m.begin(rid); live[rid] = 0
        elif op < 0.85 and live:
            rid = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 5, 13])
            before = [p.num_free for p in m.pools]
            tables = [list(m.block_table(rid, g)) for g in range(2)]
            if m.allocate(rid, n):
                m.commit(rid, n); live[rid] += n
                assert m.num_computed(rid) == live[rid]
            else:
                # nothing is taken when it does not fit (a window may still have let go of pages)
                assert [p.num_free for p in m.pools] >= before
                assert [len(m.block_table(rid, g)) for g in range(2)] == [len(t) for t in tables]
        elif live:
            rid = rng.choice(sorted(live))
            m.free(rid); del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.free(rid)
    m.check_invariants()
    assert all(p.num_free == p.num_usable for p in m.pools)


def test_block_table_changes_travel_once_and_again_if_not_acknowledged():
    """The device keeps every request's block-table row; the manager says what that copy lacks."""
    m = CacheManager([GroupSpec("full"), GroupSpec("window", 8)], 32, 4, 4)
    m.begin("a")
    assert m.allocate("a", 10)                          # three pages in both groups
    changes, receipt = m.table_updates("a", 0)
    assert [i for i, _ in changes] == [0, 1, 2] and [p for _, p in changes] == m.block_table("a", 0)
    again, _ = m.table_updates("a", 0)
    assert again == changes, "a packed step that is never launched sends its entries again"
    m.table_synced(receipt)
    assert m.table_updates("a", 0)[0] == []
    m.commit("a", 10)
    assert m.allocate("a", 3)                           # one more page
    changes, receipt = m.table_updates("a", 0)
    assert changes == [(3, m.block_table("a", 0)[3])]
    m.table_synced(receipt)
    # the window group gives pages back behind the window: those entries travel as zeros
    w_changes, w_receipt = m.table_updates("a", 1)
    m.table_synced(w_receipt)
    m.commit("a", 3)                                    # 13 computed: keys below 13 - 8 + 1 = 6 are gone: page 0
    released, receipt = m.table_updates("a", 1)
    assert (0, 0) in released and m.block_table("a", 1)[0] == 0
    m.table_synced(receipt)
    assert m.table_updates("a", 1)[0] == []
    m.free("a")
    m.check_invariants()
