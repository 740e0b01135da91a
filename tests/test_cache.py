"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random orders of requests."""
import random

import numpy as np
import pytest

from liyab_b200 import ErrorCode, LiyabError
from liyab_b200.cache import UNMAPPED, CacheManager, KvNeed, OutOfPages, StateNeed


def manager(num_pages=16, page_size=4, window_units=(), max_requests=4, state=False):
    needs = {u: KvNeed(2, 16, 8 if u in window_units else 0) for u in range(4)}
    states = {1: StateNeed((3, 5))} if state else {}
    return CacheManager(needs, states, page_size, num_pages, max_requests)


def test_pool_hands_out_every_page_once_and_reuses_freed_ones():
    m = CacheManager({0: KvNeed(1, 16, 0)}, {}, page_size=4, num_pages=3, max_requests=3)
    for r in "abc":
        m.open(r)
        m.reserve(r, 4); m.commit(r, 4)
    pages = [int(m.block_table(0, [r])[0, 0]) for r in "abc"]
    assert sorted(pages) == [0, 1, 2] and m.free_pages() == {0: 0}
    with pytest.raises(OutOfPages):
        m.reserve("a", 1)
    m.close("b")
    with pytest.raises(LiyabError):
        m.close("b")                 # a second close cannot free its pages twice
    m.open("d")
    m.reserve("d", 1)
    assert int(m.block_table(0, ["d"])[0, 0]) == pages[1]          # most recently freed first: pages are used again
    m.check()


def test_groups_by_need_and_tables_per_group():
    m = manager(window_units=(1, 3))
    assert len(m.groups) == 2
    assert m.groups[m.group_of_unit[0]]["units"] == [0, 2] and m.groups[m.group_of_unit[1]]["units"] == [1, 3]
    m.open("a")
    m.reserve("a", 10)
    m.commit("a", 10)
    full, win = m.group_of_unit[0], m.group_of_unit[1]
    assert (m.block_table(full, ["a"]) >= 0).sum() == 3 and (m.block_table(win, ["a"]) >= 0).sum() == 3
    m.reserve("a", 7)
    m.commit("a", 7)              # 17 tokens: window 8 sees positions >= 10, so pages 0 and 1 are dead
    t = m.block_table(win, ["a"])[0]
    assert list(t[:2]) == [UNMAPPED, UNMAPPED] and (t[2:] >= 0).all()
    assert (m.block_table(full, ["a"]) >= 0).sum() == 5
    assert m.pages_in_use() == {full: 5, win: 3}
    m.check()
    m.close("a")
    assert m.pages_in_use() == {full: 0, win: 0}


def test_reservation_is_all_or_nothing_across_groups():
    m = CacheManager({0: KvNeed(1, 16, 0), 1: KvNeed(1, 32, 0)}, {}, 4, 4, 4, pages_per_group={KvNeed(1, 32, 0): 2})
    m.open("a")
    m.reserve("a", 8)
    m.commit("a", 8)
    before = m.free_pages()
    with pytest.raises(OutOfPages) as e:
        m.reserve("a", 4)         # group 0 has room, group 1 has not: nothing may be taken
    assert e.value.code == ErrorCode.OUT_OF_MEMORY
    assert m.free_pages() == before and m.length("a") == 8
    m.check()


def test_slot_mapping_and_block_table():
    m = manager()
    m.open("a"); m.open("b")
    m.reserve("a", 6); m.commit("a", 6)
    m.reserve("b", 3); m.commit("b", 3)
    m.reserve("a", 5)
    ta = m.block_table(0, ["a", "b"])
    assert ta.shape == (2, 3) and ta[1, 1] == UNMAPPED
    slots = m.slot_mapping(0, "a", 6, 5)
    assert list(slots) == [ta[0, 1] * 4 + 2, ta[0, 1] * 4 + 3, ta[0, 2] * 4, ta[0, 2] * 4 + 1, ta[0, 2] * 4 + 2]
    assert m.block_table(0, ["a"], width=8).shape == (1, 8)


def test_truncate_gives_pages_back():
    m = manager()
    m.open("a")
    m.reserve("a", 13); m.commit("a", 13)
    assert m.pages_in_use()[0] == 4
    m.truncate("a", 5)
    assert m.pages_in_use()[0] == 2 and m.length("a") == 5
    m.reserve("a", 4); m.commit("a", 4)
    assert m.length("a") == 9
    m.check()


def test_requests_limits_and_state_slots():
    m = manager(max_requests=2, state=True)
    m.open("a"); m.open("b")
    assert {m.state_slot("a"), m.state_slot("b")} == {0, 1}
    with pytest.raises(LiyabError) as e:
        m.open("c")
    assert e.value.code == ErrorCode.BUSY
    with pytest.raises(LiyabError):
        m.open("a")
    m.close("a")
    m.open("c")
    assert m.state_slot("c") in (0, 1) and m.state_slot("c") != m.state_slot("b")
    with pytest.raises(LiyabError):
        m.close("zzz")
    m.reserve("c", 2); m.commit("c", 2)
    with pytest.raises(LiyabError):          # state cannot be rolled back
        m.truncate("c", 1)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = manager(num_pages=12, page_size=4, window_units=(1, 3) if seed % 2 else (), max_requests=5)
    live, next_id = {}, 0
    for _ in range(400):
        op = rng.random()
        if (op < 0.25 and len(live) < 5) or not live:
            rid = f"r{next_id}"; next_id += 1
            m.open(rid); live[rid] = 0
        elif op < 0.8:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 16])
            if m.can_reserve({rid: n}):
                m.reserve(rid, n); m.commit(rid, n); live[rid] += n
                assert m.length(rid) == live[rid]
            else:
                before = m.free_pages()
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
                assert m.free_pages() == before
        elif op < 0.9 and not m.groups[-1]["window"]:
            rid = rng.choice(list(live))
            cut = rng.randint(0, live[rid])
            m.truncate(rid, cut); live[rid] = cut
        else:
            rid = rng.choice(list(live))
            m.close(rid); del live[rid]
        m.check()
        for gi, g in enumerate(m.groups):      # every page a request can still see is mapped
            for rid, n in live.items():
                t = m.table_of(gi, rid)
                first = 0 if not g["window"] else max(0, n - g["window"] + 1) // m.page_size
                assert len(t) >= (n + m.page_size - 1) // m.page_size or n == 0
                assert all(p != UNMAPPED for p in t[first:(n + m.page_size - 1) // m.page_size])
    for rid in list(live):
        m.close(rid)
    m.check()
    assert all(v == 0 for v in m.pages_in_use().values())
