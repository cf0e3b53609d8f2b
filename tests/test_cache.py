"""The cache manager on the CPU: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots."""
import random

import pytest
import torch

from rllm_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from rllm_b200.parts.base import KVCacheSpec, StateSpec

FULL, WIN = KVCacheSpec(2, 16), KVCacheSpec(2, 16, window=10)


def manager(specs=(FULL,), pages=8, page=4, reqs=4, allocate=False):
    return CacheManager(list(specs), page, pages, reqs, torch.float32, "cpu", allocate=allocate)


def test_pool_order_exhaustion_and_reuse():
    p = PagePool(3)
    assert [p.alloc("a") for _ in range(3)] == [0, 1, 2]       # the reference's order
    with pytest.raises(OutOfPages):
        p.alloc("a")
    p.free(1, "a")
    assert p.alloc("b") == 1                                   # given back -> handed out next
    with pytest.raises(CacheError):
        p.free(0, "b")                                         # not the holder
    p.free(0, "a")
    with pytest.raises(CacheError):
        p.free(0, "a")                                         # twice
    with pytest.raises(CacheError):
        p.free(7, "a")
    p.check()


def test_grouping_by_needs():
    m = manager([FULL, WIN, FULL, WIN, StateSpec((("s", (3,), torch.float32),))], allocate=True)
    assert [g.layers for g in m.groups] == [[0, 2], [1, 3]]
    assert m.groups[0].k[2].shape == (8, 2, 4, 16) and list(m.state[4]) == ["s"]
    assert m.state[4]["s"].shape == (4, 3)


def test_reserve_is_all_or_nothing_and_commit_counts():
    m = manager(pages=5)
    a, b = m.open("a"), m.open("b")
    m.reserve(a, 9)                      # 3 pages
    m.commit(a, 9)
    with pytest.raises(OutOfPages):
        m.reserve(b, 12)                 # needs 3, 2 free: nothing is taken
    assert m.free_pages() == [2] and b.pages == [[]]
    m.reserve(b, 8)
    m.commit(b, 5)
    m.trim(b)                            # pages beyond what is stored go back
    assert m.free_pages() == [0] and len(b.pages[0]) == 2
    m.check()
    assert m.slot_of(a, 0, 6) == a.pages[0][1] * 4 + 2
    m.close("a"); m.close("b")
    assert m.free_pages() == [5]
    with pytest.raises(CacheError):
        m.close("a")


def test_window_gives_pages_back_and_they_are_used_again():
    m = manager([FULL, WIN], pages=6)
    a = m.open("a")
    held = []
    for n in range(1, 25):
        m.reserve(a, n)
        m.commit(a, n)
        m.check()
        held.append(sum(p >= 0 for p in a.pages[1]))
    # the next query (position n) sees keys n-9..n: pages wholly below n-9 are back in the pool
    assert max(held) <= 4 and a.pages[1][0] == -1 and a.pages[0][0] >= 0
    assert len(a.pages[0]) == 6 and m.free_pages()[0] == 0
    first_key = 24 - 10 + 1
    assert all((p == -1) == ((i + 1) * 4 <= first_key) for i, p in enumerate(a.pages[1]))
    with pytest.raises(CacheError):
        m.slot_of(a, 1, 3)
    m.close("a")
    assert m.free_pages() == [6, 6]


def test_state_slots_are_zeroed_and_bounded():
    m = manager([StateSpec((("s", (2,), torch.float32),))], reqs=2, allocate=True)
    a = m.open("a")
    slot = a.state_slot
    m.state[0]["s"][slot] = 5.0
    m.close("a")
    b = m.open("b")
    assert b.state_slot == slot                  # the slot given back is handed out next
    assert float(m.state[0]["s"][b.state_slot].abs().sum()) == 0.0
    m.open("c")
    with pytest.raises(OutOfPages):
        m.open("d")
    with pytest.raises(CacheError):
        m.open("b")


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    m = manager([FULL, WIN, FULL], pages=12, page=4, reqs=5)
    live, next_id, reused = {}, 0, set()
    ever = [set(), set()]
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            live[next_id] = m.open(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            rc = live[rid]
            n = rc.num_tokens + rng.choice([1, 1, 1, 2, 5, 9])
            try:
                m.reserve(rc, n)
            except OutOfPages:
                assert all(len(p) == -(-rc.num_tokens // 4) or len(p) >= 0 for p in rc.pages)
                victim = rng.choice(list(live))      # somebody gives way
                m.close(victim)
                del live[victim]
            else:
                for gi in range(2):
                    for p in rc.pages[gi]:
                        if p >= 0 and p in ever[gi] and m.groups[gi].pool.owner(p) == rid:
                            reused.add((gi, p))
                        if p >= 0:
                            ever[gi].add(p)
                m.commit(rc, n - rng.choice([0, 0, 1]) if n - 1 > rc.num_tokens else n)
                m.trim(rc) if rng.random() < 0.3 else None
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.close(rid)
    m.check()
    assert m.free_pages() == [12, 12] and reused
