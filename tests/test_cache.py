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


def test_native_decode_metadata_rows_follow_their_holdings():
    """The native writer of a decode step's metadata: the vectors are right every step, and a
    block-table row is rewritten exactly when it has to be: when it grew, when another holding
    took the row (also one with the same request id, after a close), and when a window gave
    pages back; otherwise the call reports that no row was touched."""
    import numpy as np
    from rllm_b200.engine.step import MetaLayout
    m = manager([FULL, WIN], pages=16, page=4, reqs=4)
    L, P, S, G = m._L, 8, 2, 2
    lay = MetaLayout(S, S, P, S, G)
    host = np.full(lay.total, -7, dtype=np.int32)
    rows = L.rows_new(S, G)
    handles, tokens = np.zeros(S, dtype=np.int32), np.zeros(S, dtype=np.int32)

    def fill(rcs, toks):
        handles[:] = [rc.handle for rc in rcs]
        tokens[:] = toks
        return L.fill_decode(m._ptr, rows, S, handles.ctypes.data, tokens.ctypes.data, P, host.ctypes.data,
                             lay.offs.ctypes.data)

    def table(g):
        return lay.view(host, 8 + 2 * g, S * P).reshape(S, P)

    def expect(rcs):
        for s, rc in enumerate(rcs):
            n = rc.num_tokens
            assert lay.view(host, 1, S)[s] == n and lay.view(host, 4, S)[s] == n + 1
            assert lay.view(host, 5, S)[s] == rc.state_slot
            for g in range(G):
                pages = rc.pages[g]
                assert list(table(g)[s, : len(pages)]) == pages and all(table(g)[s, len(pages):] == -1)
                assert lay.view(host, 7 + 2 * g, S)[s] == pages[n // 4] * 4 + n % 4

    a, b = m.open("a"), m.open("b")
    for rc, n in ((a, 6), (b, 3)):
        m.reserve(rc, n); m.commit(rc, n)
    for rc in (a, b):
        m.reserve(rc, rc.num_tokens + 1)
    assert fill([a, b], [11, 12]) == 1 and list(lay.view(host, 0, S)) == [11, 12]
    expect([a, b])
    for rc in (a, b):
        m.commit(rc, rc.num_tokens + 1)
    # next token: b crosses a page edge (4), a does not (7): the row of b grows, a's stays
    for rc in (a, b):
        m.reserve(rc, rc.num_tokens + 1)
    assert fill([a, b], [13, 14]) == 1
    expect([a, b])
    m.commit(a, 8); m.commit(b, 5)
    m.reserve(a, 9); m.reserve(b, 6)
    assert fill([a, b], [1, 2]) == 1          # a crossed to its third page
    expect([a, b])
    m.commit(a, 9); m.commit(b, 6)
    m.reserve(a, 10); m.reserve(b, 7)
    assert fill([a, b], [3, 4]) == 0          # nobody grew, nobody changed: no row touched
    expect([a, b])
    # the window (10 keys) passes a's first page: its epoch moves, its rows are rewritten with -1 in front
    for n in range(10, 15):
        m.commit(a, n); m.reserve(a, n + 1)
    assert a.pages[1][0] == -1 and fill([a, b], [5, 6]) == 1
    expect([a, b])
    # b ends; a request with the same id takes the same row and slot: the row is written afresh
    m.close("b")
    b2 = m.open("b")
    m.reserve(b2, 2); m.commit(b2, 1)
    assert fill([a, b2], [7, 8]) == 1
    expect([a, b2])
    # a token without a page is refused, not written past the table
    m.reserve(b2, 4); m.commit(b2, 4)         # its one page is full and no page is reserved for position 4
    assert fill([a, b2], [9, 9]) < 0
    L.rows_delete(rows)
    m.check()


def test_a_step_that_fails_leaves_every_request_as_it_was():
    """Whatever is raised while a step's batch runs (a refused size, a failed launch), nothing is
    committed: reserved pages go back, and a request that the step opened is closed again."""
    from rllm_b200.engine.step import Engine, Entry

    class Backend:
        device, fast = torch.device("cpu"), False

    class Model:
        vocab_size = 50

        def parts(self):
            return []

    m = manager(pages=6, page=4, reqs=3)
    eng = Engine(Model(), Backend(), m, use_graphs=False)
    old = m.open("old")
    m.reserve(old, 5)
    m.commit(old, 5)
    free, slots = m.free_pages(), m.slots.num_free

    def boom(entries, rcs):
        assert m.free_pages() != free            # the step had reserved its pages by then
        raise RuntimeError("a kernel refused the size")

    eng.build_context = boom
    with pytest.raises(RuntimeError, match="refused"):
        eng.step([Entry("old", [1, 2, 3, 4], [3]), Entry("new", [5, 6, 7, 8, 9], [])])
    assert m.free_pages() == free and m.slots.num_free == slots
    assert "new" not in m.live and old.num_tokens == 5
    m.check()
    with pytest.raises(OutOfPages):              # and the all-or-nothing rule as before
        eng.step([Entry("old", [1] * 4, []), Entry("big", [2] * 40, [])])
    assert m.free_pages() == free and "big" not in m.live
    m.check()


def test_a_cache_kind_registered_from_outside_and_pools_of_different_size():
    """The manager serves a spec class it has never heard of once a kind is registered for it: here
    a paged kind with one tensor per page and a pool three pages larger than the others'. Its pages
    go through the same tables and checks. A spec class with no kind is refused by name."""
    from dataclasses import dataclass
    from rllm_b200.parts import CacheKind, register_cache_kind

    @dataclass(frozen=True)
    class JointSpec:
        width: int

    @dataclass(frozen=True)
    class Unknown:
        x: int = 0

    register_cache_kind(JointSpec, CacheKind(
        paged=True,
        allocate=lambda spec, pages, page, dtype, device: {"kv": torch.zeros(pages, page, spec.width, dtype=dtype, device=device)},
        num_pages=lambda spec, default: default + 3,
        page_bytes=lambda spec, page, dtype: page * spec.width * 4))
    m = manager([FULL, JointSpec(6), FULL, JointSpec(6), JointSpec(10)], pages=8, page=4, allocate=True)
    assert [g.layers for g in m.groups] == [[0, 2], [1, 3], [4]]
    assert [g.pool.num_pages for g in m.groups] == [8, 11, 11] and m.free_pages() == [8, 11, 11]
    assert m.groups[1].tensors[3]["kv"].shape == (11, 4, 6) and m.groups[2].tensors[4]["kv"].shape == (11, 4, 10)
    assert CacheManager.bytes_per_page([FULL, JointSpec(6), None], 4, torch.float32) == 2 * 2 * 16 * 4 * 4 + 4 * 6 * 4
    a = m.open("a")
    m.reserve(a, 30)                         # 8 pages in every group: the small pool is empty then
    m.commit(a, 30)
    assert m.free_pages() == [0, 3, 3]
    b = m.open("b")
    with pytest.raises(OutOfPages):
        m.reserve(b, 1)
    m.check()
    m.close("a"); m.close("b")
    assert m.free_pages() == [8, 11, 11]
    m2 = CacheManager([FULL, JointSpec(6)], 4, {FULL: 5, JointSpec(6): 9}, 2, torch.float32, "cpu", allocate=False)
    assert [g.pool.num_pages for g in m2.groups] == [5, 9]
    with pytest.raises(TypeError, match="Unknown"):
        manager([FULL, Unknown()])
