"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders of
requests; groups; windows; slots; errors."""

import numpy as np
import pytest
import torch

from distengine_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagePool
from distengine_b200.parts.base import PagedKVSpec, StateSpec

FULL = PagedKVSpec(2, 16, None)
WIN = PagedKVSpec(2, 16, 24)


def manager(specs=None, reads=None, page=8, pages=16, seqs=4, max_len=256, **kw):
    specs = specs if specs is not None else [FULL, FULL]
    reads = reads if reads is not None else [None] * len(specs)
    return CacheManager(specs, reads, page, pages, seqs, max_len, torch.float32, "cpu", **kw)


def test_page_pool_is_last_in_first_out():
    pool = PagePool(4)
    assert pool.take(2) == [3, 2]                    # popped from the end, like the reference
    pool.give([3])
    assert pool.take(1) == [3]                       # the page just given back is used again first
    with pytest.raises(OutOfPages):
        pool.take(5)
    with pytest.raises(KeyError):
        pool.give([0])                               # never taken
    pool.give([2])
    with pytest.raises(KeyError):
        pool.give([2])                               # freed twice


def test_reserve_commit_release():
    m = manager()
    slot = m.admit("a")
    assert slot == 0 and m.length("a") == 0 and m.pages_needed("a", 9) == 2
    m.reserve([("a", 9)])
    m.commit("a", 9)
    assert m.length("a") == 9 and m.num_free_pages() == 14
    assert m.pages_needed("a", 16) == 0 and m.pages_needed("a", 17) == 1
    table = m.paged[0].tables["a"]
    assert table == [15, 14] and m.paged[0].host_table[0, :3].tolist() == [15, 14, -1]
    m.check_invariants()
    m.release("a")
    assert m.num_free_pages() == 16 and m.paged[0].host_table[0, :3].tolist() == [-1, -1, -1]
    m.check_invariants()
    with pytest.raises(KeyError):
        m.release("a")                               # released twice
    with pytest.raises(KeyError):
        m.length("nobody")


def test_errors_follow_the_reference_classes():
    m = manager(seqs=2)
    m.admit("a")
    with pytest.raises(ValueError):
        m.admit("a")                                 # duplicate
    with pytest.raises(ValueError):
        m.admit("")
    m.admit("b")
    with pytest.raises(OutOfSlots):
        m.admit("c")
    with pytest.raises(ValueError):
        m.reserve([("a", 257)])                      # beyond what the cache was made for
    with pytest.raises(ValueError):
        m.commit("a", -1)


def test_a_tentative_step_is_taken_back_or_confirmed():
    """A step that was launched ahead: taken back, the length is what it was, the pages stay, and
    the same tokens can be reserved and committed again; confirmed, it counts like any other."""
    m = manager()
    m.admit("a")
    m.reserve([("a", 8)])
    m.commit("a", 8)
    m.reserve([("a", 9)])
    m.commit("a", 9, tentative=True)
    free = m.num_free_pages()
    assert m.length("a") == 9
    with pytest.raises(ValueError):
        m.commit("a", 10)                                   # not while a step is undecided
    m.rewind("a")
    assert m.length("a") == 8 and m.num_free_pages() == free
    assert m.pages_needed("a", 9) == 0                      # the page of token 9 is still held
    with pytest.raises(ValueError):
        m.rewind("a")                                       # nothing tentative is left
    m.reserve([("a", 9)])
    m.commit("a", 9, tentative=True)
    m.confirm("a")
    m.confirm("a")                                          # harmless when nothing is pending
    assert m.length("a") == 9
    m.reserve([("a", 10)])
    m.commit("a", 10)
    m.check_invariants()
    m.release("a")
    assert m.num_free_pages() == m.num_pages


@pytest.mark.parametrize("length", range(8, 40))
def test_a_window_keeps_its_pages_until_a_tentative_step_is_confirmed(length):
    """With page 4 and window 6, a step to ``length + 1`` passes a page whenever
    (length - 4) % 4 == 0.  Launched ahead, it must not give that page back: taken back, the token
    at ``length`` is fed again and still reads key ``length - 5``."""
    page, window = 4, 6
    m = manager(specs=[PagedKVSpec(2, 16, window)], page=page, pages=16)
    m.admit("a")
    m.reserve([("a", length)])
    m.commit("a", length)
    first_key = max(0, length - window + 1)
    m.reserve([("a", length + 1)])
    m.commit("a", length + 1, tentative=True)
    table = m.paged[0].tables["a"]
    assert all(table[p] >= 0 for p in range(first_key // page, length // page + 1))
    m.rewind("a")
    assert m.pages_needed("a", length + 1) == 0
    m.reserve([("a", length + 1)])
    assert all(table[p] >= 0 for p in range(first_key // page, length // page + 1))
    m.commit("a", length + 1, tentative=True)
    m.confirm("a")
    lo = max(0, length + 1 - window + 1) // page             # now the passed pages are back
    assert all(p < 0 for p in table[:lo]) and all(p >= 0 for p in table[lo:])
    m.check_invariants()
    m.release("a")
    assert m.num_free_pages() == m.num_pages


def test_a_window_page_that_is_gone_is_seen_as_missing():
    """The quick answer of ``pages_needed`` (the new positions lie in a held page) must not hide a
    window's first page that is not held."""
    m = manager(specs=[PagedKVSpec(2, 16, 6)], page=4, pages=16)
    m.admit("a")
    m.reserve([("a", 13)])
    m.commit("a", 13)                                   # keys from 8 on are needed: page 2 on
    group = m.paged[0]
    table = group.tables["a"]
    lost = table[2]
    m._give(group, [lost])                              # as if a commit had gone one step too far
    table[2] = -1
    group.host_table[m.slot("a"), 2] = -1
    assert m.pages_needed("a", 14) == 1


def test_state_rows_come_back_when_a_tentative_step_is_taken_back():
    m = manager(specs=[FULL, StateSpec((3,))])
    state = m.bindings()[1].state
    a, b = m.admit("a"), m.admit("b")
    state[a], state[b] = 1.0, 2.0
    m.reserve([("a", 1), ("b", 1)])
    m.save_states(["a", "b"])
    state[a] += 10.0                                    # what the step launched ahead does
    state[b] += 10.0
    m.commit("a", 1, tentative=True)
    m.commit("b", 1, tentative=True)
    m.release("b")                                      # b ended meanwhile
    m.rewind("a")
    assert torch.all(state[a] == 1.0) and m.length("a") == 0
    m.reserve([("a", 1)])
    m.save_states(["a"])
    state[a] += 5.0
    m.commit("a", 1, tentative=True)
    m.confirm("a")
    assert torch.all(state[a] == 6.0) and m.length("a") == 1


def test_reserve_is_all_or_nothing():
    m = manager(pages=4)
    m.admit("a"), m.admit("b")
    m.reserve([("a", 16)])
    m.commit("a", 16)
    with pytest.raises(OutOfPages):
        m.reserve([("a", 24), ("b", 16)])            # needs 1 + 2, 2 are free
    assert m.num_free_pages() == 2 and m.paged[0].tables["b"] == []
    m.check_invariants()
    m.reserve([("a", 24), ("b", 8)])
    assert m.num_free_pages() == 0
    m.check_invariants()


def test_groups_have_pools_of_their_own_and_window_pages_come_back():
    m = manager(specs=[FULL, WIN, FULL, WIN], page=8, pages=12)
    assert len(m.paged) == 2 and [g.entries for g in m.paged] == [[0, 2], [1, 3]]
    assert m.paged[0].k.shape == (2, 12, 2, 8, 16)
    m.admit("a")
    fed = 0
    for step in (20, 13, 1, 1, 30, 7, 1):
        m.reserve([("a", fed + step)])
        fed += step
        m.commit("a", fed)
        m.check_invariants()
        full, win = m.paged[0].tables["a"], m.paged[1].tables["a"]
        assert all(p >= 0 for p in full) and len(full) == (fed + 7) // 8
        first_needed = max(0, fed - 24 + 1) // 8
        assert all(p < 0 for p in win[:first_needed]) and all(p >= 0 for p in win[first_needed:])
    # the window group holds at most window/page + 2 pages however long the request grows
    assert sum(p >= 0 for p in m.paged[1].tables["a"]) <= 24 // 8 + 2
    assert m.paged[1].pool.num_free > m.paged[0].pool.num_free
    m.release("a")
    assert all(g.pool.num_free == 12 for g in m.paged)
    m.check_invariants()


def test_bindings_share_and_state_slots():
    specs = [FULL, None, StateSpec((3, 5)), None]
    m = manager(specs=specs, reads=[None, 0, None, None])
    b = m.bindings()
    assert b[0].kind == "paged" and b[0].writes and b[1].kind == "paged" and not b[1].writes
    assert b[1].k_pages.data_ptr() == b[0].k_pages.data_ptr()
    assert b[2].kind == "state" and b[2].state.shape == (4, 3, 5) and b[3] is None
    slot = m.admit("a")
    b[2].state[slot] = 7.0
    m.release("a")
    assert m.admit("b") == slot                       # the slot is used again ...
    assert torch.all(b[2].state[slot] == 0)           # ... and its state starts at zero


def test_freed_pages_can_be_poisoned():
    m = manager(poison_freed_pages=True, pages=4)
    assert torch.isnan(m.paged[0].k).all()
    m.admit("a")
    m.reserve([("a", 8)])
    page = m.paged[0].tables["a"][0]
    m.paged[0].k[:, page] = 1.0
    m.commit("a", 8)
    m.release("a")
    assert torch.isnan(m.paged[0].k[:, page]).all()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    rng = np.random.default_rng(seed)
    specs = [FULL, WIN, FULL] if seed % 2 else [FULL, FULL]
    m = manager(specs=specs, page=4 if seed % 3 else 16, pages=40, seqs=5, max_len=400)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            rid = f"r{counter}"
            counter += 1
            m.admit(rid)
            live[rid] = 0
        elif action < 0.85 and live:
            picked = [r for r in live if rng.random() < 0.6] or [next(iter(live))]
            wanted = [(r, live[r] + int(rng.choice([1, 1, 1, 2, 5, 17, 40]))) for r in picked]
            wanted = [(r, n) for r, n in wanted if n <= 400]
            before = [g.pool.num_free for g in m.paged]
            try:
                m.reserve(wanted)
            except OutOfPages:
                assert [g.pool.num_free for g in m.paged] == before      # nothing was taken
                victim = max(live, key=live.get)
                m.release(victim)
                del live[victim]
            else:
                ahead = rng.random() < 0.3               # a step launched ahead of the host
                for r, n in wanted:
                    m.commit(r, n, tentative=ahead)
                if ahead and rng.random() < 0.5:
                    for r, _ in wanted:
                        m.rewind(r)
                else:
                    for r, n in wanted:
                        m.confirm(r)
                        live[r] = n
        elif live:
            rid = list(live)[int(rng.integers(len(live)))]
            m.release(rid)
            del live[rid]
        m.check_invariants()
        for g in m.paged:
            for rid, n in live.items():
                table = g.tables[rid]
                lo = 0 if g.spec.window is None else max(0, n - g.spec.window + 1) // m.page_size
                assert all(table[p] >= 0 for p in range(lo, (n + m.page_size - 1) // m.page_size))
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert all(g.pool.num_free == 40 for g in m.paged) and m.slots.num_free == 5
