"""The cache manager on the host: pages, block tables, windows, slots.  No page is
lost, held twice or freed twice, under random orders of requests."""
import random

import pytest
import torch

from inferflux_b200.cache import CacheManager, OutOfPages, OutOfSlots, PageAccountingError, PageAllocator
from inferflux_b200.config import ScheduleEntry
from inferflux_b200.parts import KVCacheSpec, StateSpec


def manager(num_pages=16, page=4, max_seqs=4, window=None, state=False, max_len=256):
    full = (KVCacheSpec(2, 8, None), None)
    specs = [full, full]
    if window:
        specs += [(KVCacheSpec(2, 8, window), StateSpec((3,), torch.float32) if state else None)]
    return CacheManager(specs, page_size=page, num_pages=num_pages, max_seqs=max_seqs, max_seq_len=max_len,
                        dtype=torch.float32, device="cpu")


def test_allocator_refuses_double_free_and_foreign_free():
    a = PageAllocator(4)
    p = a.allocate(3, "x")
    assert p == [0, 1, 2] and a.num_free == 1
    with pytest.raises(OutOfPages):
        a.allocate(2, "y")
    assert a.num_free == 1                                   # nothing taken by the failed call
    with pytest.raises(PageAccountingError, match="belongs to"):
        a.release([0], "y")
    a.release([1], "x")
    with pytest.raises(PageAccountingError, match="freed twice"):
        a.release([1], "x")
    with pytest.raises(PageAccountingError, match="named twice"):
        a.release([0, 0], "x")
    with pytest.raises(PageAccountingError, match="outside"):
        a.release([9], "x")
    assert a.allocate(1, "z") == [1]                         # the page freed last is used again first
    a.check()


def test_groups_by_need_and_block_tables():
    m = manager(window=6)
    assert len(m.groups) == 2 and m.groups[0].spec.window is None and m.groups[1].spec.window == 6
    assert m.groups[0].pool.shape == (2, 16, 2, 2, 4, 8) and m.groups[1].pool.shape == (1, 16, 2, 2, 4, 8)
    v0, v2 = m.view(ScheduleEntry(0, 0)), m.view(ScheduleEntry(2, 2))
    assert v0.kv.data_ptr() == m.groups[0].pool[0].data_ptr() and v2.group == 1
    slot = m.add_request("a")
    m.reserve("a", 10)
    ups = m.drain_table_updates()
    assert [len(u) for u in ups] == [3, 3]                   # 10 tokens of 4-token pages, in both groups
    assert all(idx // m.max_blocks == slot for idx, _p in ups[0])
    m.commit("a", 10)
    # the window (6) has moved past block 0 (positions 0..3): next query is 10, needs keys >= 5
    assert sorted(m.pages_of("a", 1)) == [1, 2] and sorted(m.pages_of("a", 0)) == [0, 1, 2]
    m.reserve("a", 11); m.commit("a", 11)
    m.reserve("a", 13); m.commit("a", 13)                     # needs keys >= 8: block 1 goes too
    assert sorted(m.pages_of("a", 1)) == [2, 3]
    assert m.groups[1].alloc.num_free == 14 and m.groups[0].alloc.num_free == 12
    m.check()
    m.free("a")
    assert m.free_pages() == [16, 16] and m.num_free_slots == 4
    with pytest.raises(KeyError):
        m.free("a")


def test_reserve_is_all_or_nothing_across_groups():
    m = manager(num_pages=5, window=6)
    m.add_request("a"); m.add_request("b")
    m.reserve("a", 12); m.commit("a", 12)                    # 3 pages in the full group, window group keeps 2
    with pytest.raises(OutOfPages):
        m.reserve("b", 12)                                   # the full group has 2 free: nothing is taken
    assert m.free_pages() == [2, 3] and not m.pages_of("b", 0) and not m.pages_of("b", 1)
    assert m.can_reserve("b", 8) and not m.can_reserve("b", 9)
    m.check()


def test_slots_state_and_stale_generations():
    m = manager(max_seqs=2, window=6, state=True)
    s0 = m.add_request("a")
    gen = m.generation("a")
    m.state[2][s0] += 5.0
    m.add_request("b")
    with pytest.raises(OutOfSlots):
        m.add_request("c")
    m.free("a")
    s1 = m.add_request("c")
    assert s1 == s0 and float(m.state[2][s1].abs().sum()) == 0.0   # the slot's state starts at zero again
    with pytest.raises(PageAccountingError, match="stale"):
        m.free("c", generation=gen)                          # a handle from the slot's previous holder
    m.free("c", generation=m.generation("c"))
    with pytest.raises(KeyError):
        m.add_request("b")
    m.check()


def test_limits():
    m = manager(max_len=20)
    m.add_request("a")
    with pytest.raises(OutOfPages, match="longest"):
        m.reserve("a", 21)
    m.reserve("a", 20); m.commit("a", 20)
    with pytest.raises(ValueError):
        m.reserve("a", 10)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = manager(num_pages=24, page=4, max_seqs=5, window=rng.choice([3, 7, 16]))
    live, n_id, reused = {}, 0, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.num_free_slots:
            rid = f"r{n_id}"; n_id += 1
            m.add_request(rid); live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            new = live[rid] + rng.choice([1, 1, 1, 2, 5, 9, 17])
            if new > m.max_seq_len:
                continue
            if m.can_reserve(rid, new):
                m.reserve(rid, new); m.commit(rid, new); live[rid] = new
            else:
                before = m.free_pages()
                with pytest.raises(OutOfPages):
                    m.reserve(rid, new)
                assert m.free_pages() == before
        elif live:
            rid = rng.choice(list(live))
            m.free(rid); del live[rid]
        m.check()
        for rid, n in live.items():
            held = m.pages_of(rid, 0)
            assert sorted(held) == list(range(-(-n // 4))), "a full-attention request lost a block"
            w = m.groups[1].spec.window
            need_from = max(0, n - w + 1) // 4
            assert sorted(m.pages_of(rid, 1)) == list(range(need_from, -(-n // 4))) or n == 0
    for rid in list(live):
        m.free(rid)
    m.check()
    assert m.free_pages() == [24, 24] and m.num_free_slots == 5
    assert m.groups[0].alloc.allocations > 24, "pages were never used again"


def test_a_failed_step_gives_back_what_it_reserved():
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.parts import KVCacheSpec
    import torch
    cm = CacheManager([(KVCacheSpec(1, 8, None), None), (KVCacheSpec(1, 8, 6), None)], page_size=4, num_pages=10,
                      max_seqs=2, max_seq_len=64, dtype=torch.float32, device="cpu")
    cm.add_request("a")
    cm.reserve("a", 9)
    cm.commit("a", 9)
    cm.drain_table_updates()
    free = cm.free_pages()
    held = cm.pages_of("a", 0)
    cm.reserve("a", 22)                                    # the step takes pages ...
    assert cm.free_pages() != free
    cm.release_uncommitted("a")                            # ... and fails before commit
    assert cm.free_pages() == free and cm.pages_of("a", 0) == held and cm.length("a") == 9
    assert all(not ups for ups in cm.drain_table_updates())
    cm.check()
    cm.reserve("a", 13)                                    # and goes on as if nothing had happened
    cm.commit("a", 13)
    cm.check()
    cm.free("a")
    assert cm.free_pages() == [10, 10]
