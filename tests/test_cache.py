"""The cache manager: no page lost, held twice or freed twice, under random orders of requests;
groups with a window give pages back as the window passes; state slots."""

from __future__ import annotations

import random

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from llmserve_triton_kernels_b200.cache import CacheManager, IdAllocator, OutOfPages, num_pages_for_budget
from llmserve_triton_kernels_b200.models.plan import LayerRun
from llmserve_triton_kernels_b200.parts.base import PagedKVSpec, StateSpec


def manager(specs, page_size=4, num_pages=12, max_requests=4, schedule=None):
    schedule = schedule or [LayerRun(i) for i in range(len(specs))]
    return CacheManager(specs, schedule, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                        dtype=torch.float32, device="cpu")


def test_allocator_fifo_reuse_and_double_free():
    a = IdAllocator(4)
    got = [a.allocate() for _ in range(4)]
    assert got == [0, 1, 2, 3]
    with pytest.raises(OutOfPages):
        a.allocate()
    a.free([1, 0])
    assert [a.allocate(), a.allocate()] == [1, 0]  # freed ids go to the tail in the order given
    a.free([2])
    with pytest.raises(ValueError, match="double free"):
        a.free([2])
    with pytest.raises(ValueError):
        a.free([7])
    a.check()


@given(st.lists(st.integers(0, 1), min_size=1, max_size=80), st.integers(0, 2**16))
@settings(max_examples=60, deadline=None)
def test_allocator_invariants_under_random_orders(ops_list, seed):
    rng = random.Random(seed)
    a = IdAllocator(7)
    held = []
    for op in ops_list:
        if op == 0 and a.num_free:
            held.append(a.allocate())
        elif held:
            a.free([held.pop(rng.randrange(len(held)))])
        a.check()
        assert a.num_free + a.num_used == 7 and len(set(held)) == len(held)
    a.free(held)
    assert a.num_free == 7


def test_tables_grow_by_pages_and_everything_comes_back():
    m = manager([PagedKVSpec(2, 8)] * 3)
    assert len(m.groups) == 1 and m.groups[0].pool.shape == (3, 12, 2, 2, 4, 8)
    m.add_request("a")
    with pytest.raises(ValueError, match="already"):
        m.add_request("a")
    m.reserve([("a", 5)])
    assert m.groups[0].tables["a"] == [0, 1] and m.lengths["a"] == 0  # reserved, not yet committed
    m.commit([("a", 5)])
    assert m.lengths["a"] == 5 and m.extra_pages_needed("a", 3) == 0 and m.extra_pages_needed("a", 4) == 1
    m.add_request("b")
    m.reserve([("a", 4), ("b", 1)])
    m.commit([("a", 4), ("b", 1)])
    assert m.num_free_pages == 12 - 3 - 1
    assert abs(m.internal_fragmentation() - (1 - 10 / 16)) < 1e-9
    m.check()
    m.free_request("a")
    m.free_request("b")
    assert m.num_free_pages == 12 and m.utilization() == 0.0
    with pytest.raises(KeyError):
        m.free_request("a")
    m.check()


def test_reserve_is_atomic():
    m = manager([PagedKVSpec(1, 8)], num_pages=4)
    for r in "ab":
        m.add_request(r)
    m.reserve([("a", 8)])
    m.commit([("a", 8)])
    before = (m.num_free_pages, dict(m.lengths), [list(t) for t in m.groups[0].tables.values()])
    with pytest.raises(OutOfPages):
        m.reserve([("a", 4), ("b", 8)])  # needs 1 + 2, only 2 free
    assert before == (m.num_free_pages, dict(m.lengths), [list(t) for t in m.groups[0].tables.values()])
    with pytest.raises(ValueError, match="twice"):
        m.reserve([("a", 1), ("a", 1)])
    m.check()


def test_groups_by_need_and_window_pages_come_back_as_the_window_passes():
    full, windowed = PagedKVSpec(2, 8), PagedKVSpec(2, 8, window=6)
    m = manager([full, windowed, full, windowed], num_pages=16)
    assert [g.spec.window for g in m.groups] == [None, 6] and [g.entries for g in m.groups] == [[0, 2], [1, 3]]
    m.add_request("r")
    fed = 0
    for n in (5, 3, 1, 1, 6, 1):
        m.reserve([("r", n)])
        tables, _ = m.step_tables([("r", n)])
        # every key a new token may see lies on a held page of the windowed group
        wtable = m.groups[1].tables["r"]
        for pos in range(fed, fed + n):
            for key in range(max(0, pos - 6 + 1), pos + 1):
                assert wtable[key // 4] >= 0, (pos, key, wtable)
        m.commit([("r", n)])
        fed += n
        m.check()
    assert m.groups[0].allocator.num_used == -(-fed // 4)  # all keys kept
    # the next query (position 17) sees keys 12..17: pages before logical page 3 are back in the pool
    assert m.groups[1].tables["r"][:3] == [-1, -1, -1] and m.groups[1].allocator.num_used == 2
    assert m.peak_pages_for(100, chunk=8) == 25 and manager([windowed]).peak_pages_for(100, chunk=8) == 5
    m.free_request("r")
    assert all(g.allocator.num_free == 16 for g in m.groups)


def test_shared_cache_entries_see_the_same_plane_and_state_slots_are_zeroed():
    specs = [PagedKVSpec(1, 8), None, StateSpec((3, 2))]
    schedule = [LayerRun(0), LayerRun(1, cache_of=0), LayerRun(2)]
    m = manager(specs, schedule=schedule, max_requests=2)
    m.add_request("x")
    m._state_entries[2][m.slot_of["x"]].fill_(7.0)
    m.free_request("x")
    m.add_request("y")  # takes the other slot first (FIFO), then x's old one
    m.add_request("z")
    assert float(m._state_entries[2][m.slot_of["z"]].abs().sum()) == 0.0  # zeroed at the request's start
    with pytest.raises(OutOfPages):
        m.add_request("w")  # only two request slots
    m.reserve([("y", 2)])
    tables, slots = m.step_tables([("y", 2)])
    views = m.views([(torch.from_numpy(t), torch.from_numpy(s)) for t, s in tables], torch.from_numpy(slots), slots.tolist())
    assert views[0].pool.data_ptr() == views[1].pool.data_ptr()  # entry 1 reads entry 0's cache
    assert views[2].states.shape == (2, 3, 2) and views[2].host_slots == [m.slot_of["y"]]


@given(st.integers(0, 2**20))
@settings(max_examples=40, deadline=None)
def test_random_request_orders_never_lose_a_page(seed):
    rng = random.Random(seed)
    m = manager([PagedKVSpec(1, 8), PagedKVSpec(1, 8, window=5)], num_pages=10, max_requests=3)
    live = {}
    for step in range(60):
        roll = rng.random()
        if roll < 0.25 and len(live) < 3:
            name = f"r{step}"
            m.add_request(name)
            live[name] = 0
        elif roll < 0.4 and live:
            name = rng.choice(sorted(live))
            m.free_request(name)
            del live[name]
        elif live:
            batch = [(n, rng.randint(1, 7)) for n in rng.sample(sorted(live), rng.randint(1, len(live)))]
            try:
                m.reserve(batch)
            except OutOfPages:
                m.check()
                continue
            if rng.random() < 0.9:  # a step that failed after reserving simply does not commit
                m.commit(batch)
                for n, k in batch:
                    live[n] += k
        m.check()
        assert {k: m.lengths[k] for k in live} == live
    for name in list(live):
        m.free_request(name)
    assert all(g.allocator.num_free == 10 for g in m.groups) and m.slots.num_free == 3


def test_budget_to_pages():
    specs = [PagedKVSpec(4, 64)] * 22
    per_page = 2 * 22 * 4 * 16 * 64 * 2
    assert num_pages_for_budget(specs, 16, 2, 10 * per_page + 5) == 10  # src/llmserve/kvcache/paged.py:221-227
    assert num_pages_for_budget(specs, 16, 2, 1) == 1


def test_a_steps_tables_and_slots_for_portions_and_single_tokens():
    """`step_tables` for a mixed step: every request's table padded to the widest, released pages as 0, and the slot
    of every new token, token by token."""
    m = manager([PagedKVSpec(1, 8, 6)], page_size=4, num_pages=12)  # a window of 6 keys: early pages are given back
    m.add_request("a")
    m.add_request("b")
    m.reserve([("a", 11)])
    m.commit([("a", 11)])  # a holds positions 0..10; its first page has passed out of the window
    assert m.groups[0].tables["a"][0] == -1
    entries = [("a", 1), ("b", 6)]
    m.reserve(entries)
    (table, slots), = m.step_tables(entries)[0]
    ta, tb = m.groups[0].tables["a"], m.groups[0].tables["b"]
    assert table.shape == (2, 3)
    assert table[0].tolist() == [max(p, 0) for p in ta] and table[1].tolist()[:2] == tb
    want = [ta[11 // 4] * 4 + 11 % 4] + [tb[p // 4] * 4 + p % 4 for p in range(6)]
    assert slots.tolist() == want
    m.commit(entries)
    m.check()


def test_attention_routes_are_worked_out_once_per_step():
    from types import SimpleNamespace

    from llmserve_triton_kernels_b200 import ops

    ctx = SimpleNamespace(host_cu_tokens=[0, 1, 2, 300, 303, 343])  # 1, 1, 298, 3 and 40 tokens
    # groups of 4 heads: 1 and 3 tokens are at most 16 rows (split-key shape), 40 tokens are 160 rows, 298 go to tcgen05
    assert ops._attention_route(ctx, 4, 128) == (5, 298, 3, 160, True)
    assert ops._attention_route(ctx, 4, 0) == (5, 0, 3, 298 * 4, True)
    ctx.host_cu_tokens = None  # kept on the context: not worked out again
    assert ops._attention_route(ctx, 4, 128) == (5, 298, 3, 160, True)
    only_long = SimpleNamespace(host_cu_tokens=[0, 200])
    assert ops._attention_route(only_long, 8, 128) == (1, 200, 0, 0, False)
