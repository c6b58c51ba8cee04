"""The cache manager: no page lost, held twice or freed twice, under random orders of requests."""

import random

import pytest
import torch
from hypothesis import given, settings, strategies as st

import tesseract_b200.parts  # noqa: F401
from tesseract_b200.cache import CacheManager, OutOfPages, PagePool, StateSlots
from tesseract_b200.parts import PagedKVNeed, StateNeed


def manager(num_pages=16, page_size=16, max_requests=4, window=None, needs=None, cache_of=None, max_step_tokens=8):
    if needs is None:
        need = PagedKVNeed(2, 16, window)
        needs, cache_of = [need, need], [None, None]
    return CacheManager(needs, cache_of, num_pages=num_pages, page_size=page_size, max_requests=max_requests,
                        dtype=torch.float32, device="cpu", max_step_tokens=max_step_tokens, allocate_storage=False)


def test_pool_lifo_reuse_and_ownership():
    pool = PagePool(4, first_page=1)
    pool.register("a")
    pages = [pool.allocate("a") for _ in range(3)]
    assert pages == [1, 2, 3] and pool.free_pages == 1
    pool.give_back("a", 2)
    assert pool.allocate("a") == 2          # the page given back is the next one used
    with pytest.raises(ValueError):
        pool.give_back("b", 1)              # not the owner
    pool.release("a", [1, 2, 3])
    pool.check()
    pool.register("a")
    with pytest.raises(ValueError):
        pool.release("a", [1])              # freeing a page twice is refused
    pool.check()


def test_reservation_blocks_others_and_cannot_run_out():
    pool = PagePool(6)
    assert pool.reserve("a", 4)
    assert not pool.reserve("b", 3)         # only 2 left to reserve
    assert pool.reserve("b", 2)
    pool.register("c")
    with pytest.raises(OutOfPages):
        pool.allocate("c")                  # everything is spoken for
    for _ in range(4):
        pool.allocate("a")                  # a's reservation always succeeds
    pool.check()
    assert pool.available_to_reserve == 0


def test_state_slots_exclusive_and_reused():
    slots = StateSlots(2)
    assert slots.allocate("a") == 0 and slots.allocate("b") == 1
    assert slots.allocate("c") is None and slots.allocate("a") is None
    slots.release("a")
    assert slots.allocate("c") == 0
    slots.check()


def test_block_tables_follow_positions():
    m = manager()
    assert m.admit("r")
    m.extend("r", 17)                       # crosses into the second page
    m.commit("r", 17)
    assert sorted(m.pages_of("r")) == [0, 1]
    rows = m.block_table_rows(0, [m.slot("r")], 4)
    assert rows.shape == (1, 4) and rows[0, 0] > 0 and rows[0, 1] > 0 and rows[0, 2] == 0
    m.extend("r", 15)                       # stays within page 1
    m.commit("r", 15)
    assert sorted(m.pages_of("r")) == [0, 1]
    m.extend("r", 1)
    assert sorted(m.pages_of("r")) == [0, 1, 2]
    m.release("r")
    assert m.used_pages() == 0
    m.check()


def test_admission_reserves_peak_need_in_every_group():
    full, windowed = PagedKVNeed(2, 16), PagedKVNeed(2, 16, 32)
    m = manager(num_pages=8, needs=[full, windowed, full], cache_of=[None, None, None])
    assert len(m.groups) == 2
    assert m.admit("a", reserve_tokens=100)             # 7 pages of the full group
    assert not m.admit("b", reserve_tokens=40)          # 3 more do not fit
    assert m.admit("c", reserve_tokens=16)
    m.release("a")
    assert m.admit("b", reserve_tokens=40)
    m.check()


def test_window_gives_pages_back_as_it_passes():
    need = PagedKVNeed(1, 16, 20)
    m = manager(num_pages=6, needs=[need], cache_of=[None], max_step_tokens=16)
    assert m.admit("w", reserve_tokens=400)             # far more tokens than pages: the window bounds the need
    held_max = 0
    for _ in range(25):
        m.extend("w", 16)
        held_max = max(held_max, len(m.pages_of("w")))
        m.commit("w", 16)
        m.check()
    assert m.length("w") == 400 and held_max <= 4
    first_live = min(m.pages_of("w"))
    assert first_live == (400 - 20 + 1) // 16
    assert m.pages_reused > 0
    m.release("w")
    assert m.used_pages() == 0


def test_state_group_and_shared_cache_bindings():
    kv, state = PagedKVNeed(2, 16), StateNeed((4, 8))
    m = manager(needs=[kv, state, None, kv], cache_of=[None, None, 0, None])
    assert [b.group if b else None for b in m.bindings] == [0, 1, 0, 0]
    assert m.bindings[2].writes is False and m.bindings[0].writes is True
    assert m.admit("r")
    m.release("r")


def test_on_demand_exhaustion_raises_before_any_damage():
    m = manager(num_pages=3)
    assert m.admit("a") and m.admit("b")
    m.extend("a", 32)
    m.commit("a", 32)
    m.extend("b", 16)
    m.commit("b", 16)
    with pytest.raises(OutOfPages):
        m.extend("b", 1)
    m.check()
    m.release("a")
    m.extend("b", 1)                                    # a's pages are used again
    assert m.pages_reused >= 1
    m.check()


@settings(max_examples=60, deadline=None)
@given(seed=st.integers(0, 10_000), window=st.sampled_from([None, 24, 40]), pages=st.integers(6, 24))
def test_random_orders_keep_every_page_accounted(seed, window, pages):
    rng = random.Random(seed)
    m = manager(num_pages=pages, max_requests=4, window=window, max_step_tokens=20)
    live, counter = {}, 0
    for _ in range(120):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            rid = f"r{counter}"
            counter += 1
            reserve = rng.choice([None, rng.randint(1, 120)])
            if m.admit(rid, reserve_tokens=reserve):
                live[rid] = reserve
        elif action < 0.85 and live:
            rid = rng.choice(sorted(live))
            n = rng.randint(1, 20)
            if live[rid] is not None and m.length(rid) + n > live[rid]:
                n = live[rid] - m.length(rid)
            if n > 0:
                try:
                    m.extend(rid, n)
                    m.commit(rid, n)
                except OutOfPages:
                    assert live[rid] is None, "a request with a reservation ran out of pages"
        elif live:
            rid = rng.choice(sorted(live))
            m.release(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.release(rid)
    m.check()
    assert m.used_pages() == 0 and m.slots.free_slots == 4
    assert all(g.pool.available_to_reserve == pages for g in m.groups)
