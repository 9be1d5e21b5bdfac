"""The page allocator and the state slots: slot arithmetic, growth, exhaustion, windows,
and accounting under random orders of requests (no page lost, held twice or freed twice)."""

from __future__ import annotations

import random

import pytest

from kvforge_b200.cache.block_manager import BlockManager, GroupSpec, NoFreeBlocksError
from kvforge_b200.cache.state_slots import NoFreeSlotsError, StateSlotPool


def test_alloc_free_roundtrip_and_block_major_slots():
    bm = BlockManager(8, 4)
    bm.allocate("a", 10)
    assert bm.get_block_table("a") == [0, 1, 2]  # block 0 is handed out first
    assert bm.slots("a", 0, 10) == [0, 1, 2, 3, 4, 5, 6, 7, 8, 9]
    bm.allocate("b", 5)
    assert bm.slot("b", 4) == 4 * 4 + 0
    bm.free("a")
    bm.check_invariants()
    bm.allocate("c", 4)
    assert bm.get_block_table("c") == [0]  # the page freed last (tail first) is used again first
    bm.free("b"), bm.free("c")
    assert bm.num_free_blocks == 8
    bm.free("nobody")  # unknown request: ignored
    bm.check_invariants()


def test_growth_only_at_block_boundary_and_exhaustion():
    bm = BlockManager(3, 4)
    bm.allocate("a", 4)
    assert bm.can_append_slots("a", 5, 4)
    bm.append_slots("a", 5, 4)
    assert len(bm.get_block_table("a")) == 2
    bm.append_slots("a", 8, 5)
    assert len(bm.get_block_table("a")) == 2
    bm.allocate("b", 1)
    assert not bm.can_append_slots("a", 9, 8)
    with pytest.raises(NoFreeBlocksError):
        bm.append_slots("a", 9, 8)
    with pytest.raises(NoFreeBlocksError):
        bm.allocate("c", 1)
    with pytest.raises(ValueError):
        bm.allocate("a", 1)
    bm.check_invariants()


def test_watermark_holds_pages_back_at_admission():
    bm = BlockManager(100, 4, watermark=0.1)
    assert bm.watermark_blocks == 10
    assert bm.can_allocate(90 * 4) and not bm.can_allocate(91 * 4)


def test_double_free_is_caught():
    bm = BlockManager(4, 4)
    bm.allocate("a", 4)
    pool = bm._pools[0]
    b = bm.get_block_table("a")[0]
    pool.release(b)
    with pytest.raises(RuntimeError, match="double free"):
        pool.release(b)


def test_window_group_gives_pages_back_when_the_window_has_passed():
    bm = BlockManager(16, 4, groups=[GroupSpec("full"), GroupSpec("window", 6)])
    bm.allocate("a", 10, num_scheduled=10)
    assert len(bm.get_block_table("a", 0)) == 3 and len(bm.get_block_table("a", 1)) == 3
    # the next query is at 10 and sees keys 5..10: page 0 (positions 0-3) is out of every window
    bm.append_slots("a", 11, 10)
    assert bm.get_block_table("a", 1)[0] == -1 and bm.get_block_table("a", 1)[1] >= 0
    assert all(b >= 0 for b in bm.get_block_table("a", 0))
    with pytest.raises(RuntimeError):
        bm.slot("a", 2, 1)
    used_before = 16 - bm.free_blocks_of(1)
    for n in range(12, 60):
        bm.append_slots("a", n, n - 1)
        bm.check_invariants()
    assert 16 - bm.free_blocks_of(1) <= used_before + 1  # the window group stays small
    assert 16 - bm.free_blocks_of(0) == 15  # the full group keeps everything
    bm.free("a")
    assert bm.free_blocks_of(0) == 16 and bm.free_blocks_of(1) == 16


def test_window_group_with_portions():
    bm = BlockManager(8, 4, groups=[GroupSpec("window", 5)])
    assert bm.can_allocate(100, 8)  # only the first portion has to fit
    bm.allocate("a", 100, num_scheduled=8)
    start = 8
    while start < 100:
        end = min(100, start + 7)
        assert bm.can_append_slots("a", end, start)
        bm.append_slots("a", end, start)
        table = bm.get_block_table("a", 0)
        first_needed = max(0, start - 5 + 1) // 4
        assert all(b >= 0 for b in table[first_needed:]) and all(b < 0 for b in table[:first_needed])
        bm.check_invariants()
        start = end


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    groups = [GroupSpec("full"), GroupSpec("window", 9)] if seed % 2 else None
    bm = BlockManager(40, 4, groups=groups)
    slots = StateSlotPool(6)
    live: dict[str, int] = {}
    for step in range(600):
        op = rng.random()
        if op < 0.3 and len(live) < 6:
            name, n = f"r{step}", rng.randint(1, 30)
            if bm.can_allocate(n, n):
                bm.allocate(name, n, n)
                slots.allocate(name)
                live[name] = n
        elif op < 0.8 and live:
            name = rng.choice(sorted(live))
            grow = rng.randint(1, 9)
            if bm.can_append_slots(name, live[name] + grow, live[name]):
                bm.append_slots(name, live[name] + grow, live[name])
                live[name] += grow
                bm.slot(name, live[name] - 1, bm.num_groups - 1)  # the newest position always has a page
        elif live:
            name = rng.choice(sorted(live))
            bm.free(name), slots.free(name)
            del live[name]
        bm.check_invariants()
        slots.check_invariants()
        held = sum(1 for t in bm._pools[0].tables.values() for b in t if b >= 0)
        assert held + bm.free_blocks_of(0) == 40
    for name in list(live):
        bm.free(name), slots.free(name)
    assert bm.num_free_blocks == 40 and slots.num_free == 6


def test_state_slots():
    p = StateSlotPool(2)
    assert p.allocate("a") == 0 and p.allocate("b") == 1
    assert p.take_fresh() == [0, 1] and p.take_fresh() == []
    with pytest.raises(NoFreeSlotsError):
        p.allocate("c")
    with pytest.raises(ValueError):
        p.allocate("a")
    p.free("a")
    assert p.allocate("c") == 0 and p.slot("c") == 0 and p.take_fresh() == [0]
    p.free("zzz")
    p.check_invariants()
