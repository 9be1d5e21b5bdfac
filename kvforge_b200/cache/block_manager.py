"""Host-side page allocator: pools of fixed-size pages, one block table per request and
cache group, slot arithmetic.  It never touches tensors.

Follows umarhassan-cloud/kvforge's ``BlockManager`` (src/tokenvault/cache/block_manager.py:55-314)
in what the scheduler sees: ``can_allocate`` / ``allocate`` at admission (with a watermark),
``can_append_slots`` / ``append_slots`` for every running request every step, ``free`` when a
request ends, is aborted or is preempted; a last-in-first-out free list whose block 0 is
handed out first (block_manager.py:73-74), so freed pages are the first used again.
Left out: sharing (fork, copy-on-write) and the prefix cache.

Added: cache *groups*.  Layers that keep the same thing per token form a group with pages
and tables of its own.  A ``full`` group keeps every key.  A ``window`` group keeps the last
``window`` keys: ``append_slots`` gives pages back once every position in them lies before
``write_start - window + 1`` (no later query can see them); the table entry becomes ``-1``.
"""

from __future__ import annotations

import numpy as np

from collections.abc import Sequence
from dataclasses import dataclass


class NoFreeBlocksError(RuntimeError):
    pass


RELEASED = -1


@dataclass(frozen=True)
class GroupSpec:
    kind: str = "full"  # "full" or "window"
    window: int | None = None

    def __post_init__(self) -> None:
        if self.kind not in ("full", "window"):
            raise ValueError(f"cache group kind {self.kind!r} is not 'full' or 'window'")
        if self.kind == "window" and (self.window is None or self.window <= 0):
            raise ValueError("a window group needs a positive window")


@dataclass(frozen=True)
class BlockManagerStats:
    num_blocks: int
    block_size: int
    num_used_blocks: int
    num_free_blocks: int
    num_tokens: int
    utilization: float
    internal_fragmentation: float


class _Pool:
    def __init__(self, num_blocks: int, spec: GroupSpec) -> None:
        self.spec = spec
        self.num_blocks = num_blocks
        self.free: list[int] = list(range(num_blocks - 1, -1, -1))
        self.held = [False] * num_blocks
        self.tables: dict[str, list[int]] = {}

    def pop(self) -> int:
        if not self.free:
            raise NoFreeBlocksError("KV cache exhausted")
        b = self.free.pop()
        self.held[b] = True
        return b

    def release(self, b: int) -> None:
        if b < 0 or b >= self.num_blocks or not self.held[b]:
            raise RuntimeError(f"double free of block {b}")
        self.held[b] = False
        self.free.append(b)


class BlockManager:
    def __init__(
        self,
        num_blocks: int,
        block_size: int,
        watermark: float = 0.0,
        groups: Sequence[GroupSpec] | None = None,
    ) -> None:
        if num_blocks <= 0 or block_size <= 0:
            raise ValueError("num_blocks and block_size must be positive")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.watermark_blocks = int(watermark * num_blocks)
        self.group_specs = list(groups) if groups is not None else [GroupSpec()]
        self._pools = [_Pool(num_blocks, g) for g in self.group_specs]
        self._num_tokens: dict[str, int] = {}

    # ------------------------------------------------------------------ queries
    @property
    def num_groups(self) -> int:
        return len(self._pools)

    @property
    def num_free_blocks(self) -> int:
        """Free pages of the tightest group."""
        return min((len(p.free) for p in self._pools), default=self.num_blocks)

    def free_blocks_of(self, group: int) -> int:
        return len(self._pools[group].free)

    def has_seq(self, seq_id: str) -> bool:
        return seq_id in self._num_tokens

    def get_block_table(self, seq_id: str, group: int = 0) -> list[int]:
        return self._pools[group].tables[seq_id]

    def blocks_needed(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    def slot(self, seq_id: str, position: int, group: int = 0) -> int:
        """``block * block_size + offset`` of a position (block_manager.py:101-104)."""
        table = self._pools[group].tables[seq_id]
        b = table[position // self.block_size]
        if b < 0:
            raise RuntimeError(f"position {position} of {seq_id} lies in a page that was given back")
        return b * self.block_size + position % self.block_size

    def slots(self, seq_id: str, start: int, end: int, group: int = 0) -> list[int]:
        """Slots of positions ``start .. end-1``."""
        return self.slots_array(seq_id, start, end, group).tolist()

    def slots_array(self, seq_id: str, start: int, end: int, group: int = 0) -> np.ndarray:
        """The same as an int32 array (a prompt portion has thousands of positions)."""
        table, bs = self._pools[group].tables[seq_id], self.block_size
        if end <= start:
            return np.empty(0, dtype=np.int32)
        first, last = start // bs, (end - 1) // bs
        pages = np.asarray(table[first : last + 1], dtype=np.int64)
        if (pages < 0).any():
            p = (first + int(np.argmax(pages < 0))) * bs
            raise RuntimeError(f"position {max(p, start)} of {seq_id} lies in a page that was given back")
        pos = np.arange(start, end, dtype=np.int64)
        return (pages[pos // bs - first] * bs + pos % bs).astype(np.int32)

    # ------------------------------------------------------------------ sizing
    def _first_live_block(self, pool: _Pool, write_start: int) -> int:
        """First page a query at ``write_start`` or later can still see."""
        if pool.spec.kind != "window":
            return 0
        return max(0, write_start - pool.spec.window + 1) // self.block_size

    def _demand(self, pool: _Pool, seq_id: str | None, total_tokens: int, write_start: int) -> tuple[int, int]:
        """(pages to take, pages that come back first) for holding ``total_tokens`` tokens
        when writing starts at ``write_start``."""
        table = pool.tables.get(seq_id, []) if seq_id is not None else []
        want = self.blocks_needed(total_tokens)
        if pool.spec.kind != "window":
            return max(0, want - len(table)), 0  # a full group never gives pages back: no holes in its table
        first = self._first_live_block(pool, write_start)
        take = sum(1 for i in range(first, want) if i >= len(table) or table[i] < 0)
        back = sum(1 for i in range(min(first, len(table))) if table[i] >= 0)
        return take, back

    def can_ever_fit(self, num_tokens: int, max_portion: int) -> bool:
        """Could a request that grows to ``num_tokens``, fed at most ``max_portion`` tokens a
        step, run in an otherwise empty pool (leaving the watermark free)?"""
        for pool in self._pools:
            need = self.blocks_needed(num_tokens)
            if pool.spec.kind == "window":
                need = min(need, self.blocks_needed(pool.spec.window - 1 + max_portion) + 1)
            if need > pool.num_blocks - self.watermark_blocks:
                return False
        return True

    # ------------------------------------------------------------------ admission
    def can_allocate(self, num_tokens: int, num_scheduled: int | None = None) -> bool:
        """Room for a new request of ``num_tokens`` known tokens, keeping the watermark free
        (block_manager.py:165-170).  A window group only needs the first portion
        (``num_scheduled`` tokens) at once."""
        for pool in self._pools:
            n = num_tokens if pool.spec.kind == "full" else min(num_tokens, num_scheduled or num_tokens)
            if self.blocks_needed(n) > len(pool.free) - self.watermark_blocks:
                return False
        return True

    def allocate(self, seq_id: str, num_tokens: int, num_scheduled: int | None = None) -> int:
        """Make the tables of a new request.  Full groups get pages for all ``num_tokens``
        at once (block_manager.py:172-197).  Returns the number of tokens already in the
        cache, which is always 0 here (no prefix cache)."""
        if seq_id in self._num_tokens:
            raise ValueError(f"sequence {seq_id} already allocated")
        plan = []
        for pool in self._pools:
            n = num_tokens if pool.spec.kind == "full" else min(num_tokens, num_scheduled or num_tokens)
            need = self.blocks_needed(n)
            if need > len(pool.free):
                raise NoFreeBlocksError(f"cannot allocate {need} blocks for {seq_id}")
            plan.append(need)
        for pool, need in zip(self._pools, plan):
            pool.tables[seq_id] = [pool.pop() for _ in range(need)]
        self._num_tokens[seq_id] = num_tokens
        return 0

    # ------------------------------------------------------------------ growth
    def can_append_slots(self, seq_id: str, total_tokens: int, write_start: int) -> bool:
        for pool in self._pools:
            take, back = self._demand(pool, seq_id, total_tokens, write_start)
            if take > len(pool.free) + back:
                return False
        return True

    def append_slots(self, seq_id: str, total_tokens: int, write_start: int) -> list[tuple[int, int]]:
        """Pages for positions up to ``total_tokens`` (block_manager.py:209-236); window groups
        first give back the pages no query from ``write_start`` on can see.  Returns the
        copies to make before the step: always none (nothing is shared)."""
        if seq_id not in self._num_tokens:
            raise KeyError(f"sequence {seq_id} has no tables")
        if not self.can_append_slots(seq_id, total_tokens, write_start):
            raise NoFreeBlocksError(f"cannot append slots for {seq_id}")
        want = self.blocks_needed(total_tokens)
        for pool in self._pools:
            table = pool.tables[seq_id]
            if pool.spec.kind != "window":
                while len(table) < want:
                    table.append(pool.pop())
                continue
            first = self._first_live_block(pool, write_start)
            for i in range(min(first, len(table))):
                if table[i] >= 0:
                    pool.release(table[i])
                    table[i] = RELEASED
            while len(table) < want:
                table.append(RELEASED if len(table) < first else pool.pop())
            for i in range(first, want):
                if table[i] < 0:
                    table[i] = pool.pop()
        self._num_tokens[seq_id] = max(self._num_tokens[seq_id], total_tokens)
        return []

    def mark_computed(self, seq_id: str, num_tokens: int) -> None:
        """Record the live token count (block_manager.py:249-266, without the prefix hashes)."""
        if seq_id in self._num_tokens:
            cap = max(len(p.tables[seq_id]) for p in self._pools) * self.block_size
            self._num_tokens[seq_id] = min(num_tokens, cap)

    def free(self, seq_id: str) -> None:
        """Give back every page of a request, tail first (block_manager.py:268-276).  A request
        that holds nothing is ignored."""
        if self._num_tokens.pop(seq_id, None) is None:
            return
        for pool in self._pools:
            table = pool.tables.pop(seq_id, [])
            for b in reversed(table):
                if b >= 0:
                    pool.release(b)

    # ------------------------------------------------------------------ checks and figures
    def check_invariants(self) -> None:
        """Every page is free or in exactly one table, never both, never twice."""
        for gi, pool in enumerate(self._pools):
            seen: dict[int, str] = {}
            for seq, table in pool.tables.items():
                for b in table:
                    if b < 0:
                        continue
                    if b in seen:
                        raise AssertionError(f"group {gi}: block {b} held by {seen[b]} and {seq}")
                    seen[b] = seq
            free = set(pool.free)
            if len(free) != len(pool.free):
                raise AssertionError(f"group {gi}: a block is on the free list twice")
            if free & set(seen):
                raise AssertionError(f"group {gi}: blocks {sorted(free & set(seen))} are free and held")
            if len(free) + len(seen) != pool.num_blocks:
                raise AssertionError(f"group {gi}: {pool.num_blocks - len(free) - len(seen)} blocks lost")
            for b in range(pool.num_blocks):
                if pool.held[b] != (b in seen):
                    raise AssertionError(f"group {gi}: held flag of block {b} is wrong")

    @property
    def utilization(self) -> float:
        """Share of the first group's pages that are in use."""
        pool = self._pools[0]
        return (pool.num_blocks - len(pool.free)) / self.num_blocks

    def stats(self) -> BlockManagerStats:
        """Figures of the first group (block_manager.py:288-314)."""
        pool = self._pools[0]
        used = pool.num_blocks - len(pool.free)
        tokens = 0
        for seq, table in pool.tables.items():
            n = self._num_tokens.get(seq, 0)
            for i, b in enumerate(table):
                if b >= 0:
                    tokens += min(self.block_size, max(0, n - i * self.block_size))
        slots = used * self.block_size
        return BlockManagerStats(
            num_blocks=self.num_blocks,
            block_size=self.block_size,
            num_used_blocks=used,
            num_free_blocks=len(pool.free),
            num_tokens=tokens,
            utilization=used / self.num_blocks,
            internal_fragmentation=(1.0 - tokens / slots) if slots else 0.0,
        )
