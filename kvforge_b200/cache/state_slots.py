"""Slots for per-request state of fixed size.

umarhassan-cloud/kvforge has no such state (its ``Request`` carries counters only,
src/tokenvault/batching/request.py:40-61), and the Llama decoder needs none; the slot is
handed out all the same, at admission, beside the block table, and is given back when the
request ends, is aborted or is preempted.  A mixer that keeps a running state per request
declares its shape; the pool then holds one device tensor per such mixer call, indexed by
slot.  A request's slot is cleared when it is handed out, so a preempted request that is
admitted again starts from zero.
"""

from __future__ import annotations


class NoFreeSlotsError(RuntimeError):
    pass


class StateSlotPool:
    def __init__(self, num_slots: int) -> None:
        if num_slots <= 0:
            raise ValueError("num_slots must be positive")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._of: dict[str, int] = {}
        self.fresh: list[int] = []  # slots handed out since the last ``take_fresh``

    @property
    def num_free(self) -> int:
        return len(self._free)

    def has(self, seq_id: str) -> bool:
        return seq_id in self._of

    def slot(self, seq_id: str) -> int:
        return self._of[seq_id]

    def allocate(self, seq_id: str) -> int:
        if seq_id in self._of:
            raise ValueError(f"sequence {seq_id} already holds a state slot")
        if not self._free:
            raise NoFreeSlotsError("no free state slot")
        s = self._free.pop()
        self._of[seq_id] = s
        self.fresh.append(s)
        return s

    def free(self, seq_id: str) -> None:
        s = self._of.pop(seq_id, None)
        if s is not None:
            self._free.append(s)

    def take_fresh(self) -> list[int]:
        """Slots handed out since the last call: their device state has to be cleared."""
        out, self.fresh = self.fresh, []
        return out

    def check_invariants(self) -> None:
        held = list(self._of.values())
        if len(set(held)) != len(held):
            raise AssertionError("a state slot is held twice")
        if set(held) & set(self._free):
            raise AssertionError("a state slot is free and held")
        if len(set(self._free)) != len(self._free):
            raise AssertionError("a state slot is on the free list twice")
        if len(held) + len(self._free) != self.num_slots:
            raise AssertionError("a state slot was lost")
