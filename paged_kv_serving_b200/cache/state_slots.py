"""Slots for per-request state of fixed size.

A mixer that keeps a state of its own (not keys and values) gets one slot per running request:
taken when the request is admitted, given back when it ends, is aborted or is preempted, copied
when a request forks, and cleared before a request (re)starts from position zero. The reference
has no such state (its only mixer is attention); the slots exist so that another mixer needs no
change to the cache manager, the scheduler or the step function.
"""

from __future__ import annotations

from collections import deque

__all__ = ["StateSlotPool"]


class StateSlotPool:
    def __init__(self, num_slots: int) -> None:
        if num_slots < 1:
            raise ValueError("num_slots must be >= 1")
        self.num_slots = num_slots
        self._free: deque[int] = deque(range(num_slots))
        self._held: set[int] = set()
        self._to_clear: list[int] = []

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, clear: bool = True) -> int:
        if not self._free:
            raise RuntimeError("no state slot left: more running requests than max_running_seqs")
        slot = self._free.popleft()
        self._held.add(slot)
        if clear:
            self._to_clear.append(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise AssertionError(f"state slot {slot} was given back twice or never taken")
        self._held.remove(slot)
        self._free.append(slot)
        if slot in self._to_clear:
            self._to_clear.remove(slot)

    def take_slots_to_clear(self) -> list[int]:
        """Slots whose state must be zeroed before the next step runs (then forgotten)."""
        out, self._to_clear = self._to_clear, []
        return out

    def check_invariants(self) -> None:
        if len(self._free) + len(self._held) != self.num_slots or set(self._free) & self._held:
            raise AssertionError("state slots are lost or held twice")
