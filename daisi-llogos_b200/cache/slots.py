"""Host-side bookkeeping of the cache: sequence slots and pages of 64 tokens.

The reference's cache holds one sequence with one length counter (Inference/KvCache.cs:25,
:90-108, Reset :136).  Here a slot is one sequence's place in the cache: its length, its pages
in every storage group, its row in the fixed-size state.  Slots and pages come from free lists
and go back to them when a batch ends; a slot or page can never be held twice or given back
twice without an error.
"""
from __future__ import annotations

from typing import Dict, Iterable, List


class CacheError(RuntimeError):
    """Misuse of the cache or no room left: raised on the host, before any kernel is launched."""


class FreeList:
    """Integers ``0 .. n-1``; ``take`` hands out the lowest free ones, ``give`` returns them."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise ValueError(f"number of {what}s must not be negative")
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))   # pop() gives the lowest index first
        self._held = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held(self) -> frozenset:
        return frozenset(self._held)

    def take(self, count: int = 1) -> List[int]:
        if count < 0:
            raise ValueError("count must not be negative")
        if count > len(self._free):
            raise CacheError(f"out of {self.what}s: {count} wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        self._held.update(out)
        return out

    def give(self, items: Iterable[int]) -> None:
        items = list(items)
        for i in items:
            if i not in self._held:
                raise CacheError(f"{self.what} {i} is given back but is not held")
        if len(set(items)) != len(items):
            raise CacheError(f"{self.what}s given back twice in one call: {items}")
        for i in items:
            self._held.discard(i)
            self._free.append(i)
        self._free.sort(reverse=True)


class SlotTable:
    """Slots of live sequences with their lengths."""

    def __init__(self, n_slots: int):
        self._slots = FreeList(n_slots, "slot")
        self.length: Dict[int, int] = {}

    @property
    def n_slots(self) -> int:
        return self._slots.n

    @property
    def free_count(self) -> int:
        return self._slots.free_count

    def live(self) -> frozenset:
        return self._slots.held

    def acquire(self) -> int:
        (slot,) = self._slots.take(1)
        self.length[slot] = 0
        return slot

    def release(self, slot: int) -> None:
        self._slots.give([slot])
        del self.length[slot]

    def check_live(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not in use")
