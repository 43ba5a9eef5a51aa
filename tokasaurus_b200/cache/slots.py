"""Slots for per-request state of fixed size.

The reference gives every running sequence a ``batch_index`` from ``BatchIndexAllocator``
(tokasaurus/manager/allocator.py:421-431) and keys one device table by it: the last token each
sequence produced (tokasaurus/model/basic_worker.py:101-137,198-200).  Here the slot also
addresses the state regions that mixers with ``StateNeed`` ask for; the dense Llama decoder asks
for none, so for it only the last-token table is used.
"""

from __future__ import annotations


class NoSlotError(ValueError):
    pass


class StateSlotAllocator:
    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("need at least one slot")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._owner: list[object | None] = [None] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, owner: object) -> int:
        if not self._free:
            raise NoSlotError(f"all {self.num_slots} request slots are in use")
        s = self._free.pop()
        self._owner[s] = owner
        return s

    def release(self, slot: int, owner: object) -> None:
        if not 0 <= slot < self.num_slots or self._owner[slot] is None:
            raise ValueError(f"slot {slot} is not in use")
        if self._owner[slot] != owner:
            raise ValueError(f"slot {slot} belongs to {self._owner[slot]!r}, not to {owner!r}")
        self._owner[slot] = None
        self._free.append(slot)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a slot is in the free list twice")
        for s in range(self.num_slots):
            if (s in free) == (self._owner[s] is not None):
                raise AssertionError(f"slot {s}: free={s in free}, owner={self._owner[s]!r}")
