"""Host-side bookkeeping of the cache: which pages and which slots are free.

Both pools fail loudly on misuse (a page or slot freed twice, or one that was
never handed out), because a page held by two sequences is a silent corruption
that would only show as wrong tokens much later.
"""
from __future__ import annotations

from typing import List

PAGE = 64  # positions per page; the kernels (csrc/common.cuh) use the same number


class CacheFull(RuntimeError):
    """No free page or slot is left (the reference's JANAS_LLM_EFULL,
    include/janas/llm.h:43-53)."""

    code = -5


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class PagePool:
    """The pages of one layer group.  Pages are handed out lowest-free first
    and come back when a sequence ends or a window has moved past them."""

    def __init__(self, n_pages: int, name: str = "cache"):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self.name = name
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{self.name}: {count} pages wanted, {len(self._free)} of "
                            f"{self.n_pages} free ({self.n_pages * PAGE} tokens in all)")
        got = [self._free.pop() for _ in range(count)]
        for p in got:
            self._held[p] = True
        return got

    def give_back(self, pages: List[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages or not self._held[p]:
                raise RuntimeError(f"{self.name}: page {p} given back but not held")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or held, and none is both or twice free."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise RuntimeError(f"{self.name}: a page is free twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise RuntimeError(f"{self.name}: page {p} is "
                                   + ("held and free" if self._held[p] else "lost"))


class SlotPool:
    """The slots: one per live sequence."""

    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("at least one slot is needed")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))
        self._live = [False] * n_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def live(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._live[slot]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} sequence slots are in use")
        s = self._free.pop()
        self._live[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not self.live(slot):
            raise RuntimeError(f"slot {slot} given back but not in use")
        self._live[slot] = False
        self._free.append(slot)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise RuntimeError("a slot is free twice")
        for s in range(self.n_slots):
            if self._live[s] == (s in free):
                raise RuntimeError(f"slot {s} is " + ("live and free" if self._live[s] else "lost"))
