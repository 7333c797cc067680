"""Free lists for cache blocks and sequence slots, with ownership checks.

The reference's ``BlockPool`` is a LIFO list that hands out block 0 first and
throws ``"OOM"`` when empty; its ``free_block`` checks nothing
(``src/memory/block_pool.cpp:72-75, 193-207``).  Here an id can be held once
only: freeing an id that is not held, or one outside the range, raises.  And the
lowest free id is handed out first, always (a heap, not a stack): as requests
come and go, a sequence's blocks then stay close together in the cache instead
of being scattered over it in the order of earlier releases.
"""
from __future__ import annotations

import heapq
from typing import Iterable, List


class CacheFull(RuntimeError):
    """Not enough free blocks or slots for the request; nothing was taken."""


class IdAllocator:
    def __init__(self, total: int, what: str = "block"):
        if total <= 0:
            raise ValueError(f"number of {what}s must be positive")
        self.total = total
        self.what = what
        self._free: List[int] = list(range(total))               # a heap: the lowest id is handed out first
        self._held = [False] * total

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.total - len(self._free)

    def is_held(self, ident: int) -> bool:
        return 0 <= ident < self.total and self._held[ident]

    def take(self, count: int = 1) -> List[int]:
        """``count`` ids, or ``CacheFull`` with nothing taken."""
        if count < 0:
            raise ValueError("count must be non-negative")
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) wanted, {len(self._free)} of {self.total} free")
        taken = [heapq.heappop(self._free) for _ in range(count)]
        for ident in taken:
            self._held[ident] = True
        return taken

    def give_back(self, idents: Iterable[int]) -> None:
        idents = list(idents)
        for ident in idents:
            if not (0 <= ident < self.total):
                raise ValueError(f"{self.what} id {ident} is outside [0, {self.total})")
            if not self._held[ident]:
                raise ValueError(f"{self.what} id {ident} is freed but not held")
        if len(set(idents)) != len(idents):
            raise ValueError(f"a {self.what} id is freed twice in one call")
        for ident in idents:
            self._held[ident] = False
            heapq.heappush(self._free, ident)
