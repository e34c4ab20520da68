"""Fixed pools of numbered things handed out and taken back on the CPU: cache pages and
per-request slots.

Same contract as the reference's ``FixedBlockAllocator``
(src/mini_llm_runtime/paged_kv_cache.py:36-113): ``allocate(n)`` is atomic (all or nothing),
``free`` detects ids that are not held (double free, foreign id), and the lowest free id is
always handed out first so that runs are reproducible.  On top of that sits a count of
*promised* items: admission promises a request the pages of its whole lifetime without taking
them, so a running request can never find the pool empty.  An allocation made on behalf of a
promise draws the promise down; one made without a promise is refused if it would leave fewer
free items than the promises still outstanding.
"""

from __future__ import annotations

import heapq
from typing import Iterable


class OutOfPages(RuntimeError):
    """The pool cannot satisfy an allocation; nothing was taken."""


class PoolAllocator:
    def __init__(self, total: int, what: str = "page") -> None:
        if total <= 0:
            raise ValueError(f"a {what} pool needs at least one {what}")
        self.total = int(total)
        self.what = what
        self._free = list(range(self.total))  # already a valid min-heap
        self._held: set[int] = set()
        self._promised = 0
        self._drawn = 0        # items currently held on behalf of promises

    # ---- physical items
    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return len(self._held)

    @property
    def held(self) -> frozenset[int]:
        return frozenset(self._held)

    def allocate(self, count: int, *, promised: bool = False) -> list[int]:
        """``promised=True``: the items were promised to the caller before (``promise``)."""
        if count < 0:
            raise ValueError("cannot allocate a negative count")
        available = len(self._free)
        if not promised:
            available -= max(0, self._promised - self._drawn)     # keep what is promised to others
        if count > available:
            raise OutOfPages(f"{count} {self.what}s wanted, {len(self._free)} of {self.total} free"
                             + ("" if promised else f", {max(0, self._promised - self._drawn)} of them promised"))
        taken = [heapq.heappop(self._free) for _ in range(count)]
        self._held.update(taken)
        if promised:
            self._drawn += count
        return taken

    def free(self, ids: Iterable[int], *, promised: bool = False) -> None:
        """``promised=True``: the items had been taken with ``allocate(promised=True)``."""
        ids = list(ids)
        if len(set(ids)) != len(ids):
            raise ValueError(f"the same {self.what} is freed twice in one call: {sorted(ids)}")
        foreign = [i for i in ids if i not in self._held]
        if foreign:
            raise ValueError(f"{self.what}s {sorted(foreign)} are not held (double free or foreign id)")
        if promised:
            if len(ids) > self._drawn:
                raise ValueError(f"more {self.what}s returned under a promise than were taken under one")
            self._drawn -= len(ids)
        for i in ids:
            self._held.discard(i)
            heapq.heappush(self._free, i)

    # ---- promises (counted reservations)
    @property
    def promised(self) -> int:
        return self._promised

    @property
    def unpromised(self) -> int:
        return self.total - self._promised

    def promise(self, count: int) -> bool:
        """Promise ``count`` more items if the pool can still honour every promise."""
        if count < 0:
            raise ValueError("cannot promise a negative count")
        if self._promised + count > self.total:
            return False
        self._promised += count
        return True

    def unpromise(self, count: int) -> None:
        if count < 0 or count > self._promised:
            raise ValueError(f"cannot take back {count} promises, {self._promised} are out")
        if self._promised - count < self._drawn:
            raise ValueError(f"{self._drawn} {self.what}s are still held under the promises being taken back")
        self._promised -= count
