"""Host-side bookkeeping of the cache: page pools, per-request block tables and
state slots.  No device memory here; ``manager.py`` pairs this with the pools.

The reference keeps one contiguous, left-padded array per layer and copies the
whole cache on every admission and eviction (src/cache/batch_kv_cache.cpp:199-299);
its only "pages" are the prefix cache's immutable blocks, which attention never
reads in place (src/cache/block_pool.h:3-4,40-47).  The page pool, block tables
and slots below are this engine's own design.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np


class OutOfPages(RuntimeError):
    """A reservation that the pool cannot serve.  Nothing was taken."""

    def __init__(self, group: int, wanted: int, free: int, total: int):
        super().__init__(f"cache group {group}: needs {wanted} more pages, {free} of {total} are free")
        self.group, self.wanted, self.free, self.total = group, wanted, free, total


class OutOfSlots(RuntimeError):
    pass


class PagePool:
    """Fixed set of page ids with a LIFO free list.  Every page is either free or
    held by exactly one owner; giving back a page that is not held is an error."""

    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise ValueError("n_pages must be >= 0")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages
        self.high_water = 0

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def take(self, n: int, group: int = 0) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(group, n, len(self._free), self.n_pages)
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        self.high_water = max(self.high_water, self.n_held)
        return out

    def give_back(self, pages: List[int]) -> None:
        for p in pages:
            if not (0 <= p < self.n_pages) or not self._held[p]:
                raise RuntimeError(f"page {p} given back but not held")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """No page lost and none on the free list twice."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise AssertionError(f"page {p} is {'both held and free' if self._held[p] else 'lost'}")


class SlotPool:
    """Ids for per-request state of fixed size; same discipline as pages."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = [False] * n_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.n_slots} request slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, s: int) -> None:
        if not (0 <= s < self.n_slots) or not self._held[s]:
            raise RuntimeError(f"slot {s} given back but not held")
        self._held[s] = False
        self._free.append(s)


@dataclass
class SequenceCache:
    """What one live request holds: its length, one block list per paged group
    (entry -1 = a block that a window has passed and that was given back) and
    its state slot."""

    seq_id: int
    slot: int
    length: int = 0
    blocks: List[List[int]] = field(default_factory=list)   # [group][logical block] -> page or -1
    closed: bool = False
    # int32 copies of `blocks`, kept by the manager, so that a step's block table is a memcpy
    block_rows: List[np.ndarray] = field(default_factory=list)

    def row(self, group: int) -> np.ndarray:
        return self.block_rows[group][:len(self.blocks[group])]

    def _extend(self, group: int, pages: List[int]) -> None:
        have = len(self.blocks[group])
        arr = self.block_rows[group]
        if have + len(pages) > arr.shape[0]:
            grown = np.full(max(2 * arr.shape[0], have + len(pages), 16), -1, dtype=np.int32)
            grown[:have] = arr[:have]
            self.block_rows[group] = arr = grown
        arr[have:have + len(pages)] = pages
        self.blocks[group].extend(pages)

    def pages_held(self, group: int) -> int:
        return sum(1 for p in self.blocks[group] if p >= 0)
