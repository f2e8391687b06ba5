"""Bookkeeping of a pool of fixed-size pages: which are free, which are held.

Pages come out lowest id first from a fresh pool and last-freed first afterwards; releasing a
page that is not held (an id out of range, or freed twice) is an error, and so is asking for a
page when none is free (cuongvng/bare-cuda-4gib engine/src/allocator.cpp:18-53).  The pool
knows nothing about memory; the group that owns it maps page ids to storage.
"""

from __future__ import annotations

import random
from typing import List

from ..errors import CacheError, OutOfPages


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() yields 0, 1, 2, ...
        self._held = [False] * num_pages
        self.high_water = 0
        self.acquired_total = 0   # pages handed out since the start (reuse shows as > num_pages)

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def pages_in_use(self) -> int:
        return self.num_pages - len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise OutOfPages(f"out of pages: all {self.num_pages} pages of the pool are held")
        page = self._free.pop()
        self._held[page] = True
        self.acquired_total += 1
        self.high_water = max(self.high_water, self.pages_in_use)
        return page

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page {page} is not a page of this pool (0..{self.num_pages - 1})")
        if not self._held[page]:
            raise CacheError(f"page {page} is released twice (it is not held)")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return 0 <= page < self.num_pages and self._held[page]

    def shuffle_free_list(self, seed: int) -> None:
        """Tests: hand pages out in a scrambled order so nothing relies on neighbouring ids."""
        random.Random(seed).shuffle(self._free)
