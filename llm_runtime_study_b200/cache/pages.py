"""Free list of page ids with strict ownership accounting."""

from __future__ import annotations

import heapq

from ..errors import KVCacheError


class PageAllocator:
    """Hands out the lowest free id first, so reuse is deterministic
    (mini_llm/cache/paged/blocks.py:15-40).  It knows which ids are out: a page
    can be neither handed out twice nor given back twice, and ``check()``
    verifies that free and held ids together are exactly ``0..num_pages-1``."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise KVCacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages))
        heapq.heapify(self._free)
        self._held: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return len(self._held)

    def allocate(self, count: int) -> list[int]:
        if count < 0:
            raise KVCacheError(f"cannot allocate {count} pages")
        if count > len(self._free):
            raise KVCacheError(
                f"KV page pool exhausted: need {count} pages but only {len(self._free)} are free"
            )
        pages = [heapq.heappop(self._free) for _ in range(count)]
        self._held.update(pages)
        return pages

    def free(self, pages) -> None:
        pages = list(pages)
        for page in pages:
            if page not in self._held:
                raise KVCacheError(f"page {page} is given back but is not held")
        if len(set(pages)) != len(pages):
            raise KVCacheError("a page is given back twice in one call")
        for page in pages:
            self._held.remove(page)
            heapq.heappush(self._free, page)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise KVCacheError("a page is on the free list twice")
        if free & self._held:
            raise KVCacheError("a page is both free and held")
        if free | self._held != set(range(self.num_pages)):
            raise KVCacheError("a page was lost")
