"""Page allocator shared by the engines: a free list over the pages of the engine's paged KV pools.

Every sequence owns a list of page indices; the same index addresses that sequence's rows in the pool of every
layer.  Pages go back to the head of the free list when a sequence ends, so a new sequence takes over pages (and,
in the slot scheduler, a page-table row) that another one used before."""
from __future__ import annotations

from typing import List


class PagePool:
    """Mixin for an engine with `num_pages` pages of `page_size` entries."""

    num_pages: int
    page_size: int

    def _init_pool(self, num_pages: int) -> None:
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))

    def _alloc_pages(self, n: int) -> List[int]:
        if n > len(self._free):
            raise RuntimeError(f"KV pool exhausted: need {n} pages, {len(self._free)} free "
                               f"(pool holds {self.num_pages * self.page_size} tokens; raise kv_pool_tokens)")
        return [self._free.pop() for _ in range(n)]

    def _free_pages(self, pages: List[int]) -> None:
        self._free.extend(reversed(pages))

    def pages_in_use(self) -> int:
        return self.num_pages - len(self._free)
