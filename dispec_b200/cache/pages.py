"""Page allocator of one cache group: a free stack, reference counts and reservations.

Follows puneethgv/DiSpec dispec/kv/block_manager.py:37-64,89-96 (free list popped from
the end, a reference count per page that returns the page at zero) and adds reservations:
pages promised to a request at admission that no other request can take.

The stack is laid so that a fresh pool hands out ascending page ids, and a request's pages go
back in the reverse of their table order (cache/manager.py), so that the next request gets them
ascending again: pages that follow each other in a table then follow each other in memory, and
the attention kernel for portions of prompts fetches such a run with one request.  Nothing is
wrong when they do not; it only takes more requests.
"""
from __future__ import annotations


class OutOfPagesError(RuntimeError):
    """No page can be handed out (dispec/kv/block_manager.py:18-19 names it OutOfBlocksError)."""


OutOfBlocksError = OutOfPagesError


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: list[int] = list(range(num_pages - 1, -1, -1))
        self._ref: list[int] = [0] * num_pages
        self.reserved = 0  # pages promised but not yet handed out

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def available(self) -> int:
        """Free pages nobody holds a promise on."""
        return len(self._free) - self.reserved

    def reserve(self, n: int) -> None:
        if n > self.available:
            raise OutOfPagesError(f"cannot reserve {n} pages, {self.available} available")
        self.reserved += n

    def unreserve(self, n: int) -> None:
        if n > self.reserved:
            raise RuntimeError(f"unreserve({n}) exceeds the {self.reserved} reserved pages")
        self.reserved -= n

    def alloc(self, from_reservation: bool = False) -> int:
        if from_reservation:
            if self.reserved <= 0 or not self._free:
                raise RuntimeError("allocation from an empty reservation")
            self.reserved -= 1
        elif self.available <= 0:
            raise OutOfPagesError("page pool exhausted")
        page = self._free.pop()
        self._ref[page] = 1
        return page

    def add_ref(self, page: int) -> None:
        if self._ref[page] <= 0:
            raise RuntimeError(f"page {page} is not in use")
        self._ref[page] += 1

    def release(self, page: int) -> bool:
        """Drops one reference; True when the page went back to the free stack."""
        if not 0 <= page < self.num_pages or self._ref[page] <= 0:
            raise RuntimeError(f"page {page} released but not in use (double free)")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)
            return True
        return False

    def ref_count(self, page: int) -> int:
        return self._ref[page]

    def in_use(self) -> int:
        return self.num_pages - len(self._free)
