"""Page allocator: fixed-size pages, a reservation per owner, lowest id first.

Two ideas are kept apart, as in the reference's ``BlockAllocator``
(``serving/block_allocator.py:22-140``): a request *reserves* the number of
pages it may need at most when it is admitted, so it can never run out in
mid-flight, and it *receives* a physical page only when a token first reaches
that page.  Pages come from a min-heap, so the lowest free id is handed out
first and reuse is deterministic (``block_allocator.py:28-29,86``).  Every page
has exactly one owner (the reference's reference counts exist for prefix
sharing, which is not built).  ``free_page`` gives one page back early and
returns it to the owner's reservation: a windowed layer group uses it when its
window has passed a page.
"""

from __future__ import annotations

import heapq
from typing import Hashable


class OutOfPages(MemoryError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"num_pages must be positive, got {num_pages}")
        self.num_pages = num_pages
        self._free: list[int] = list(range(num_pages))
        heapq.heapify(self._free)
        self._owner_of: list[Hashable | None] = [None] * num_pages
        self._reserved: dict[Hashable, int] = {}   # pages promised, not yet handed out
        self._owned: dict[Hashable, set[int]] = {}

    # ------------------------------------------------------------- counters
    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def reserved_pages(self) -> int:
        return sum(self._reserved.values())

    @property
    def available(self) -> int:
        """Pages that can still be promised to a new owner."""
        return self.free_pages - self.reserved_pages

    def owned(self, owner: Hashable) -> frozenset[int]:
        return frozenset(self._owned.get(owner, ()))

    def has_owner(self, owner: Hashable) -> bool:
        return owner in self._reserved

    # ------------------------------------------------------------ lifecycle
    def can_reserve(self, count: int) -> bool:
        return 0 <= count <= self.available

    def reserve(self, owner: Hashable, count: int) -> None:
        if owner in self._reserved:
            raise ValueError(f"owner {owner!r} already holds a reservation")
        if count < 0:
            raise ValueError(f"cannot reserve {count} pages")
        if count > self.available:
            raise OutOfPages(f"cannot reserve {count} pages for {owner!r}: {self.available} left")
        self._reserved[owner] = count
        self._owned[owner] = set()

    def reserve_more(self, owner: Hashable, count: int) -> None:
        """Promise ``count`` further pages to an owner that already holds a reservation."""
        if owner not in self._reserved:
            raise KeyError(f"owner {owner!r} holds no reservation")
        if count < 0:
            raise ValueError(f"cannot reserve {count} pages")
        if count > self.available:
            raise OutOfPages(f"cannot reserve {count} more pages for {owner!r}: "
                             f"{self.available} left")
        self._reserved[owner] += count

    def allocate(self, owner: Hashable) -> int:
        if owner not in self._reserved:
            raise KeyError(f"owner {owner!r} holds no reservation")
        if self._reserved[owner] <= 0:
            raise OutOfPages(f"owner {owner!r} has used up its reserved pages")
        if not self._free:
            raise RuntimeError("reservation invariant broken: a promised page is not free")
        page = heapq.heappop(self._free)
        self._owner_of[page] = owner
        self._owned[owner].add(page)
        self._reserved[owner] -= 1
        return page

    def free_page(self, owner: Hashable, page: int) -> None:
        """Give one page back early; the owner may later allocate another in its place."""
        if not (0 <= page < self.num_pages):
            raise IndexError(f"page {page} outside [0, {self.num_pages})")
        if self._owner_of[page] != owner or owner not in self._owned or page not in self._owned[owner]:
            raise RuntimeError(f"page {page} is not held by {owner!r} (freed twice?)")
        self._owned[owner].remove(page)
        self._owner_of[page] = None
        self._reserved[owner] += 1
        heapq.heappush(self._free, page)

    def release(self, owner: Hashable) -> int:
        """Give back every page and the reservation of ``owner``; returns the page count."""
        if owner not in self._reserved:
            raise KeyError(f"owner {owner!r} holds nothing (released twice?)")
        pages = self._owned.pop(owner)
        for page in pages:
            self._owner_of[page] = None
            heapq.heappush(self._free, page)
        del self._reserved[owner]
        return len(pages)

    # ------------------------------------------------------------ self-check
    def check(self) -> None:
        """Raise if a page is lost, held twice, or free and owned at once."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise AssertionError("a page is in the free list twice")
        held: list[int] = []
        for owner, pages in self._owned.items():
            for p in pages:
                if self._owner_of[p] != owner:
                    raise AssertionError(f"page {p}: owner table disagrees with {owner!r}")
            held.extend(pages)
        if len(set(held)) != len(held):
            raise AssertionError("a page is held by two owners")
        if set(held) & set(free):
            raise AssertionError("a page is both free and held")
        if len(held) + len(free) != self.num_pages:
            raise AssertionError(f"{self.num_pages - len(held) - len(free)} pages lost")
        if self.reserved_pages > self.free_pages:
            raise AssertionError("more pages promised than free")
