"""Cache manager: paged keys/values per layer group, block tables, state slots.

Layers whose mixers need the same kind of cache (equal cache specs: for keys and
values the same number of heads, head size and window) form a *group*.  A group has
its own pool of pages ``[entries, pages+1, *spec.page_shape(page_size)]`` (for keys
and values ``[entries, pages+1, 2, kv_heads, page_size, head_dim]``; one page id
addresses the same slot in every cache entry of the group; the last page is scratch
for padding rows of a fixed-size batch), its own page size if the spec names one, its
own allocator and, for every live request, its own block table.  The manager only
counts pages: how a page is shaped is the spec's business.  A group that keeps every key holds a request's
pages until the request ends; a group with a window gives a page back as soon
as every key on it lies before the window of the request's next query.

Beside the pages there are *slots*: one row per admitted request in every
state tensor ``[slots+1, *shape]`` (last row scratch).  A slot is the
reference's admission slot (``serving/request.py:59``, ``scheduler.py:59,116``);
mixers with fixed-size state keep it there.  An architecture whose mixers keep
no such state, as Llama, has slots with no tensors behind them.

Reference: ``serving/paged_kv_cache.py:41-332`` (one group, one geometry,
``block_tables`` and ``lengths`` per request, pages reserved at admission and
allocated lazily, ``:167,300-304``; freed on release, ``:286-289``).
"""

from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Callable, Hashable

import torch

from ..parts.base import CacheSpec, LayerCache
from .allocator import OutOfPages, PageAllocator

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


def pages_for(tokens: int, page_size: int) -> int:
    return (tokens + page_size - 1) // page_size


@dataclass
class _RequestPages:
    table: list[int] = field(default_factory=list)  # logical page -> physical page, -1 = given back
    first_live: int = 0                              # logical pages below this were given back


class PageGroup:
    """One layer group's pages."""

    def __init__(self, index: int, spec: CacheSpec, entries: list[int], page_size: int,
                 num_pages: int, dtype: torch.dtype, device: torch.device | None):
        self.index = index
        self.spec = spec
        self.entries = entries
        self.page_size = page_size = int(getattr(spec, "page_size", None) or page_size)
        self.page_shape = tuple(spec.page_shape(page_size))
        self.window = getattr(spec, "window", None)
        if callable(num_pages):
            num_pages = int(num_pages(page_size))
        self.num_pages = num_pages
        self.scratch_page = num_pages
        self.allocator = PageAllocator(num_pages)
        self.requests: dict[Hashable, _RequestPages] = {}
        self.pool: torch.Tensor | None = None
        if device is not None:
            self.pool = torch.zeros((len(entries), num_pages + 1, *self.page_shape),
                                    dtype=dtype, device=device)

    def pages_needed(self, total_tokens: int, max_step_tokens: int) -> int:
        """Most pages a request of ``total_tokens`` holds at any one time."""
        full = pages_for(total_tokens, self.page_size)
        if self.window is None:
            return full
        live_keys = self.window + max_step_tokens - 1
        return min(full, pages_for(live_keys, self.page_size) + 1)

    def bytes_per_page(self) -> int:
        elt = self.pool.element_size() if self.pool is not None else 2
        numel = 1
        for n in self.page_shape:
            numel *= n
        return len(self.entries) * numel * elt


class CacheManager:
    def __init__(self, specs: list[CacheSpec | None], page_size: int,
                 num_pages: "int | dict[int, int] | Callable[[int], int]",
                 max_requests: int, max_step_tokens: int, dtype: torch.dtype = torch.bfloat16,
                 device: torch.device | str | None = None):
        """``page_size``: tokens per page for every group whose spec names no size of its own.
        ``num_pages``: pages per group: one number for all, a number per group index, or a
        function of the group's page size."""
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        if max_requests <= 0:
            raise ValueError(f"max_requests must be positive, got {max_requests}")
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_step_tokens = max_step_tokens
        self.device = torch.device(device) if device is not None else None
        self.dtype = dtype
        self.specs = list(specs)

        # group cache entries by identical paged spec, in order of first appearance
        self.groups: list[PageGroup] = []
        self._entry_group: dict[int, tuple[int, int]] = {}  # entry -> (group, index in group)
        by_spec: dict[CacheSpec, list[int]] = {}
        for e, spec in enumerate(self.specs):
            if spec is None:
                continue
            if spec.storage == "pages":
                by_spec.setdefault(spec, []).append(e)
            elif spec.storage != "slots":
                raise ValueError(f"cache entry {e}: storage {spec.storage!r} is neither "
                                 f"'pages' nor 'slots'")
        for gi, (spec, entries) in enumerate(by_spec.items()):
            n = num_pages[gi] if isinstance(num_pages, dict) else num_pages
            self.groups.append(PageGroup(gi, spec, entries, page_size, n, dtype, self.device))
            for k, e in enumerate(entries):
                self._entry_group[e] = (gi, k)

        # fixed-size state: one tensor per cache entry that asks for it
        self.scratch_slot = max_requests
        self.state: dict[int, torch.Tensor] = {}
        for e, spec in enumerate(self.specs):
            if spec is not None and spec.storage == "slots" and self.device is not None:
                self.state[e] = torch.zeros((max_requests + 1, *spec.slot_shape()),
                                            dtype=_STATE_DTYPES[spec.dtype], device=self.device)
        self._free_slots: list[int] = list(range(max_requests))
        heapq.heapify(self._free_slots)
        self._slot_of: dict[Hashable, int] = {}
        self._length: dict[Hashable, int] = {}
        self._admission: dict[Hashable, int] = {}   # request -> serial number of its admission
        self._admissions = 0

    # ----------------------------------------------------------- admission
    def fits_at_all(self, total_tokens: int) -> bool:
        """Could a request of this many tokens ever be admitted into an empty cache?"""
        return all(g.pages_needed(total_tokens, self.max_step_tokens) <= g.num_pages
                   for g in self.groups)

    def can_admit(self, total_tokens: int) -> bool:
        if not self._free_slots:
            return False
        return all(g.allocator.can_reserve(g.pages_needed(total_tokens, self.max_step_tokens))
                   for g in self.groups)

    def admit(self, request: Hashable, total_tokens: int) -> int:
        """Reserve pages in every group and a slot; returns the slot.  State rows are zeroed."""
        if request in self._slot_of:
            raise ValueError(f"request {request!r} is already admitted")
        if not self.can_admit(total_tokens):
            raise OutOfPages(f"request {request!r} of {total_tokens} tokens does not fit now")
        for g in self.groups:
            g.allocator.reserve(request, g.pages_needed(total_tokens, self.max_step_tokens))
            g.requests[request] = _RequestPages()
        slot = heapq.heappop(self._free_slots)
        self._slot_of[request] = slot
        self._length[request] = 0
        self._admissions += 1
        self._admission[request] = self._admissions
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def reserve_to(self, request: Hashable, total_tokens: int) -> None:
        """Raise an admitted request's reservation so that it can reach ``total_tokens``.

        For callers that do not know a request's final length when they admit
        it (trace replay).  Raises ``OutOfPages`` when the pool cannot promise it.
        """
        for g in self.groups:
            need = g.pages_needed(total_tokens, self.max_step_tokens)
            rp = g.requests[request]
            live = sum(1 for p in rp.table if p >= 0)
            have = live + g.allocator._reserved[request]
            if need > have and need - have > g.allocator.available:
                raise OutOfPages(f"request {request!r} cannot grow to {total_tokens} tokens: "
                                 f"group {g.index} has {g.allocator.available} pages to promise")
        for g in self.groups:
            need = g.pages_needed(total_tokens, self.max_step_tokens)
            rp = g.requests[request]
            have = sum(1 for p in rp.table if p >= 0) + g.allocator._reserved[request]
            if need > have:
                g.allocator.reserve_more(request, need - have)

    def release(self, request: Hashable) -> None:
        """Give back every page and the slot of a finished request."""
        if request not in self._slot_of:
            raise KeyError(f"request {request!r} is not admitted (released twice?)")
        for g in self.groups:
            g.allocator.release(request)
            del g.requests[request]
        heapq.heappush(self._free_slots, self._slot_of.pop(request))
        del self._length[request]
        del self._admission[request]

    # -------------------------------------------------------------- growth
    def length(self, request: Hashable) -> int:
        return self._length[request]

    def slot(self, request: Hashable) -> int:
        return self._slot_of[request]

    def admission(self, request: Hashable) -> int:
        """Serial number of this admission: tells a request from an earlier one of the same name."""
        return self._admission[request]

    def is_admitted(self, request: Hashable) -> bool:
        return request in self._slot_of

    def extend(self, request: Hashable, new_tokens: int) -> int:
        """Make room for ``new_tokens`` more tokens; returns the position of the first.

        In windowed groups, pages that no query of this or a later step can see
        are given back first, so their ids may be handed out again at once.
        """
        if new_tokens <= 0:
            raise ValueError("a step must bring at least one token for a request")
        if new_tokens > self.max_step_tokens:
            raise ValueError(f"{new_tokens} tokens in one step exceed max_step_tokens "
                             f"{self.max_step_tokens}")
        start = self._length[request]
        end = start + new_tokens
        for g in self.groups:
            rp = g.requests[request]
            if g.window is not None:
                first_needed_key = start - g.window + 1
                keep_from = max(0, first_needed_key) // g.page_size
                for lp in range(rp.first_live, min(keep_from, len(rp.table))):
                    if rp.table[lp] >= 0:
                        g.allocator.free_page(request, rp.table[lp])
                        rp.table[lp] = -1
                rp.first_live = max(rp.first_live, min(keep_from, len(rp.table)))
            while len(rp.table) < pages_for(end, g.page_size):
                rp.table.append(g.allocator.allocate(request))
        self._length[request] = end
        return start

    # --------------------------------------------------------------- views
    def block_table(self, request: Hashable, group: int) -> list[int]:
        return self.groups[group].requests[request].table

    def write_slot(self, request: Hashable, group: int, position: int) -> int:
        """Flat slot (page * page_size + offset) where ``position``'s keys/values go."""
        g = self.groups[group]
        page = g.requests[request].table[position // g.page_size]
        if page < 0:
            raise RuntimeError(f"position {position} of {request!r} lies on a page given back")
        return page * g.page_size + position % g.page_size

    def max_table_len(self, group: int, max_seq_len: int) -> int:
        return pages_for(max_seq_len, self.groups[group].page_size)

    def layer_caches(self) -> list[LayerCache | None]:
        """One view per cache entry, in entry order."""
        out: list[LayerCache | None] = []
        for e, spec in enumerate(self.specs):
            if spec is None:
                out.append(None)
            elif spec.storage == "pages":
                gi, k = self._entry_group[e]
                g = self.groups[gi]
                out.append(LayerCache(spec, group=gi,
                                      pool=None if g.pool is None else g.pool[k],
                                      page_size=g.page_size))
            else:
                out.append(LayerCache(spec, state=self.state.get(e)))
        return out

    # ---------------------------------------------------------- accounting
    @property
    def live_requests(self) -> int:
        return len(self._slot_of)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.free_pages

    def check(self) -> None:
        """Raise if any page or slot is lost, held twice or freed twice."""
        for g in self.groups:
            g.allocator.check()
            for request, rp in g.requests.items():
                live = [p for p in rp.table if p >= 0]
                if set(live) != set(g.allocator.owned(request)) or len(set(live)) != len(live):
                    raise AssertionError(f"group {g.index}: table of {request!r} disagrees with "
                                         f"the allocator")
        slots = sorted(self._free_slots) + sorted(self._slot_of.values())
        if sorted(slots) != list(range(self.max_requests)):
            raise AssertionError("a slot is lost or held twice")
