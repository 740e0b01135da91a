"""The cache manager: keys and values in pages, a block table per request and
group, and slots for per-request state of fixed size.

What it owns.  Cache *units* (one per entry of the run order that writes keys
and values) are sorted into *groups* by what they need: number of key/value
heads, head size and attention window.  Each group has pages of its own (one
device tensor [unit, page, K|V, kv_head, slot, head_dim] and one free list) and
one block table per request, shared by the group's units, so a page id means the
same positions in every unit of the group.  Pages return to the free list when a
request closes, when it is cut back, and, in a windowed group, as soon as no
later query can see them; freed pages are handed out again, most recently freed
first.

The reference keeps one `KvCache` per sequence with groups by window, a page
table per group, on-demand mapping in `reserve()`, `truncate()`, windowed
release and `clear()` (include/liyab/kv_cache.h:10-32, 72-428;
src/core/kv_cache.cpp:186-265, 418-439, 474-515) and keeps recurrent state
beside the cache in the sequence's context (src/core/transformer.h:854-865,
1283-1308).  Here one pool serves all requests, which is what lets a finished
request's pages serve the next one.

Nothing in this file touches a GPU except allocating the storage tensors; all
bookkeeping is host-side and runs in the CPU tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, Iterable, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..status import ErrorCode, LiyabError, invalid_argument

UNMAPPED = -1


@dataclass(frozen=True)
class KvNeed:
    """What one cache unit stores per position."""
    n_kv_head: int
    head_dim: int
    window: int = 0          # 0: every position is kept; w: the w latest positions


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size for one unit (e.g. a recurrent mixer)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class OutOfPages(LiyabError):
    """A reservation that the free pages cannot cover; nothing was taken."""

    def __init__(self, message: str):
        super().__init__(ErrorCode.OUT_OF_MEMORY, message)


class PagePool:
    """Free list over page ids 0 .. n-1 with its invariants checked on every move."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise invalid_argument(f"a page pool needs at least one page (got {num_pages})")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() hands out 0 first
        self._held = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.num_pages - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        if self._held[page]:
            raise LiyabError(ErrorCode.INTERNAL, f"page {page} was on the free list while held")
        self._held[page] = True
        return page

    def give_back(self, page: int) -> None:
        if not (0 <= page < self.num_pages) or not self._held[page]:
            raise LiyabError(ErrorCode.INTERNAL, f"page {page} is given back but not held")
        self._held[page] = False
        self._free.append(page)

    def check(self) -> None:
        """No page lost, none held twice, none free twice."""
        if len(set(self._free)) != len(self._free):
            raise LiyabError(ErrorCode.INTERNAL, "a page is on the free list twice")
        for p in self._free:
            if self._held[p]:
                raise LiyabError(ErrorCode.INTERNAL, f"page {p} is both free and held")
        if sum(self._held) + len(self._free) != self.num_pages:
            raise LiyabError(ErrorCode.INTERNAL, "a page is lost")


class KvGroup:
    """Units with the same needs: one storage tensor, one free list, one table per request."""

    def __init__(self, need: KvNeed, units: Sequence[int], page_size: int, num_pages: int):
        self.need = need
        self.units = list(units)
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.tables: Dict[Hashable, List[int]] = {}
        self._released: Dict[Hashable, int] = {}     # logical pages below this were freed by the window
        self.storage: Optional[torch.Tensor] = None

    def unit_index(self, unit: int) -> int:
        return self.units.index(unit)

    def allocate_storage(self, dtype: torch.dtype, device) -> None:
        n = self.need
        self.storage = torch.zeros((len(self.units), self.pool.num_pages, 2, n.n_kv_head, self.page_size, n.head_dim),
                                   dtype=dtype, device=device)

    def unit_storage(self, unit: int) -> torch.Tensor:
        return self.storage[self.unit_index(unit)]

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * len(self.units) * self.need.n_kv_head * self.need.head_dim * element_size

    # -- per request ------------------------------------------------------

    def pages_to_map(self, request: Hashable, end: int) -> int:
        """Pages that `reserve(request, end)` would take."""
        table = self.tables[request]
        n_logical = (end + self.page_size - 1) // self.page_size
        need = 0
        for i in range(self._released.get(request, 0), n_logical):
            if i >= len(table) or table[i] == UNMAPPED:
                need += 1
        return need

    def reserve(self, request: Hashable, end: int) -> None:
        """Maps every page that positions < end need; all or nothing."""
        need = self.pages_to_map(request, end)
        if need > self.pool.free_count:
            raise OutOfPages(f"request {request!r} needs {need} more page(s) of {self.page_size} positions, "
                             f"{self.pool.free_count} of {self.pool.num_pages} are free")
        table = self.tables[request]
        n_logical = (end + self.page_size - 1) // self.page_size
        while len(table) < n_logical:
            table.append(UNMAPPED)
        for i in range(self._released.get(request, 0), n_logical):   # released pages are never mapped again
            if table[i] == UNMAPPED:
                table[i] = self.pool.take()

    def release_unreachable(self, request: Hashable, length: int) -> int:
        """Windowed groups: frees the pages that no query at a position >= length
        can see (its earliest visible key is length - window + 1)."""
        w = self.need.window
        if w <= 0:
            return 0
        table = self.tables[request]
        first_visible = max(0, length - w + 1)
        n_dead = min(first_visible // self.page_size, len(table))
        freed = 0
        for i in range(self._released.get(request, 0), n_dead):
            if table[i] != UNMAPPED:
                self.pool.give_back(table[i])
                table[i] = UNMAPPED
                freed += 1
        self._released[request] = max(self._released.get(request, 0), n_dead)
        return freed

    def truncate(self, request: Hashable, length: int) -> None:
        """Frees the pages that start at or after `length` (a roll-back)."""
        if self.need.window > 0 and \
                self._released.get(request, 0) * self.page_size > max(0, length - self.need.window + 1):
            raise invalid_argument(f"request {request!r} cannot be cut back to {length}: a windowed group has "
                                   f"already released pages that position would need")
        table = self.tables[request]
        keep = (length + self.page_size - 1) // self.page_size
        for i in range(keep, len(table)):
            if table[i] != UNMAPPED:
                self.pool.give_back(table[i])
        del table[keep:]

    def open(self, request: Hashable) -> None:
        self.tables[request] = []

    def close(self, request: Hashable) -> None:
        for page in self.tables.pop(request):
            if page != UNMAPPED:
                self.pool.give_back(page)
        self._released.pop(request, None)


class StateSlots:
    """Slots of fixed size, one per live request, for units that keep state."""

    def __init__(self, needs: Mapping[int, StateNeed], n_slots: int):
        self.needs = dict(needs)
        self.n_slots = n_slots
        self.pool = PagePool(n_slots)
        self.slot_of: Dict[Hashable, int] = {}
        self.storage: Dict[int, torch.Tensor] = {}

    def allocate_storage(self, device) -> None:
        for unit, need in self.needs.items():
            self.storage[unit] = torch.zeros((self.n_slots, *need.shape), dtype=need.dtype, device=device)

    def open(self, request: Hashable) -> int:
        slot = self.pool.take()
        self.slot_of[request] = slot
        for t in self.storage.values():         # state starts at zero for every request
            t[slot].zero_()
        return slot

    def close(self, request: Hashable) -> None:
        self.pool.give_back(self.slot_of.pop(request))


class CacheManager:
    """Everything a request holds between steps."""

    def __init__(self, kv_needs: Mapping[int, KvNeed], state_needs: Mapping[int, StateNeed], page_size: int,
                 num_pages: int, max_requests: int, dtype: torch.dtype = torch.float32, device=None,
                 pages_per_group: Optional[Mapping[KvNeed, int]] = None):
        if page_size <= 0:
            raise invalid_argument(f"page_size must be positive (got {page_size})")
        self.page_size = page_size
        self.max_requests = max_requests
        self.dtype = dtype
        by_need: Dict[KvNeed, List[int]] = {}
        for unit in sorted(kv_needs):
            by_need.setdefault(kv_needs[unit], []).append(unit)
        self.groups: List[KvGroup] = []
        self.group_of_unit: Dict[int, int] = {}
        for need, units in by_need.items():
            n = (pages_per_group or {}).get(need, num_pages)
            g = KvGroup(need, units, page_size, n)
            for u in units:
                self.group_of_unit[u] = len(self.groups)
            self.groups.append(g)
        self.states = StateSlots(state_needs, max_requests)
        self.lengths: Dict[Hashable, int] = {}
        if device is not None:
            for g in self.groups:
                g.allocate_storage(dtype, device)
            self.states.allocate_storage(device)

    # -- requests -----------------------------------------------------------

    def open(self, request: Hashable) -> None:
        if request in self.lengths:
            raise LiyabError(ErrorCode.BUSY, f"request {request!r} is already open")
        if len(self.lengths) >= self.max_requests:
            raise LiyabError(ErrorCode.BUSY, f"{self.max_requests} requests are open already")
        self.lengths[request] = 0
        for g in self.groups:
            g.open(request)
        self.states.open(request)

    def close(self, request: Hashable) -> None:
        if request not in self.lengths:
            raise invalid_argument(f"request {request!r} is not open")
        del self.lengths[request]
        for g in self.groups:
            g.close(request)
        self.states.close(request)

    def is_open(self, request: Hashable) -> bool:
        return request in self.lengths

    def length(self, request: Hashable) -> int:
        return self.lengths[request]

    def pages_needed(self, request: Hashable, n_new: int) -> Dict[int, int]:
        """Per group, the pages that appending n_new tokens would take."""
        end = self.lengths[request] + n_new
        return {i: g.pages_to_map(request, end) for i, g in enumerate(self.groups)}

    def can_reserve(self, wants: Mapping[Hashable, int]) -> bool:
        """Whether all of {request: n_new} fit the free pages together."""
        for i, g in enumerate(self.groups):
            need = sum(g.pages_to_map(r, self.lengths[r] + n) for r, n in wants.items())
            if need > g.pool.free_count:
                return False
        return True

    def reserve(self, request: Hashable, n_new: int) -> None:
        """Maps pages for positions [length, length + n_new) in every group, or none at all."""
        if n_new <= 0:
            raise invalid_argument(f"request {request!r}: a reservation needs at least one token")
        end = self.lengths[request] + n_new
        for g in self.groups:
            need = g.pages_to_map(request, end)
            if need > g.pool.free_count:
                raise OutOfPages(f"request {request!r} needs {need} more page(s) of {self.page_size} positions "
                                 f"for {end} tokens; {g.pool.free_count} of {g.pool.num_pages} are free")
        for g in self.groups:
            g.reserve(request, end)

    def commit(self, request: Hashable, n_new: int) -> None:
        """The step ran: the request is n_new tokens longer; windows move on."""
        self.lengths[request] += n_new
        for g in self.groups:
            g.release_unreachable(request, self.lengths[request])

    def truncate(self, request: Hashable, length: int) -> None:
        if not (0 <= length <= self.lengths[request]):
            raise invalid_argument(f"request {request!r} holds {self.lengths[request]} tokens, cannot cut to {length}")
        if self.states.needs and length != self.lengths[request]:
            raise LiyabError(ErrorCode.UNSUPPORTED, "per-request state cannot be rolled back")
        for g in self.groups:
            g.truncate(request, length)
        self.lengths[request] = length

    # -- what a step needs ----------------------------------------------------

    def block_table(self, group: int, requests: Sequence[Hashable], width: Optional[int] = None) -> np.ndarray:
        g = self.groups[group]
        w = max([len(g.tables[r]) for r in requests] + [1])
        if width is not None:
            if width < w:
                raise invalid_argument(f"block table of width {width} cannot hold {w} pages")
            w = width
        out = np.full((len(requests), w), UNMAPPED, dtype=np.int32)
        for i, r in enumerate(requests):
            t = g.tables[r]
            out[i, :len(t)] = t
        return out

    def slot_mapping(self, group: int, request: Hashable, start: int, n: int) -> np.ndarray:
        """Flat slot (page * page_size + offset) of positions start .. start+n-1."""
        g = self.groups[group]
        pos = np.arange(start, start + n, dtype=np.int64)
        table = np.asarray(g.tables[request], dtype=np.int64)
        pages = table[pos // self.page_size]
        if (pages < 0).any():
            raise LiyabError(ErrorCode.INTERNAL, f"request {request!r}: a position of the step has no page")
        return (pages * self.page_size + pos % self.page_size).astype(np.int32)

    def state_slot(self, request: Hashable) -> int:
        return self.states.slot_of[request]

    # -- accounting -----------------------------------------------------------

    def pages_in_use(self) -> Dict[int, int]:
        return {i: g.pool.held_count for i, g in enumerate(self.groups)}

    def free_pages(self) -> Dict[int, int]:
        return {i: g.pool.free_count for i, g in enumerate(self.groups)}

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(es) for g in self.groups)

    def check(self) -> None:
        """Invariants: every held page is in exactly one table, pools are consistent."""
        for g in self.groups:
            g.pool.check()
            seen = set()
            for r, table in g.tables.items():
                for p in table:
                    if p == UNMAPPED:
                        continue
                    if p in seen:
                        raise LiyabError(ErrorCode.INTERNAL, f"page {p} is in two tables")
                    seen.add(p)
            if len(seen) != g.pool.held_count:
                raise LiyabError(ErrorCode.INTERNAL, "a held page is in no table (lost)")
        self.states.pool.check()
