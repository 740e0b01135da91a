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

Bookkeeping is host-side and runs in the CPU tests; only the storage tensors
live on the GPU.  Every open request has a *row* (its state slot); tables and
lengths are NumPy arrays indexed by row, so a step of many requests is laid out
with a handful of array operations (`reserve_rows`, `commit_rows`,
`table_rows`, `decode_slots`) instead of a Python loop per request.

Invariant of a request's table in a group: logical pages below `released` are
unmapped for good, pages in [released, n_logical) are all mapped, and nothing
exists beyond n_logical.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, Iterator, List, Mapping, Optional, Sequence, Tuple

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
        self._held = np.zeros(num_pages, dtype=bool)

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
        self._free.append(int(page))

    def check(self) -> None:
        """No page lost, none held twice, none free twice."""
        if len(set(self._free)) != len(self._free):
            raise LiyabError(ErrorCode.INTERNAL, "a page is on the free list twice")
        for p in self._free:
            if self._held[p]:
                raise LiyabError(ErrorCode.INTERNAL, f"page {p} is both free and held")
        if int(self._held.sum()) + len(self._free) != self.num_pages:
            raise LiyabError(ErrorCode.INTERNAL, "a page is lost")


class _Tables:
    """Read-only, dictionary-like view of a group's tables: request -> its page ids (a NumPy row)."""

    def __init__(self, group: "KvGroup", rows: Mapping[Hashable, int]):
        self._g, self._rows = group, rows

    def __getitem__(self, request: Hashable) -> np.ndarray:
        row = self._rows[request]
        return self._g.table[row, :self._g.n_logical[row]]

    def __contains__(self, request: Hashable) -> bool:
        return request in self._rows

    def items(self) -> Iterator[Tuple[Hashable, np.ndarray]]:
        return ((r, self[r]) for r in self._rows)

    def __len__(self) -> int:
        return len(self._rows)


class KvGroup:
    """Units with the same needs: one storage tensor, one free list, one table row per request."""

    def __init__(self, need: KvNeed, units: Sequence[int], page_size: int, num_pages: int, max_requests: int,
                 rows: Mapping[Hashable, int]):
        self.need = need
        self.units = list(units)
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.table = np.full((max_requests, 16), UNMAPPED, dtype=np.int32)      # columns grow on demand
        self.n_logical = np.zeros(max_requests, dtype=np.int64)                  # pages a row's table spans
        self.released = np.zeros(max_requests, dtype=np.int64)                   # pages below this were freed by the window
        self.tables = _Tables(self, rows)
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

    # -- by row -------------------------------------------------------------

    def pages_for(self, end: np.ndarray) -> np.ndarray:
        return (end + self.page_size - 1) // self.page_size

    def need_rows(self, rows: np.ndarray, end: np.ndarray) -> np.ndarray:
        """Pages each row would take to cover positions < end."""
        return np.maximum(self.pages_for(end) - np.maximum(self.n_logical[rows], self.released[rows]), 0)

    def map_rows(self, rows: np.ndarray, end: np.ndarray) -> None:
        """Maps what `need_rows` counted (the caller has checked that the pool can cover it)."""
        want = self.pages_for(end)
        have = self.n_logical[rows]
        grow = np.nonzero(want > have)[0]
        if grow.size == 0:
            return
        top = int(want.max())
        if top > self.table.shape[1]:
            wider = np.full((self.table.shape[0], max(top, 2 * self.table.shape[1])), UNMAPPED, dtype=np.int32)
            wider[:, :self.table.shape[1]] = self.table
            self.table = wider
        for i in grow:
            row, lo, hi = int(rows[i]), int(have[i]), int(want[i])
            for j in range(max(lo, int(self.released[row])), hi):      # released pages are never mapped again
                self.table[row, j] = self.pool.take()
            self.n_logical[row] = hi

    def release_unreachable_rows(self, rows: np.ndarray, length: np.ndarray) -> None:
        """Windowed groups: frees the pages that no query at a position >= length can see
        (its earliest visible key is length - window + 1)."""
        w = self.need.window
        if w <= 0:
            return
        dead = np.minimum(np.maximum(length - w + 1, 0) // self.page_size, self.n_logical[rows])
        for i in np.nonzero(dead > self.released[rows])[0]:
            row = int(rows[i])
            for j in range(int(self.released[row]), int(dead[i])):
                if self.table[row, j] != UNMAPPED:
                    self.pool.give_back(int(self.table[row, j]))
                    self.table[row, j] = UNMAPPED
            self.released[row] = int(dead[i])

    def truncate_row(self, row: int, length: int, request: Hashable) -> None:
        """Frees the pages that start at or after `length` (a roll-back)."""
        if self.need.window > 0 and self.released[row] * self.page_size > max(0, length - self.need.window + 1):
            raise invalid_argument(f"request {request!r} cannot be cut back to {length}: a windowed group has "
                                   f"already released pages that position would need")
        keep = (length + self.page_size - 1) // self.page_size
        for j in range(keep, int(self.n_logical[row])):
            if self.table[row, j] != UNMAPPED:
                self.pool.give_back(int(self.table[row, j]))
                self.table[row, j] = UNMAPPED
        self.n_logical[row] = min(int(self.n_logical[row]), keep)

    def clear_row(self, row: int) -> None:
        for j in range(int(self.n_logical[row])):
            if self.table[row, j] != UNMAPPED:
                self.pool.give_back(int(self.table[row, j]))
        self.table[row, :] = UNMAPPED
        self.n_logical[row] = 0
        self.released[row] = 0


class StateSlots:
    """Slots of fixed size, one per live request, for units that keep state.  A request's slot is also its
    row in the cache manager's tables."""

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
        self.states = StateSlots(state_needs, max_requests)
        self.row_of = self.states.slot_of                       # request -> row
        self.length_arr = np.zeros(max_requests, dtype=np.int64)
        by_need: Dict[KvNeed, List[int]] = {}
        for unit in sorted(kv_needs):
            by_need.setdefault(kv_needs[unit], []).append(unit)
        self.groups: List[KvGroup] = []
        self.group_of_unit: Dict[int, int] = {}
        for need, units in by_need.items():
            n = (pages_per_group or {}).get(need, num_pages)
            g = KvGroup(need, units, page_size, n, max_requests, self.row_of)
            for u in units:
                self.group_of_unit[u] = len(self.groups)
            self.groups.append(g)
        self.windowed = any(g.need.window > 0 for g in self.groups)
        if device is not None:
            for g in self.groups:
                g.allocate_storage(dtype, device)
            self.states.allocate_storage(device)

    # -- requests -----------------------------------------------------------

    @property
    def lengths(self) -> Dict[Hashable, int]:
        return {r: int(self.length_arr[row]) for r, row in self.row_of.items()}

    def open(self, request: Hashable) -> None:
        if request in self.row_of:
            raise LiyabError(ErrorCode.BUSY, f"request {request!r} is already open")
        if len(self.row_of) >= self.max_requests:
            raise LiyabError(ErrorCode.BUSY, f"{self.max_requests} requests are open already")
        row = self.states.open(request)
        self.length_arr[row] = 0

    def close(self, request: Hashable) -> None:
        if request not in self.row_of:
            raise invalid_argument(f"request {request!r} is not open")
        row = self.row_of[request]
        for g in self.groups:
            g.clear_row(row)
        self.length_arr[row] = 0
        self.states.close(request)

    def is_open(self, request: Hashable) -> bool:
        return request in self.row_of

    def length(self, request: Hashable) -> int:
        return int(self.length_arr[self.row_of[request]])

    def rows(self, requests: Sequence[Hashable]) -> np.ndarray:
        return np.fromiter((self.row_of[r] for r in requests), dtype=np.int64, count=len(requests))

    # -- reserving and committing, by row ---------------------------------------

    def need_rows(self, rows: np.ndarray, n_new: np.ndarray) -> List[int]:
        """Per group, the pages that appending n_new[i] tokens to row rows[i] would take, summed over the rows."""
        end = self.length_arr[rows] + n_new
        return [int(g.need_rows(rows, end).sum()) for g in self.groups]

    def reserve_rows(self, rows: np.ndarray, n_new: np.ndarray) -> None:
        """Maps pages for positions [length, length + n_new) of every row in every group, or none at all."""
        end = self.length_arr[rows] + n_new
        for g in self.groups:
            need = int(g.need_rows(rows, end).sum())
            if need > g.pool.free_count:
                raise OutOfPages(f"{len(rows)} request(s) need {need} more page(s) of {self.page_size} positions; "
                                 f"{g.pool.free_count} of {g.pool.num_pages} are free")
        for g in self.groups:
            g.map_rows(rows, end)

    def commit_rows(self, rows: np.ndarray, n_new: np.ndarray) -> None:
        """The step ran: the rows are n_new tokens longer; windows move on."""
        self.length_arr[rows] += n_new
        if self.windowed:
            for g in self.groups:
                g.release_unreachable_rows(rows, self.length_arr[rows])

    # -- the same by request ---------------------------------------------------------

    def pages_needed(self, request: Hashable, n_new: int) -> Dict[int, int]:
        """Per group, the pages that appending n_new tokens would take."""
        rows, n = self.rows([request]), np.array([n_new])
        return dict(enumerate(self.need_rows(rows, n)))

    def can_reserve(self, wants: Mapping[Hashable, int]) -> bool:
        """Whether all of {request: n_new} fit the free pages together."""
        if not wants:
            return True
        rows = self.rows(list(wants))
        need = self.need_rows(rows, np.fromiter(wants.values(), dtype=np.int64, count=len(wants)))
        return all(n <= g.pool.free_count for n, g in zip(need, self.groups))

    def reserve(self, request: Hashable, n_new: int) -> None:
        if n_new <= 0:
            raise invalid_argument(f"request {request!r}: a reservation needs at least one token")
        self.reserve_rows(self.rows([request]), np.array([n_new], dtype=np.int64))

    def commit(self, request: Hashable, n_new: int) -> None:
        self.commit_rows(self.rows([request]), np.array([n_new], dtype=np.int64))

    def truncate(self, request: Hashable, length: int) -> None:
        row = self.row_of[request]
        if not (0 <= length <= self.length_arr[row]):
            raise invalid_argument(f"request {request!r} holds {int(self.length_arr[row])} tokens, cannot cut to {length}")
        if self.states.needs and length != self.length_arr[row]:
            raise LiyabError(ErrorCode.UNSUPPORTED, "per-request state cannot be rolled back")
        for g in self.groups:
            g.truncate_row(row, length, request)
        self.length_arr[row] = length

    # -- what a step needs ----------------------------------------------------

    def table_rows(self, group: int, rows: np.ndarray, width: Optional[int] = None) -> np.ndarray:
        """The block tables of `rows`, [len(rows), width] int32 (width: the widest of them unless given)."""
        g = self.groups[group]
        w = max(int(g.n_logical[rows].max()) if len(rows) else 1, 1)
        if width is not None:
            if width < w:
                raise invalid_argument(f"block table of width {width} cannot hold {w} pages")
            w = width
        if w <= g.table.shape[1]:
            return g.table[rows, :w]
        out = np.full((len(rows), w), UNMAPPED, dtype=np.int32)
        out[:, :g.table.shape[1]] = g.table[rows]
        return out

    def block_table(self, group: int, requests: Sequence[Hashable], width: Optional[int] = None) -> np.ndarray:
        return self.table_rows(group, self.rows(requests), width)

    def slots_of(self, group: int, token_rows: np.ndarray, positions: np.ndarray) -> np.ndarray:
        """Flat slot (page * page_size + offset) of each (row, position) pair."""
        g = self.groups[group]
        pages = g.table[token_rows, positions // self.page_size].astype(np.int64)
        if (pages < 0).any():
            raise LiyabError(ErrorCode.INTERNAL, "a position of the step has no page")
        return (pages * self.page_size + positions % self.page_size).astype(np.int32)

    def slot_mapping(self, group: int, request: Hashable, start: int, n: int) -> np.ndarray:
        pos = np.arange(start, start + n, dtype=np.int64)
        return self.slots_of(group, np.full(n, self.row_of[request], dtype=np.int64), pos)

    def state_slot(self, request: Hashable) -> int:
        return self.row_of[request]

    # -- accounting -----------------------------------------------------------

    def pages_in_use(self) -> Dict[int, int]:
        return {i: g.pool.held_count for i, g in enumerate(self.groups)}

    def free_pages(self) -> Dict[int, int]:
        return {i: g.pool.free_count for i, g in enumerate(self.groups)}

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(es) for g in self.groups)

    def check(self) -> None:
        """Invariants: every held page is in exactly one table, pools are consistent, rows of closed requests are empty."""
        live = set(self.row_of.values())
        for g in self.groups:
            g.pool.check()
            seen = set()
            for row in range(self.max_requests):
                pages = g.table[row][g.table[row] != UNMAPPED]
                if row not in live and pages.size:
                    raise LiyabError(ErrorCode.INTERNAL, f"row {row} of a closed request still holds pages")
                if (g.table[row, int(g.n_logical[row]):] != UNMAPPED).any():
                    raise LiyabError(ErrorCode.INTERNAL, f"row {row} has pages beyond its end")
                for p in pages.tolist():
                    if p in seen:
                        raise LiyabError(ErrorCode.INTERNAL, f"page {p} is in two tables")
                    seen.add(p)
            if len(seen) != g.pool.held_count:
                raise LiyabError(ErrorCode.INTERNAL, "a held page is in no table (lost)")
        self.states.pool.check()
