"""The cache manager as seen from Python: pages, block tables per request and group, state slots.

The bookkeeping is the library's (host/cache.cpp).  A `CacheManager` made here owns
host bookkeeping only (no device storage); the one of a replayer or an engine is
reached through that object.  Requests may be named by any hashable value.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass
from typing import Dict, Hashable, List, Mapping, Optional, Sequence, Tuple

import numpy as np

from .. import _capi
from ..status import OutOfPages

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
    dtype: str = "float32"


class _Ids:
    """Any hashable request name -> the library's integer request id."""

    def __init__(self):
        self.of: Dict[Hashable, int] = {}

    def __call__(self, request: Hashable) -> int:
        if request not in self.of:
            self.of[request] = len(self.of)
        return self.of[request]


class CacheManager:
    def __init__(self, kv_needs: Mapping[int, KvNeed] = None, state_needs: Mapping[int, StateNeed] = None, page_size: int = 16,
                 num_pages: int = 1, max_requests: int = 1, pages_per_group: Optional[Mapping[KvNeed, int]] = None, _borrowed=None):
        self._lib = _capi.lib()
        self.ids = _Ids()
        self._owned = _borrowed is None
        if _borrowed is not None:
            self._h = _borrowed
        else:
            needs = {"kv": {str(u): [n.n_kv_head, n.head_dim, n.window] for u, n in (kv_needs or {}).items()},
                     "state": {str(u): {"shape": list(n.shape), "dtype": n.dtype} for u, n in (state_needs or {}).items()},
                     "pages_per_group": [[n.n_kv_head, n.head_dim, n.window, p] for n, p in (pages_per_group or {}).items()]}
            h = C.c_void_p()
            _capi.check(self._lib.lb_cache_create(_capi.b(json.dumps(needs)), page_size, num_pages, max_requests, C.byref(h)))
            self._h = h
        self._refresh()

    def _refresh(self) -> None:
        d = self.describe()
        self.page_size, self.max_requests = d["page_size"], d["max_requests"]
        self.groups = d["groups"]                                   # [{"units", "n_kv_head", "head_dim", "window", "num_pages"}]
        self.group_of_unit = {int(u): g for u, g in d["group_of_unit"].items()}

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "_h", None):
            self._lib.lb_cache_destroy(self._h)
            self._h = None

    def describe(self) -> dict:
        return _capi.json_of(self._lib.lb_cache_describe, self._h)

    # -- requests
    def open(self, request: Hashable) -> None:
        _capi.check(self._lib.lb_cache_open(self._h, self.ids(request)))

    def close(self, request: Hashable) -> None:
        if request not in self.ids.of:
            raise _capi.LiyabError(_capi.ErrorCode.INVALID_ARGUMENT, f"request {request!r} is not open")
        _capi.check(self._lib.lb_cache_close(self._h, self.ids(request)))

    def is_open(self, request: Hashable) -> bool:
        return request in self.ids.of and bool(self._lib.lb_cache_is_open(self._h, self.ids.of[request]))

    def length(self, request: Hashable) -> int:
        n = self._lib.lb_cache_length(self._h, self.ids(request))
        if n < 0:
            raise _capi.error_from(1)
        return int(n)

    @property
    def lengths(self) -> Dict[Hashable, int]:
        names = {v: k for k, v in self.ids.of.items()}
        return {names[int(i)]: n for i, n in self.describe()["lengths"].items()}

    def reserve(self, request: Hashable, n_new: int) -> None:
        _capi.check(self._lib.lb_cache_reserve(self._h, self.ids(request), n_new))

    def commit(self, request: Hashable, n_new: int) -> None:
        _capi.check(self._lib.lb_cache_commit(self._h, self.ids(request), n_new))

    def truncate(self, request: Hashable, length: int) -> None:
        _capi.check(self._lib.lb_cache_truncate(self._h, self.ids(request), length))

    def can_reserve(self, wants: Mapping[Hashable, int]) -> bool:
        n = len(wants)
        out = C.c_int32(0)
        _capi.check(self._lib.lb_cache_can_reserve(self._h, n, (C.c_int64 * n)(*[self.ids(r) for r in wants]),
                                                   (C.c_int64 * n)(*wants.values()), C.byref(out)))
        return bool(out.value)

    def state_slot(self, request: Hashable) -> int:
        out = C.c_int32(0)
        _capi.check(self._lib.lb_cache_state_slot(self._h, self.ids(request), C.byref(out)))
        return out.value

    # -- what a step needs
    def block_table(self, group: int, requests: Sequence[Hashable], width: Optional[int] = None) -> np.ndarray:
        n = len(requests)
        ids = (C.c_int64 * n)(*[self.ids(r) for r in requests])
        w = C.c_int32(width or 0)
        _capi.check(self._lib.lb_cache_block_table(self._h, group, n, ids, C.byref(w), None, 0))
        out = np.empty((n, w.value), dtype=np.int32)
        _capi.check(self._lib.lb_cache_block_table(self._h, group, n, ids, C.byref(w), out.ctypes.data_as(C.POINTER(C.c_int32)), out.size))
        return out

    def table_of(self, group: int, request: Hashable) -> np.ndarray:
        """The request's own pages in `group`, one entry per logical page it spans."""
        pages = -(-self.length(request) // self.page_size)
        t = self.block_table(group, [request])[0]
        return t[:max(pages, 0)] if pages <= len(t) else t

    def slot_mapping(self, group: int, request: Hashable, start: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int32)
        _capi.check(self._lib.lb_cache_slot_mapping(self._h, group, self.ids(request), start, n, out.ctypes.data_as(C.POINTER(C.c_int32))))
        return out

    # -- accounting
    def _pages(self) -> Tuple[List[int], List[int]]:
        g = len(self.groups)
        used, free = (C.c_int32 * max(1, g))(), (C.c_int32 * max(1, g))()
        _capi.check(self._lib.lb_cache_pages(self._h, used, free, g))
        return list(used)[:g], list(free)[:g]

    def pages_in_use(self) -> Dict[int, int]:
        return dict(enumerate(self._pages()[0]))

    def free_pages(self) -> Dict[int, int]:
        return dict(enumerate(self._pages()[1]))

    def state_slots_free(self) -> int:
        return int(self._lib.lb_cache_state_slots_free(self._h))

    def check(self) -> None:
        """No page lost, held twice or freed twice; rows of closed requests are empty."""
        _capi.check(self._lib.lb_cache_check(self._h))


__all__ = ["UNMAPPED", "CacheManager", "KvNeed", "StateNeed", "OutOfPages"]
