"""The cache manager: pages of keys and values with a block table per request,
and slots of fixed-size per-request state.

Run steps with the same need (kv heads, head size, window) form a *group*.  A
group has a page pool and a block table per request of its own, and one key and
one value array per run step: ``[pages, kv_heads, page_size, head_dim]``.  One
page id addresses the same page in every run step of its group
(src/metal/metal_kv_cache.cc:57-69,173-178).

Pages: the free list starts as 0..n-1, pages are taken from its front and given
back at its back, so reuse is first-in first-out (src/block_manager.cc:17-23,
47-50,61-62).  ``reserve`` grows a request to a token count or changes nothing
(src/block_manager.cc:32-53); ``release`` gives everything back and may be
called twice (src/block_manager.cc:55-64).  A group with a window gives a page
back as soon as no later query can see any of its positions.

State slots: a pool of ``max_requests`` slots; a request takes one when it is
admitted (its arrays are zeroed) and gives it back with its pages.  The
reference has this only for its hybrid model
(src/qwen/qwen3_5_model_state.cc:148-166); here every model has the slots, of
size zero when no mixer declares state.

Host bookkeeping only; the arrays live in :class:`CacheStorage`.  The bookkeeping
itself is C++ (``csrc/runtime.cc``); the classes here hold a handle and turn its
status codes into :class:`CacheError`.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from . import native


class CacheError(RuntimeError):
    def __init__(self, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.code = code


def _raise(status: int, what: str = "") -> None:
    code = native.ERROR_CODES.get(status, f"status {status}")
    message = native.error_message()
    if code == "invariant":
        raise AssertionError(message)
    raise CacheError(code, f"{what}{message}" if what else message)


def _ints(values: Sequence[int]):
    return (ctypes.c_int * len(values))(*values)


class PagePool:
    """A first-in first-out free list of page ids."""

    def __init__(self, num_pages: int):
        self._lib = native.runtime()
        self._handle = self._lib.chibi_pool_new(int(num_pages))
        if not self._handle:
            raise CacheError("invalid_configuration", native.error_message())
        self.num_pages = num_pages

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.chibi_pool_delete(self._handle)
            self._handle = None

    @property
    def free_count(self) -> int:
        return self._lib.chibi_pool_free_count(self._handle)

    @property
    def used_count(self) -> int:
        return self.num_pages - self.free_count

    def take(self, count: int) -> List[int]:
        out = (ctypes.c_int * max(count, 1))()
        status = self._lib.chibi_pool_take(self._handle, int(count), out)
        if status < 0:
            _raise(status)
        return list(out[:count])

    def give(self, pages: Sequence[int]) -> None:
        for p in pages:
            status = self._lib.chibi_pool_give(self._handle, int(p))
            if status < 0:
                _raise(status)


@dataclass(frozen=True)
class GroupLayout:
    """What the pages of one group look like."""

    name: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int]
    page_size: int
    num_pages: int
    num_entries: int            # run steps that own a cache in this group
    max_blocks: int = 0         # logical blocks a request can reach (width of the device table)


@dataclass
class RequestCache:
    """What the manager holds for one request, as of the call that returned it."""

    request_id: Hashable
    length: int = 0                       # tokens whose keys are stored (committed)
    reserved: int = 0                     # tokens that the tables have room for
    state_slot: int = -1
    # per group: logical block -> page id, or -1 once the window has passed it
    tables: Dict[str, List[int]] = field(default_factory=dict)


def pages_for(tokens: int, page_size: int) -> int:
    return 0 if tokens <= 0 else 1 + (tokens - 1) // page_size


def first_needed_block(length: int, window: Optional[int], page_size: int) -> int:
    """Lowest logical block that a query at position >= ``length`` can still see.

    Such a query sees keys at positions > its own - window, so positions below
    length - window + 1 are dead."""
    if window is None:
        return 0
    first_pos = max(0, length - window + 1)
    return first_pos // page_size


class _SlotCounts:
    """The state slots of a manager, as numbers (the pool itself is in the C++ manager)."""

    def __init__(self, manager: "CacheManager"):
        self._manager = manager
        self.num_slots = manager.max_requests

    @property
    def free_count(self) -> int:
        return self._manager._lib.chibi_cache_free_slots(self._manager._handle)


class CacheManager:
    def __init__(self, groups: Sequence[GroupLayout], max_requests: int):
        self._lib = native.runtime()
        self.groups: Dict[str, GroupLayout] = {g.name: g for g in groups}
        self._group_index = {g.name: i for i, g in enumerate(groups)}
        self._handle = self._lib.chibi_cache_new(
            len(groups), _ints([g.page_size for g in groups]), _ints([g.num_pages for g in groups]),
            _ints([-1 if g.window is None else g.window for g in groups]), _ints([g.max_blocks for g in groups]),
            int(max_requests))
        if not self._handle:
            raise CacheError("invalid_configuration", native.error_message())
        self.max_requests = max_requests
        # request ids may be any hashable: the C++ side knows them by a running number
        self._numbers: Dict[Hashable, int] = {}
        self._next_number = 0
        self._info = (ctypes.c_int * 3)()
        self.slots = _SlotCounts(self)

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.chibi_cache_delete(self._handle)
            self._handle = None

    # ---- the C++ side's view
    @property
    def handle(self):
        return self._handle

    def number_of(self, request_id: Hashable) -> int:
        try:
            return self._numbers[request_id]
        except KeyError:
            raise CacheError("unknown_request", f"request {request_id!r} is not admitted") from None

    def group_order(self) -> List[str]:
        return list(self._group_index)

    def drain_updates(self, group: str) -> List[Tuple[int, int, int]]:
        """Block-table changes since the last call, for the mirror on the device:
        at most one per (row, block), the latest (they are applied in parallel)."""
        g = self._group_index[group]
        n = self._lib.chibi_cache_pending_updates(self._handle, g)
        out = (ctypes.c_int * max(3 * n, 1))()
        count = self._lib.chibi_cache_drain(self._handle, g, out, n)
        if count < 0:
            _raise(count)
        return [(out[3 * i], out[3 * i + 1], out[3 * i + 2]) for i in range(count)]

    # ---- queries
    @property
    def requests(self) -> Dict[Hashable, RequestCache]:
        return {rid: self.get(rid) for rid in self._numbers}

    def has(self, request_id: Hashable) -> bool:
        return request_id in self._numbers

    def get(self, request_id: Hashable) -> RequestCache:
        number = self.number_of(request_id)
        status = self._lib.chibi_cache_info(self._handle, number, self._info)
        if status < 0:
            _raise(status, f"request {request_id!r}: ")
        rc = RequestCache(request_id, length=self._info[0], reserved=self._info[1], state_slot=self._info[2])
        for name, g in self._group_index.items():
            n = self._lib.chibi_cache_table(self._handle, number, g, None, 0)
            buf = (ctypes.c_int * max(n, 1))()
            self._lib.chibi_cache_table(self._handle, number, g, buf, n)
            rc.tables[name] = list(buf[:n])
        return rc

    def length(self, request_id: Hashable) -> int:
        status = self._lib.chibi_cache_info(self._handle, self.number_of(request_id), self._info)
        if status < 0:
            _raise(status, f"request {request_id!r}: ")
        return self._info[0]

    def state_slot(self, request_id: Hashable) -> int:
        status = self._lib.chibi_cache_info(self._handle, self.number_of(request_id), self._info)
        if status < 0:
            _raise(status, f"request {request_id!r}: ")
        return self._info[2]

    def free_pages(self, group: str) -> int:
        return self._lib.chibi_cache_free_pages(self._handle, self._group_index[group])

    def worst_case_pages(self, group: str, tokens: int) -> int:
        """Most pages of this group that a request of ``tokens`` tokens holds at
        one time (all of them without a window)."""
        return pages_for(tokens, self.groups[group].page_size)

    # ---- life of a request
    def admit(self, request_id: Hashable) -> RequestCache:
        if request_id in self._numbers:
            raise CacheError("duplicate_request", f"request {request_id!r} is already admitted")
        number = self._next_number
        slot = self._lib.chibi_cache_admit(self._handle, number)
        if slot < 0:
            _raise(slot)
        self._next_number += 1
        self._numbers[request_id] = number
        return RequestCache(request_id, state_slot=slot, tables={name: [] for name in self.groups})

    def reserve(self, request_id: Hashable, tokens: int) -> None:
        """Make room for the request to hold ``tokens`` tokens, in every group,
        or change nothing."""
        if tokens <= 0:
            raise CacheError("invalid_reservation", "a reservation needs at least one token")
        status = self._lib.chibi_cache_reserve(self._handle, self.number_of(request_id), int(tokens))
        if status < 0:
            _raise(status, f"request {request_id!r}: ")

    def commit(self, request_id: Hashable, new_length: int) -> None:
        """The request now holds ``new_length`` tokens; pages that its windows
        have passed go back to their pools."""
        status = self._lib.chibi_cache_commit(self._handle, self.number_of(request_id), int(new_length))
        if status < 0:
            _raise(status, f"request {request_id!r}: ")

    _COMMIT, _HOLD, _SETTLE, _ROLLBACK = 0, 1, 2, 3

    def _advance(self, what: int, request_ids: Sequence[Hashable], lengths: Sequence[int]) -> None:
        n = len(request_ids)
        if n == 0:
            return
        ids = (ctypes.c_longlong * n)(*[self.number_of(r) for r in request_ids])
        status = self._lib.chibi_cache_advance(self._handle, what, n, ids, _ints([int(v) for v in lengths]))
        if status < 0:
            _raise(status)

    def commit_many(self, request_ids: Sequence[Hashable], new_lengths: Sequence[int], hold: bool = False) -> None:
        """``commit`` for the requests of a step in one call.  With ``hold`` the
        lengths advance but no window page is given back until ``settle_many``;
        until then ``rollback_many`` can take the lengths back."""
        self._advance(self._HOLD if hold else self._COMMIT, request_ids, new_lengths)

    def settle_many(self, request_ids: Sequence[Hashable]) -> None:
        self._advance(self._SETTLE, request_ids, [0] * len(request_ids))

    def rollback_many(self, request_ids: Sequence[Hashable], old_lengths: Sequence[int]) -> None:
        """Take held commits back; the pages stay with their requests."""
        self._advance(self._ROLLBACK, request_ids, old_lengths)

    def release(self, request_id: Hashable) -> None:
        number = self._numbers.pop(request_id, None)
        if number is None:
            return
        status = self._lib.chibi_cache_release(self._handle, number)
        if status < 0:
            _raise(status, f"request {request_id!r}: ")

    # ---- checks (used by tests and by debug runs)
    def check_invariants(self) -> None:
        status = self._lib.chibi_cache_check(self._handle)
        if status < 0:
            _raise(status)
        if self._lib.chibi_cache_count(self._handle) != len(self._numbers):
            raise AssertionError("the two sides disagree on the number of requests")
