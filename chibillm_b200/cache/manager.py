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

Host bookkeeping only; the arrays live in :class:`CacheStorage`.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple


class CacheError(RuntimeError):
    def __init__(self, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.code = code


class PagePool:
    """A first-in first-out free list of page ids."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("invalid_configuration", "a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = deque(range(num_pages))
        self._held = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheError("capacity_exhausted", f"{count} pages wanted, {len(self._free)} free")
        out = []
        for _ in range(count):
            p = self._free.popleft()
            assert not self._held[p], "page handed out twice"
            self._held[p] = True
            out.append(p)
        return out

    def give(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages) or not self._held[p]:
                raise CacheError("invalid_release", f"page {p} is not held")
            self._held[p] = False
            self._free.append(p)


class SlotPool:
    """State slots, lowest free index first."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError("capacity_exhausted", "no state slot is free")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots) or not self._held[slot]:
            raise CacheError("invalid_release", f"state slot {slot} is not held")
        self._held[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)


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


class CacheManager:
    def __init__(self, groups: Sequence[GroupLayout], max_requests: int):
        if max_requests <= 0:
            raise CacheError("invalid_configuration", "max_requests must be positive")
        self.groups: Dict[str, GroupLayout] = {g.name: g for g in groups}
        self.pools: Dict[str, PagePool] = {g.name: PagePool(g.num_pages) for g in groups}
        self.slots = SlotPool(max_requests)
        self.max_requests = max_requests
        self.requests: Dict[Hashable, RequestCache] = {}
        # per group: (table row, logical block, page or -1) changes since the last drain, in
        # order; the row of a request is its state slot
        self._updates: Dict[str, List[Tuple[int, int, int]]] = {g.name: [] for g in groups}

    def drain_updates(self, group: str) -> List[Tuple[int, int, int]]:
        """Block-table changes since the last call, for the mirror on the device:
        at most one per (row, block), the latest (they are applied in parallel)."""
        last: Dict[Tuple[int, int], int] = {}
        for row, index, page in self._updates[group]:
            last[(row, index)] = page
        self._updates[group] = []
        return [(row, index, page) for (row, index), page in last.items()]

    # ---- queries
    def has(self, request_id: Hashable) -> bool:
        return request_id in self.requests

    def get(self, request_id: Hashable) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError("unknown_request", f"request {request_id!r} is not admitted") from None

    def length(self, request_id: Hashable) -> int:
        return self.get(request_id).length

    def free_pages(self, group: str) -> int:
        return self.pools[group].free_count

    def worst_case_pages(self, group: str, tokens: int) -> int:
        """Most pages of this group that a request of ``tokens`` tokens holds at
        one time (all of them without a window)."""
        g = self.groups[group]
        return pages_for(tokens, g.page_size)

    # ---- life of a request
    def admit(self, request_id: Hashable) -> RequestCache:
        if request_id in self.requests:
            raise CacheError("duplicate_request", f"request {request_id!r} is already admitted")
        slot = self.slots.take()
        rc = RequestCache(request_id, state_slot=slot, tables={name: [] for name in self.groups})
        self.requests[request_id] = rc
        return rc

    def reserve(self, request_id: Hashable, tokens: int) -> None:
        """Make room for the request to hold ``tokens`` tokens, in every group,
        or change nothing."""
        if tokens <= 0:
            raise CacheError("invalid_reservation", "a reservation needs at least one token")
        rc = self.get(request_id)
        if tokens <= rc.reserved:
            return
        wanted = {}
        for name, g in self.groups.items():
            need = pages_for(tokens, g.page_size) - len(rc.tables[name])
            if need > self.pools[name].free_count:
                raise CacheError("capacity_exhausted",
                                 f"group '{name}': {need} pages wanted for request {request_id!r}, "
                                 f"{self.pools[name].free_count} free")
            wanted[name] = need
        for name, need in wanted.items():
            if need > 0:
                table = rc.tables[name]
                limit = self.groups[name].max_blocks
                if limit and len(table) + need > limit:
                    raise CacheError("invalid_reservation",
                                     f"group '{name}': {len(table) + need} blocks exceed the table's {limit}")
                for page in self.pools[name].take(need):
                    self._updates[name].append((rc.state_slot, len(table), page))
                    table.append(page)
        rc.reserved = max(rc.reserved, tokens)

    def commit(self, request_id: Hashable, new_length: int) -> None:
        """The request now holds ``new_length`` tokens; pages that its windows
        have passed go back to their pools."""
        rc = self.get(request_id)
        if new_length < rc.length or new_length > rc.reserved:
            raise CacheError("invalid_commit",
                             f"request {request_id!r}: length {rc.length} -> {new_length}, reserved {rc.reserved}")
        rc.length = new_length
        for name, g in self.groups.items():
            if g.window is None:
                continue
            table = rc.tables[name]
            dead = min(first_needed_block(new_length, g.window, g.page_size), len(table))
            gone = [p for p in table[:dead] if p >= 0]
            if gone:
                self.pools[name].give(gone)
                for i in range(dead):
                    if table[i] >= 0:
                        self._updates[name].append((rc.state_slot, i, -1))
                    table[i] = -1

    def release(self, request_id: Hashable) -> None:
        rc = self.requests.pop(request_id, None)
        if rc is None:
            return
        for name, table in rc.tables.items():
            self.pools[name].give([p for p in table if p >= 0])
        self.slots.give(rc.state_slot)

    # ---- checks (used by tests and by debug runs)
    def check_invariants(self) -> None:
        for name, pool in self.pools.items():
            held = [p for rc in self.requests.values() for p in rc.tables[name] if p >= 0]
            if len(held) != len(set(held)):
                raise AssertionError(f"group '{name}': a page is held twice")
            free = list(pool._free)
            if len(free) != len(set(free)) or set(free) & set(held):
                raise AssertionError(f"group '{name}': free list and tables overlap")
            if len(free) + len(held) != pool.num_pages:
                raise AssertionError(f"group '{name}': {pool.num_pages - len(free) - len(held)} pages lost")
        slots = [rc.state_slot for rc in self.requests.values()]
        if len(slots) != len(set(slots)):
            raise AssertionError("a state slot is held twice")
        if len(slots) + self.slots.free_count != self.slots.num_slots:
            raise AssertionError("a state slot is lost")
