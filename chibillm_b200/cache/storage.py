"""Device arrays behind the cache manager, and the views that mixers get.

Keys and values of a group: one array each per run step of the group,
``[pages, kv_heads, page_size, head_dim]`` in the runtime's activation type, so
the ``page_size * head_dim`` values of one (page, head) are contiguous.
Fixed state: one array per declared name and run step, ``[slots, *shape]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import FixedStateNeed, PagedKVNeed, Runtime
from .manager import CacheError, GroupLayout


@dataclass
class PagedKVView:
    """What an attention-like mixer sees of the cache for one run step."""

    group: str
    keys: torch.Tensor
    values: torch.Tensor
    page_size: int
    writes: bool                 # False: this run step reads another step's cache


@dataclass
class FixedStateView:
    """Per-request arrays of one run step, indexed by state slot."""

    arrays: Dict[str, torch.Tensor]


@dataclass(frozen=True)
class CachePlan:
    groups: Tuple[GroupLayout, ...]
    # per run step: ("paged", group, entry, writes) | ("state", need) | None
    steps: Tuple[Optional[tuple], ...]


def group_name(need: PagedKVNeed) -> str:
    base = f"kv{need.num_kv_heads}x{need.head_dim}"
    return base if need.window is None else f"{base}w{need.window}"


def plan_cache(needs: Sequence[object], cache_of: Sequence[Optional[int]], page_size: int,
               pool_tokens: int, max_positions: int = 0) -> CachePlan:
    """Sort the run steps' needs into groups.  ``pool_tokens`` is how many
    tokens every group's pool can hold; it is rounded up to whole pages.
    ``max_positions`` (the model's limit; default: the pool's size) bounds the
    logical blocks of one request, which is the width of the device tables."""
    if page_size <= 0 or pool_tokens <= 0:
        raise CacheError("invalid_configuration", "page_size and pool_tokens must be positive")
    num_pages = (pool_tokens + page_size - 1) // page_size
    entries: Dict[str, int] = {}
    needs_of: Dict[str, PagedKVNeed] = {}
    steps: List[Optional[tuple]] = []
    for i, need in enumerate(needs):
        src = cache_of[i]
        if src is not None:
            if not (0 <= src < i) or steps[src] is None or steps[src][0] != "paged" or not steps[src][3]:
                raise CacheError("invalid_configuration",
                                 f"run step {i} reads the cache of step {src}, which owns no paged cache")
            mine = need
            theirs = needs_of[steps[src][1]]
            if not isinstance(mine, PagedKVNeed) or (mine.num_kv_heads, mine.head_dim) != (
                    theirs.num_kv_heads, theirs.head_dim):
                raise CacheError("invalid_configuration",
                                 f"run step {i} cannot read the cache of step {src}: shapes differ")
            if mine.window != theirs.window:
                # the owner's window decides which pages are given back; a reader that looks
                # further back would meet pages that are gone
                raise CacheError("invalid_configuration",
                                 f"run step {i} (window {mine.window}) cannot read the cache of step {src} "
                                 f"(window {theirs.window}): the windows differ")
            steps.append(("paged", steps[src][1], steps[src][2], False))
        elif isinstance(need, PagedKVNeed):
            name = group_name(need)
            needs_of[name] = need
            entry = entries.get(name, 0)
            entries[name] = entry + 1
            steps.append(("paged", name, entry, True))
        elif isinstance(need, FixedStateNeed):
            steps.append(("state", need))
        elif need is None:
            steps.append(None)
        else:
            raise CacheError("invalid_configuration", f"run step {i}: unknown cache need {need!r}")
    max_blocks = (max(max_positions, 1) + page_size - 1) // page_size if max_positions else num_pages
    groups = tuple(GroupLayout(name, n.num_kv_heads, n.head_dim, n.window, page_size, num_pages,
                               entries[name], max_blocks) for name, n in needs_of.items())
    return CachePlan(groups, tuple(steps))


class CacheStorage:
    def __init__(self, plan: CachePlan, runtime: Runtime, num_slots: int):
        self.plan = plan
        self.runtime = runtime
        self.num_slots = num_slots
        self.keys: Dict[str, torch.Tensor] = {}
        self.values: Dict[str, torch.Tensor] = {}
        for g in plan.groups:
            shape = (g.num_entries, g.num_pages, g.num_kv_heads, g.page_size, g.head_dim)
            self.keys[g.name] = torch.zeros(shape, dtype=runtime.dtype, device=runtime.device)
            self.values[g.name] = torch.zeros(shape, dtype=runtime.dtype, device=runtime.device)
        # the block tables' mirror on the device: row = a request's state slot
        self.tables: Dict[str, torch.Tensor] = {
            g.name: torch.full((num_slots, max(g.max_blocks, 1)), -1, dtype=torch.int32, device=runtime.device)
            for g in plan.groups}
        self.views: List[object] = []
        self._state_arrays: List[torch.Tensor] = []
        page_sizes = {g.name: g.page_size for g in plan.groups}
        for step in plan.steps:
            if step is None:
                self.views.append(None)
            elif step[0] == "paged":
                _, name, entry, writes = step
                self.views.append(PagedKVView(name, self.keys[name][entry], self.values[name][entry],
                                              page_sizes[name], writes))
            else:
                arrays = {}
                for aname, shape, dtype in step[1].arrays:
                    t = torch.zeros((num_slots,) + tuple(shape), dtype=dtype, device=runtime.device)
                    arrays[aname] = t
                    self._state_arrays.append(t)
                self.views.append(FixedStateView(arrays))

    def zero_state_slot(self, slot: int) -> None:
        for t in self._state_arrays:
            t[slot].zero_()

    def poison(self, value: float = float("nan")) -> None:
        """Fill every page with a marker (tests use NaN so that a read of a
        position that was never written shows)."""
        for t in list(self.keys.values()) + list(self.values.values()):
            t.fill_(value)

    def bytes(self) -> int:
        total = 0
        for t in list(self.keys.values()) + list(self.values.values()) + self._state_arrays:
            total += t.numel() * t.element_size()
        return total
