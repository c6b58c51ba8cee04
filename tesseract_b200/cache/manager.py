"""The cache manager: pages with a block table per request, in groups, plus state slots.

Run entries with the same cache need (same kv heads, head size and window; or the same
fixed-size state) form a *group*.  A paged group has its own page pool and one block
table per live request, shared by the group's entries (each entry has its own storage
``[pages + 1, *need.page_shape(page_size)]`` addressed by the same page ids, for keys and
values ``[pages + 1, 2, kv_heads, page_size, head_dim]``; page 0 is a scratch page that no
request owns, for padded rows).  A state group has storage
``[entries, slots + 1, *shape]`` addressed by the request's state slot (the last slot is scratch).  Every live request
holds one state slot whether or not the model has state groups
(src/engine/recurrent.rs:6-38; groups after src/engine/state.rs:31-132).

Pages are allocated when a request's positions first reach them, returned one by one
once a sliding window has passed them, and all returned when the request ends; returned
pages are handed out again first.  ``admit`` with ``reserve_tokens`` sets aside the
request's peak need in every group (src/engine/kv.rs:36-51), so an admitted request
cannot run out; without a reservation pages come on demand and ``extend`` raises
:class:`OutOfPages` when none is left.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheBinding, PagedNeed, StateNeed
from .pages import OutOfPages, PagePool, StateSlots


@dataclass
class _Group:
    need: object
    entries: List[int]
    pool: Optional[PagePool] = None
    storage: Optional[torch.Tensor] = None
    tables: Optional[np.ndarray] = None       # int32 [slots, columns]; 0 where no page is held


@dataclass
class _Request:
    slot: int
    length: int = 0                            # tokens whose keys/values are stored
    pages: List[Dict[int, int]] = field(default_factory=list)   # per paged group: logical index -> page id
    first_live: List[int] = field(default_factory=list)         # per group: lowest logical page still held


class CacheManager:
    def __init__(self, needs: Sequence[Optional[object]], cache_of: Sequence[Optional[int]], *, num_pages: int,
                 page_size: int, max_requests: int, dtype: torch.dtype, device, max_step_tokens: int = 1,
                 allocate_storage: bool = True):
        if len(needs) != len(cache_of):
            raise ValueError("needs and cache_of must describe the same run entries")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.max_step_tokens = max(1, max_step_tokens)
        self.dtype = dtype
        self.device = device
        self.slots = StateSlots(max_requests)
        self.scratch_slot = max_requests       # one state slot more than requests: padded rows point here
        self.groups: List[_Group] = []
        self._group_of_entry: List[Optional[int]] = [None] * len(needs)
        self._index_in_group: List[Optional[int]] = [None] * len(needs)
        by_need: Dict[object, int] = {}
        for entry, need in enumerate(needs):
            if need is None:
                continue
            if need not in by_need:
                by_need[need] = len(self.groups)
                self.groups.append(_Group(need=need, entries=[]))
            group = by_need[need]
            self._group_of_entry[entry] = group
            self._index_in_group[entry] = len(self.groups[group].entries)
            self.groups[group].entries.append(entry)
        for group in self.groups:
            need = group.need
            if isinstance(need, PagedNeed):
                group.pool = PagePool(num_pages, first_page=1)
                group.tables = np.zeros((max_requests, 8), dtype=np.int32)
                if allocate_storage:      # the need says what a page looks like; page 0 is the scratch page
                    group.storage = torch.zeros(
                        (len(group.entries), num_pages + 1, *need.page_shape(page_size)),
                        dtype=need.dtype or dtype, device=device)
            elif isinstance(need, StateNeed):
                if allocate_storage:
                    group.storage = torch.zeros((len(group.entries), max_requests + 1, *need.shape),
                                                dtype=need.dtype, device=device)
            else:
                raise TypeError(f"a cache need is a PagedNeed or a StateNeed, got {need!r}")
        self.bindings: List[Optional[CacheBinding]] = []
        for entry, need in enumerate(needs):
            source = entry if cache_of[entry] is None else cache_of[entry]
            group = self._group_of_entry[source]
            if group is None:
                self.bindings.append(None)
                continue
            g = self.groups[group]
            storage = g.storage[self._index_in_group[source]] if g.storage is not None else None
            self.bindings.append(CacheBinding(group=group, storage=storage, writes=cache_of[entry] is None,
                                              page_size=page_size if g.pool is not None else 0))
        self._requests: Dict[Hashable, _Request] = {}
        self.pages_reused = 0          # pages handed out that an earlier owner had given back
        self._ever_used: List[set] = [set() for _ in self.groups]

    # ------------------------------------------------------------------ sizes
    def pages_for(self, group: _Group, tokens: int) -> int:
        """Peak pages a request of ``tokens`` tokens holds in ``group`` at any one time."""
        total = -(-tokens // self.page_size)
        window = getattr(group.need, "window", None)
        if window:
            live = -(-(window - 1 + self.max_step_tokens) // self.page_size) + 1
            return min(total, live)
        return total

    def bytes_per_token(self) -> int:
        total = 0
        for g in self.groups:
            if g.pool is not None:
                elem = torch.empty((), dtype=g.need.dtype or self.dtype).element_size()
                page = 1
                for extent in g.need.page_shape(self.page_size):
                    page *= extent
                total += len(g.entries) * (page // self.page_size) * elem
        return total

    # ------------------------------------------------------------------ lifecycle
    def can_admit(self, reserve_tokens: Optional[int]) -> bool:
        if self.slots.free_slots == 0:
            return False
        if reserve_tokens is None:
            return True
        return all(g.pool is None or self.pages_for(g, reserve_tokens) <= g.pool.available_to_reserve
                   for g in self.groups)

    def admit(self, request: Hashable, reserve_tokens: Optional[int] = None) -> bool:
        """Give ``request`` a state slot and (optionally) reserve its pages; False if it does not fit now."""
        if request in self._requests:
            raise ValueError(f"request {request!r} is already live")
        if not self.can_admit(reserve_tokens):
            return False
        slot = self.slots.allocate(request)
        assert slot is not None
        for g in self.groups:
            if g.pool is None:
                if g.storage is not None:
                    g.storage[:, slot].zero_()       # a new request starts from empty state
                continue
            if reserve_tokens is None:
                g.pool.register(request)
            else:
                ok = g.pool.reserve(request, self.pages_for(g, reserve_tokens))
                assert ok
            g.tables[slot, :] = 0
        self._requests[request] = _Request(slot=slot, pages=[{} for _ in self.groups],
                                           first_live=[0 for _ in self.groups])
        return True

    def is_live(self, request: Hashable) -> bool:
        return request in self._requests

    def length(self, request: Hashable) -> int:
        return self._requests[request].length

    def slot(self, request: Hashable) -> int:
        return self._requests[request].slot

    def extend(self, request: Hashable, new_tokens: int) -> None:
        """Make sure pages exist for positions ``[length, length + new_tokens)`` in every paged group."""
        state = self._requests[request]
        last = (state.length + new_tokens - 1) // self.page_size
        for index, g in enumerate(self.groups):
            if g.pool is None:
                continue
            held = state.pages[index]
            if g.tables.shape[1] <= last:
                columns = max(last + 1, 2 * g.tables.shape[1])
                grown = np.zeros((self.max_requests, columns), dtype=np.int32)
                grown[:, :g.tables.shape[1]] = g.tables
                g.tables = grown
            first_needed = self._first_needed_page(g, state.length)
            for logical in range(max(first_needed, state.first_live[index]), last + 1):
                if logical in held:
                    continue
                page = g.pool.allocate(request)       # may raise OutOfPages
                if page in self._ever_used[index]:
                    self.pages_reused += 1
                self._ever_used[index].add(page)
                held[logical] = page
                g.tables[state.slot, logical] = page

    def commit(self, request: Hashable, new_tokens: int) -> None:
        """The step stored ``new_tokens`` more tokens; give back pages a window has passed."""
        state = self._requests[request]
        state.length += new_tokens
        for index, g in enumerate(self.groups):
            if g.pool is None or not getattr(g.need, "window", None):
                continue
            first_needed = self._first_needed_page(g, state.length)
            held = state.pages[index]
            for logical in range(state.first_live[index], first_needed):
                page = held.pop(logical, None)
                if page is not None:
                    g.pool.give_back(request, page)
                    g.tables[state.slot, logical] = 0
            state.first_live[index] = max(state.first_live[index], first_needed)

    def release(self, request: Hashable) -> None:
        """The request ends: all its pages and its state slot go back."""
        state = self._requests.pop(request, None)
        if state is None:
            return
        for index, g in enumerate(self.groups):
            if g.pool is None:
                continue
            g.pool.release(request, list(state.pages[index].values()))
            g.tables[state.slot, :] = 0
        self.slots.release(request)

    def _first_needed_page(self, group: _Group, next_position: int) -> int:
        """Lowest logical page that a query at ``next_position`` or later can still read."""
        window = getattr(group.need, "window", None)
        if not window:
            return 0
        return max(0, next_position - window + 1) // self.page_size

    # ------------------------------------------------------------------ views
    def block_table_rows(self, group_index: int, slots: Sequence[int], columns: int) -> np.ndarray:
        """int32 ``[len(slots), columns]`` copy of the block tables of the given state slots."""
        tables = self.groups[group_index].tables
        have = min(columns, tables.shape[1])
        out = np.zeros((len(slots), columns), dtype=np.int32)
        out[:, :have] = tables[np.asarray(slots, dtype=np.int64), :have]
        return out

    def pages_of(self, request: Hashable, group_index: int = 0) -> Dict[int, int]:
        return dict(self._requests[request].pages[group_index])

    def used_pages(self) -> int:
        return sum(g.pool.used_pages for g in self.groups if g.pool is not None)

    def check(self) -> None:
        self.slots.check()
        for index, g in enumerate(self.groups):
            if g.pool is None:
                continue
            g.pool.check()
            seen = set()
            for request, state in self._requests.items():
                for page in state.pages[index].values():
                    if page in seen:
                        raise AssertionError(f"page {page} is held twice")
                    seen.add(page)
                    if g.pool.owner_of(page) != request:
                        raise AssertionError(f"page {page} ownership disagrees")
            if len(seen) != g.pool.used_pages:
                raise AssertionError("pool holds pages that no request's table names")
