"""Host-side accounting of cache pages and of fixed-size state slots.

A :class:`PagePool` owns the page ids of one cache group.  Pages are handed out LIFO, so
a page given back is the next one used again (no zeroing: lengths guard stale data).
Requests may *reserve* a number of pages at admission; a reserved page is not handed to
anyone else, so a request that was admitted with a full reservation can never run out
in the middle, which is the reference's no-deadlock rule in page units
(src/engine/kv.rs:36-67: ``reserve`` against ``free - sum(reserved)``, ``allocate`` from
the tail of the free list, ``release`` of everything at the end, src/engine/kv.rs:69-74).

:class:`StateSlots` gives each live request one exclusive slot index, reusable after
release (src/engine/recurrent.rs:6-38).
"""

from __future__ import annotations

from typing import Dict, Hashable, List, Optional


class OutOfPages(RuntimeError):
    """No page can be handed out without breaking another request's reservation."""


class PagePool:
    def __init__(self, num_pages: int, first_page: int = 0):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self.first_page = first_page
        # LIFO: the last element is handed out first; start so that low ids go first.
        self._free: List[int] = list(range(first_page + num_pages - 1, first_page - 1, -1))
        self._owner: Dict[int, Hashable] = {}
        self._quota: Dict[Hashable, int] = {}
        self._held: Dict[Hashable, int] = {}
        self._reserved_unallocated = 0

    # ---------------------------------------------------------------- queries
    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return len(self._owner)

    @property
    def available_to_reserve(self) -> int:
        return len(self._free) - self._reserved_unallocated

    def held_by(self, owner: Hashable) -> int:
        return self._held.get(owner, 0)

    def owner_of(self, page: int) -> Optional[Hashable]:
        return self._owner.get(page)

    # ---------------------------------------------------------------- reservations
    def reserve(self, owner: Hashable, pages: int) -> bool:
        """Set aside ``pages`` pages for ``owner`` (its peak simultaneous need)."""
        if owner in self._quota or owner in self._held:
            return False
        if pages > self.available_to_reserve:
            return False
        self._quota[owner] = pages
        self._held[owner] = 0
        self._reserved_unallocated += pages
        return True

    def register(self, owner: Hashable) -> None:
        """Admit ``owner`` without a reservation: its pages come on demand."""
        if owner in self._held:
            raise ValueError(f"{owner!r} is already registered in this pool")
        self._quota[owner] = 0
        self._held[owner] = 0

    # ---------------------------------------------------------------- pages
    def allocate(self, owner: Hashable) -> int:
        if owner not in self._held:
            raise KeyError(f"{owner!r} is not registered in this pool")
        held, quota = self._held[owner], self._quota[owner]
        if held < quota:
            self._reserved_unallocated -= 1   # drawing on the owner's own reservation
        elif self.available_to_reserve <= 0:
            raise OutOfPages(f"cache pool exhausted: {self.num_pages} pages, {len(self._free)} free, "
                             f"{self._reserved_unallocated} reserved for other requests")
        page = self._free.pop()
        self._owner[page] = owner
        self._held[owner] = held + 1
        return page

    def give_back(self, owner: Hashable, page: int) -> None:
        """Return one page while the owner lives on (a window has passed it)."""
        if self._owner.get(page) != owner:
            raise ValueError(f"page {page} is not held by {owner!r}")
        del self._owner[page]
        self._free.append(page)
        held = self._held[owner]
        self._held[owner] = held - 1
        if held <= self._quota[owner]:
            self._reserved_unallocated += 1   # the reservation covers the peak, so it is owed again

    def release(self, owner: Hashable, pages: List[int]) -> None:
        """The owner ends: return its remaining pages and drop its reservation."""
        if owner not in self._held:
            return
        for page in pages:
            if self._owner.get(page) != owner:
                raise ValueError(f"page {page} is not held by {owner!r}")
            del self._owner[page]
            self._free.append(page)
        held = self._held.pop(owner) - len(pages)
        quota = self._quota.pop(owner)
        if held != 0:
            raise ValueError(f"{owner!r} ended while still holding {held} pages not named in the release")
        self._reserved_unallocated -= max(0, quota - len(pages))

    def check(self) -> None:
        """Invariants: every page is free or owned, exactly once; reservations are honoured."""
        ids = list(self._free) + list(self._owner)
        if sorted(ids) != list(range(self.first_page, self.first_page + self.num_pages)):
            raise AssertionError("a page was lost, duplicated, or freed twice")
        if sum(self._held.values()) != len(self._owner):
            raise AssertionError("held counts disagree with ownership")
        expected = sum(max(0, self._quota[o] - self._held[o]) for o in self._held)
        if expected != self._reserved_unallocated or self._reserved_unallocated > len(self._free):
            raise AssertionError("reservation accounting is inconsistent")


class StateSlots:
    def __init__(self, capacity: int):
        if capacity <= 0:
            raise ValueError("state slots need a positive capacity")
        self.capacity = capacity
        self._free: List[int] = list(range(capacity - 1, -1, -1))
        self._slot: Dict[Hashable, int] = {}

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def allocate(self, owner: Hashable) -> Optional[int]:
        if owner in self._slot or not self._free:
            return None
        slot = self._free.pop()
        self._slot[owner] = slot
        return slot

    def get(self, owner: Hashable) -> Optional[int]:
        return self._slot.get(owner)

    def release(self, owner: Hashable) -> None:
        slot = self._slot.pop(owner, None)
        if slot is not None:
            self._free.append(slot)

    def check(self) -> None:
        ids = list(self._free) + list(self._slot.values())
        if sorted(ids) != list(range(self.capacity)):
            raise AssertionError("a state slot was lost, duplicated, or freed twice")
