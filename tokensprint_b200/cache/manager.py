"""Host-side bookkeeping of the paged cache and the per-request state slots.

Keys and values live in pages of `page_size` token positions.  Layers are sorted into
*groups* by what they need: a "full" group keeps every key of a request, a "window"
group may give a page back once every later query is further than `window` positions
from all of the page's keys.  Each group has a pool of pages of its own (its own device
tensors, its own free list); a request holds one block table per group.  Beside the
pages there are slots of fixed size for per-request state; a request takes one when it
is admitted and gives it back with its pages (an architecture without such state still
takes and returns the empty slot, so the life cycle is the same for all).

The reference's BlockManager (engine/generation/block_manager.py:154-404) is the model
for the arithmetic: pages popped from the head of a FIFO free list, freed pages appended
at the tail, `can_append`/`allocate_for_append` before a step, `deallocate` on finish
and on preemption.  Its prefix cache (hash -> block, reference counts) is left out:
every page here has exactly one owner.
"""

from __future__ import annotations

from collections import deque
import numpy as np
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence


class CacheError(RuntimeError):
    """A request asked for more pages or slots than are free, or broke the protocol."""


class OutOfPages(CacheError):
    pass


class OutOfSlots(CacheError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    kind: str  # "full" or "window"
    window: int = 0

    def __post_init__(self) -> None:
        if self.kind not in ("full", "window"):
            raise ValueError(f"cache group kind must be 'full' or 'window', got {self.kind!r}")
        if self.kind == "window" and self.window <= 0:
            raise ValueError("a window group needs a positive window")


class PagePool:
    """Pages 0..n-1 of one group: a FIFO free list and the owner of every page."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        self.free: deque[int] = deque(range(num_pages))
        self.owner: list[Optional[Hashable]] = [None] * num_pages

    @property
    def num_free(self) -> int:
        return len(self.free)

    def take(self, n: int, owner: Hashable) -> list[int]:
        if n > len(self.free):
            raise OutOfPages(f"{n} pages wanted, {len(self.free)} free")
        pages = [self.free.popleft() for _ in range(n)]
        for p in pages:
            if self.owner[p] is not None:
                raise CacheError(f"page {p} was on the free list while owned by {self.owner[p]!r}")
            self.owner[p] = owner
        return pages

    def give(self, pages: Sequence[int], owner: Hashable) -> None:
        for p in pages:
            if self.owner[p] != owner:
                raise CacheError(f"page {p} is given back by {owner!r} but owned by {self.owner[p]!r}")
            self.owner[p] = None
            self.free.append(p)


@dataclass
class RequestCache:
    """What one live request holds: a state slot and one block table per group."""

    request: Hashable
    slot: int
    tables: list[list[int]]  # per group; -1 where a page was given back (or never held)
    num_tokens: int = 0  # positions 0..num_tokens-1 have been given a place
    released: bool = False
    fresh_slot: bool = True  # the slot's state has not been zeroed on the device yet
    first_held: list[int] = field(default_factory=list)  # per group: first table index still held


class CacheManager:
    def __init__(
        self,
        groups: Sequence[GroupSpec],
        page_size: int,
        pages_per_group: Sequence[int],
        num_slots: int,
    ) -> None:
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        if len(groups) != len(pages_per_group):
            raise ValueError("one page count per group is needed")
        self.groups = list(groups)
        self._any_window = any(g.kind == "window" for g in self.groups)
        self.page_size = page_size
        self.pools = [PagePool(n) for n in pages_per_group]
        self.num_slots = num_slots
        self.free_slots: deque[int] = deque(range(num_slots))
        self.slot_owner: list[Optional[Hashable]] = [None] * num_slots
        self.live: dict[Hashable, RequestCache] = {}

    # -- admission and release -------------------------------------------------

    def admit(self, request: Hashable) -> RequestCache:
        if request in self.live:
            raise CacheError(f"request {request!r} is already live")
        if not self.free_slots:
            raise OutOfSlots(f"all {self.num_slots} state slots are taken")
        slot = self.free_slots.popleft()
        self.slot_owner[slot] = request
        rc = RequestCache(request, slot, [[] for _ in self.groups], first_held=[0] * len(self.groups))
        self.live[request] = rc
        return rc

    def free(self, rc: RequestCache) -> None:
        """Gives back every page and the slot (request finished, aborted or preempted)."""
        if rc.released:
            raise CacheError(f"request {rc.request!r} was already freed")
        if self.live.get(rc.request) is not rc:
            raise CacheError(f"request {rc.request!r} is not live here")
        for g, pool in enumerate(self.pools):
            held = [p for p in rc.tables[g] if p >= 0]
            pool.give(list(reversed(held)), rc.request)
            rc.tables[g] = []
        if self.slot_owner[rc.slot] != rc.request:
            raise CacheError(f"slot {rc.slot} is not owned by {rc.request!r}")
        self.slot_owner[rc.slot] = None
        self.free_slots.append(rc.slot)
        rc.released = True
        rc.num_tokens = 0
        del self.live[rc.request]

    # -- growth ------------------------------------------------------------------

    def _first_needed_page(self, g: int, start: int) -> int:
        """Index of the first page a query at position `start` (or later) can still read."""
        spec = self.groups[g]
        if spec.kind != "window":
            return 0
        oldest_key = max(0, start - spec.window + 1)
        return oldest_key // self.page_size

    def _plan(self, rc: RequestCache, start: int, new_len: int) -> list[tuple[int, int]]:
        """Per group: (pages that can go first, pages to take) for tokens start..new_len-1."""
        if new_len < rc.num_tokens or start > new_len:
            raise CacheError(f"cannot shrink request {rc.request!r} from {rc.num_tokens} to {new_len}")
        total = -(-new_len // self.page_size)
        plan = []
        for g in range(len(self.groups)):
            table = rc.tables[g]
            first = self._first_needed_page(g, start)
            droppable = sum(1 for p in table[rc.first_held[g] : min(first, len(table))] if p >= 0)
            plan.append((droppable, max(0, total - len(table))))
        return plan

    def _fits_as_is(self, rc: RequestCache, new_len: int) -> bool:
        """The common case of a decode step: no group has a window and the pages held already
        cover new_len positions, so nothing is taken and nothing given back."""
        if self._any_window or rc.released or new_len < rc.num_tokens:
            return False
        total = -(-new_len // self.page_size)
        return all(len(t) >= total for t in rc.tables)

    def can_extend(self, rc: RequestCache, start: int, new_len: int) -> bool:
        """Whether `extend` would succeed right now."""
        if self._fits_as_is(rc, new_len) and start <= new_len:
            return True
        for pool, (drop, take) in zip(self.pools, self._plan(rc, start, new_len)):
            if take > pool.num_free + drop:
                return False
        return True

    def extend(self, rc: RequestCache, start: int, new_len: int) -> None:
        """Makes room for positions up to new_len-1; the step's first query sits at `start`.

        Window groups first give back the pages that no query from `start` on can see.
        Either everything is done or, on OutOfPages, nothing was changed.
        """
        if rc.released:
            raise CacheError(f"request {rc.request!r} was freed")
        if self._fits_as_is(rc, new_len) and start <= new_len:
            rc.num_tokens = new_len
            return
        plan = self._plan(rc, start, new_len)
        for pool, (drop, take) in zip(self.pools, plan):
            if take > pool.num_free + drop:
                raise OutOfPages(f"request {rc.request!r}: {take} pages wanted, {pool.num_free + drop} can be had")
        for g, pool in enumerate(self.pools):
            table = rc.tables[g]
            first = min(self._first_needed_page(g, start), len(table))
            gone = [i for i in range(rc.first_held[g], first) if table[i] >= 0]
            if gone:
                pool.give([table[i] for i in gone], rc.request)
                for i in gone:
                    table[i] = -1
            rc.first_held[g] = max(rc.first_held[g], first)
            take = plan[g][1]
            if take:
                table.extend(pool.take(take, rc.request))
        rc.num_tokens = max(rc.num_tokens, new_len)

    # -- what a step needs ---------------------------------------------------------

    def slots_for(self, rc: RequestCache, g: int, start: int, count: int) -> "np.ndarray":
        """Flat cache slots (page * page_size + offset) of positions start..start+count-1."""
        P = self.page_size
        first = start // P
        pages = np.asarray(rc.tables[g][first : (start + count - 1) // P + 1], dtype=np.int64)
        positions = np.arange(start, start + count, dtype=np.int64)
        held = pages[positions // P - first]
        if held.size and held.min() < 0:
            pos = int(positions[int(np.argmax(held < 0))])
            raise CacheError(f"request {rc.request!r}: position {pos} lies in a page that was given back")
        return held * P + positions % P

    # -- checks --------------------------------------------------------------------

    def pages_in_use(self, g: int = 0) -> int:
        return self.pools[g].num_pages - self.pools[g].num_free

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; the same for slots."""
        for g, pool in enumerate(self.pools):
            free = list(pool.free)
            if len(set(free)) != len(free):
                raise CacheError(f"group {g}: a page is on the free list twice")
            held: dict[int, Hashable] = {}
            for rc in self.live.values():
                for p in rc.tables[g]:
                    if p < 0:
                        continue
                    if p in held:
                        raise CacheError(f"group {g}: page {p} is held by {held[p]!r} and {rc.request!r}")
                    held[p] = rc.request
            for p in free:
                if p in held or pool.owner[p] is not None:
                    raise CacheError(f"group {g}: page {p} is free and held")
            for p, owner in held.items():
                if pool.owner[p] != owner:
                    raise CacheError(f"group {g}: page {p} owner record {pool.owner[p]!r} != {owner!r}")
            if len(free) + len(held) != pool.num_pages:
                raise CacheError(f"group {g}: {pool.num_pages - len(free) - len(held)} pages are lost")
        free_slots = list(self.free_slots)
        if len(set(free_slots)) != len(free_slots):
            raise CacheError("a state slot is on the free list twice")
        held_slots = {rc.slot for rc in self.live.values()}
        if len(held_slots) != len(self.live):
            raise CacheError("two requests hold the same state slot")
        if held_slots & set(free_slots):
            raise CacheError("a state slot is free and held")
        if len(held_slots) + len(free_slots) != self.num_slots:
            raise CacheError("a state slot is lost")
