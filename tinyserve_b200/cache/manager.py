"""Host bookkeeping of the paged cache and of the per-request state slots.

Keys and values live in pages of ``page_size`` tokens.  Layers with the same needs
form a *group* (all keys; a window of keys); every group has its own page pool and
every request one block table per group.  Page 0 of a pool is the null page: it is
never handed out, and padded or released block-table entries point at it
(serve.py:206, 1849-1850).  Pages are handed out from the head of a queue and come
back at its tail (serve.py:394, 445-448).  A request's pages come back when it ends
(serve.py:441-449) or, in a window group, as soon as no later query can see them.

Beside the pages there is a pool of fixed-size state slots, one per live request;
a mixer that keeps state of its own finds it at ``state[slot]``.

tinyserve's manager (serve.py:188-449) has one pool, no groups and no slots; its
prefix cache is not part of this engine."""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field


class CacheError(RuntimeError):
    pass


class PagePool:
    """Free queue and ownership of the pages of one group."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise CacheError("a page pool needs the null page and at least one more page")
        self.num_pages = num_pages
        self.free: OrderedDict = OrderedDict((i, None) for i in range(1, num_pages))
        self.owner: dict = {}

    @property
    def num_free(self) -> int:
        return len(self.free)

    @property
    def num_usable(self) -> int:
        return self.num_pages - 1

    def take(self, owner) -> int:
        page, _ = self.free.popitem(last=False)
        self.owner[page] = owner
        return page

    def give_back(self, page: int, owner) -> None:
        if page == 0:
            raise CacheError("the null page cannot be freed")
        if self.owner.get(page, None) != owner or page in self.free:
            raise CacheError(f"page {page} freed by {owner!r} who does not hold it")
        del self.owner[page]
        self.free[page] = None


@dataclass
class GroupSpec:
    kind: str                    # "full" or "window"
    window: int = 0


@dataclass
class _RequestPages:
    pages: list = field(default_factory=list)   # logical page -> physical page (0 = released)
    first_live: int = 0                          # logical pages below this are released
    synced: int = 0                              # leading entries that the device's copy of the row holds
    dirty: list = field(default_factory=list)    # entries below ``synced`` that changed since (released pages)


class SlotPool:
    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self.free = list(range(num_slots - 1, -1, -1))
        self.owner: dict = {}

    def take(self, owner) -> int:
        if not self.free:
            raise CacheError("no state slot is free")
        slot = self.free.pop()
        self.owner[slot] = owner
        return slot

    def give_back(self, slot: int, owner) -> None:
        if self.owner.get(slot) != owner:
            raise CacheError(f"slot {slot} freed by {owner!r} who does not hold it")
        del self.owner[slot]
        self.free.append(slot)


@dataclass
class _Request:
    slot: int
    num_computed: int = 0
    groups: list = field(default_factory=list)
    fresh: bool = True           # no token committed yet: state must start at zero


class CacheManager:
    def __init__(self, groups, num_pages, page_size: int, num_slots: int):
        """``groups``: list of GroupSpec; ``num_pages``: pages per pool (an int or one per group)."""
        if page_size <= 0 or page_size & (page_size - 1):
            raise CacheError("page_size must be a power of two")
        self.page_size = page_size
        self.groups = list(groups)
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        self.pools = [PagePool(n) for n in counts]
        self.slots = SlotPool(num_slots)
        self.requests: dict = {}

    # ------------------------------------------------------------------ requests
    def begin(self, rid) -> int:
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already live")
        slot = self.slots.take(rid)
        self.requests[rid] = _Request(slot, 0, [_RequestPages() for _ in self.groups])
        return slot

    def is_live(self, rid) -> bool:
        return rid in self.requests

    def can_begin(self) -> bool:
        return bool(self.slots.free)

    def num_computed(self, rid) -> int:
        return self.requests[rid].num_computed

    def slot(self, rid) -> int:
        return self.requests[rid].slot

    def is_fresh(self, rid) -> bool:
        return self.requests[rid].fresh

    def free(self, rid) -> None:
        """Give back every page and the slot of ``rid``."""
        req = self.requests.pop(rid, None)
        if req is None:
            raise CacheError(f"request {rid!r} is not live")
        for pool, rp in zip(self.pools, req.groups):
            for page in reversed(rp.pages):
                if page:
                    pool.give_back(page, rid)
        self.slots.give_back(req.slot, rid)

    # ------------------------------------------------------------------ pages
    def _first_needed_page(self, g: int, first_query_pos: int) -> int:
        """Lowest logical page that a query at ``first_query_pos`` or later can see."""
        spec = self.groups[g]
        if spec.kind != "window":
            return 0
        lowest_key = max(0, first_query_pos - spec.window + 1)
        return lowest_key // self.page_size

    def pages_needed(self, rid, num_new: int) -> list:
        """New pages per group so that ``num_new`` more tokens fit."""
        req = self.requests[rid]
        total = req.num_computed + num_new
        want = -(-total // self.page_size)
        return [max(0, want - len(rp.pages)) for rp in req.groups]

    def allocate(self, rid, num_new: int) -> bool:
        """Make room for ``num_new`` tokens after the computed ones: all or nothing."""
        req = self.requests[rid]
        need = self.pages_needed(rid, num_new)
        # a window group may release pages before it takes new ones
        for g, rp in enumerate(req.groups):
            self._release_behind(rid, g, rp, req.num_computed)
        if any(n > pool.num_free for n, pool in zip(need, self.pools)):
            return False
        for n, pool, rp in zip(need, self.pools, req.groups):
            for _ in range(n):
                rp.pages.append(pool.take(rid))
        return True

    def _release_behind(self, rid, g, rp, num_computed) -> None:
        first = min(self._first_needed_page(g, num_computed), len(rp.pages))
        for logical in range(rp.first_live, first):
            page = rp.pages[logical]
            if page:
                self.pools[g].give_back(page, rid)
                rp.pages[logical] = 0
                if logical < rp.synced:
                    rp.dirty.append(logical)
        rp.first_live = max(rp.first_live, first)

    def commit(self, rid, num_new: int) -> None:
        """``num_new`` tokens were run: they are computed now.  Window groups give back
        the pages that no later query can see."""
        req = self.requests[rid]
        req.num_computed += num_new
        req.fresh = False
        for g, rp in enumerate(req.groups):
            if req.num_computed > len(rp.pages) * self.page_size:
                raise CacheError(f"request {rid!r} ran past its pages")
            self._release_behind(rid, g, rp, req.num_computed)

    def block_table(self, rid, g: int) -> list:
        return self.requests[rid].groups[g].pages

    def table_updates(self, rid, g: int):
        """What the device's copy of this request's block-table row lacks: ([(index, page), ...],
        receipt).  Nothing is marked as sent until ``table_synced(receipt)``: a packed step that is
        never launched leaves the entries to be sent again."""
        rp = self.requests[rid].groups[g]
        changes = [(i, rp.pages[i]) for i in rp.dirty]
        changes += [(i, rp.pages[i]) for i in range(rp.synced, len(rp.pages))]
        return changes, (rp, len(rp.pages), len(rp.dirty))

    @staticmethod
    def table_synced(receipt) -> None:
        rp, length, num_dirty = receipt
        rp.synced = max(rp.synced, length)
        del rp.dirty[:num_dirty]

    def slot_of_position(self, rid, g: int, pos: int) -> int:
        page = self.requests[rid].groups[g].pages[pos // self.page_size]
        if page == 0:
            raise CacheError(f"position {pos} of {rid!r} lies on a released page")
        return page * self.page_size + pos % self.page_size

    # ------------------------------------------------------------------ figures
    def num_free_pages(self, g: int = 0) -> int:
        return self.pools[g].num_free

    def usage(self) -> float:
        used = sum(p.num_usable - p.num_free for p in self.pools)
        return used / max(1, sum(p.num_usable for p in self.pools))

    def check_invariants(self) -> None:
        """No page lost, held twice or both free and held; slots likewise."""
        for g, pool in enumerate(self.pools):
            held = []
            for rid, req in self.requests.items():
                for page in req.groups[g].pages:
                    if page:
                        held.append(page)
                        if pool.owner.get(page) != rid:
                            raise CacheError(f"group {g}: page {page} owner mismatch")
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page is held twice")
            if set(held) & set(pool.free):
                raise CacheError(f"group {g}: a page is both free and held")
            if 0 in pool.free or 0 in held:
                raise CacheError(f"group {g}: the null page left its place")
            if len(held) + len(pool.free) != pool.num_usable:
                raise CacheError(f"group {g}: {pool.num_usable - len(held) - len(pool.free)} pages lost")
            if set(pool.owner) != set(held):
                raise CacheError(f"group {g}: owner table and block tables differ")
        slots = [r.slot for r in self.requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self.slots.free):
            raise CacheError("a state slot is held twice")
        if len(slots) + len(self.slots.free) != self.slots.num_slots:
            raise CacheError("a state slot was lost")
