"""Cache manager: pages, block tables and state slots, on the host.

Run entries of a model (see ``parts.spec.RunEntry``) that keep the same kind
of cache form a *group*.  A paged group (``PagedKV``) has a page pool of its
own; a request has one block table per paged group, and one page id stands
for that page in every entry of the group.  A group with a window gives
pages back as soon as every later query is past them; a group without keeps
them until the request ends.  A fixed-state group (``FixedState``) keeps its
state in the request's *slot*; slots exist for every request, whether or not
the architecture has such state.

Lengths are committed after a step succeeded (as the reference grows
``cache->length`` only then, engine/src/gpt2_gpu.cu:305,364); slots past the
length are never read, so nothing is cleared on reuse
(engine/src/gpt2_gpu.cu:173-179).

This module holds no device memory: ``cache.storage`` does.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..parts.spec import FixedState, NoCache, PagedKV
from .pages import PageError, PagePool

NO_PAGE = -1


@dataclass
class CacheGroup:
    index: int
    need: object                       # PagedKV or FixedState
    entries: list                      # run-entry indices that own a cache in this group
    pool: PagePool | None = None       # paged groups only
    max_blocks: int = 0
    table: np.ndarray | None = None    # [max_requests, max_blocks] int32, NO_PAGE where nothing is held

    @property
    def paged(self) -> bool:
        return isinstance(self.need, PagedKV)


@dataclass
class _Request:
    slot: int
    length: int = 0                    # committed tokens
    reserved: int = 0                  # tokens pages are reserved for (>= length)
    first_block: dict = field(default_factory=dict)   # group -> first block still held
    n_blocks: dict = field(default_factory=dict)      # group -> blocks ever appended


def group_entries(needs) -> list:
    """Group run entries by what they keep.  ``needs[i]`` is the need of run
    entry i, or None if the entry reads another entry's cache."""
    groups: dict = {}
    for entry, need in enumerate(needs):
        if need is None or isinstance(need, NoCache):
            continue
        groups.setdefault(need, []).append(entry)
    return [(need, entries) for need, entries in groups.items()]


class CacheManager:
    def __init__(self, needs, page_size: int, n_pages, max_requests: int, max_tokens_per_request: int):
        """``n_pages``: pages of every paged group's pool (an int, or a list per group)."""
        if page_size <= 0 or max_requests <= 0 or max_tokens_per_request <= 0:
            raise ValueError("page_size, max_requests and max_tokens_per_request must be positive")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_tokens_per_request = int(max_tokens_per_request)
        self.groups: list[CacheGroup] = []
        self.entry_group: dict[int, tuple] = {}        # run entry -> (group index, index within the group)
        max_blocks = -(-self.max_tokens_per_request // self.page_size)
        for index, (need, entries) in enumerate(group_entries(needs)):
            group = CacheGroup(index, need, entries)
            if group.paged:
                count = n_pages[index] if isinstance(n_pages, (list, tuple)) else n_pages
                group.pool = PagePool(int(count))
                group.max_blocks = max_blocks
                group.table = np.full((self.max_requests, max_blocks), NO_PAGE, dtype=np.int32)
            self.groups.append(group)
            for position, entry in enumerate(entries):
                self.entry_group[entry] = (index, position)
        self._free_slots = list(range(self.max_requests - 1, -1, -1))
        self._requests: dict[int, _Request] = {}
        self._paged = [(g.index, g.paged) for g in self.groups]     # what pages_needed walks
        self.freed_by_window = 0
        # Called with (group index, page ids) whenever pages go back to a pool: the device side
        # of a debugging engine overwrites them, so that a stale block-table row shows.
        self.on_free = None

    # ---- slots ------------------------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def open(self) -> int | None:
        """A slot for a new request, or None if all are taken."""
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._requests[slot] = _Request(slot, first_block={g.index: 0 for g in self.groups if g.paged},
                                        n_blocks={g.index: 0 for g in self.groups if g.paged})
        return slot

    def close(self, slot: int) -> None:
        """Give back everything the request holds: its pages in every group and its slot."""
        request = self._take(slot)
        for group in self.groups:
            if not group.paged:
                continue
            row = group.table[slot]
            held = [int(p) for p in row[request.first_block[group.index]:request.n_blocks[group.index]] if p != NO_PAGE]
            group.pool.free(held, slot)
            self._freed(group, held)
            row[:] = NO_PAGE
        del self._requests[slot]
        self._free_slots.append(slot)

    def is_open(self, slot: int) -> bool:
        return slot in self._requests

    def _take(self, slot: int) -> _Request:
        try:
            return self._requests[slot]
        except KeyError:
            raise PageError(f"slot {slot} holds no request") from None

    def length(self, slot: int) -> int:
        return self._take(slot).length

    # ---- pages ------------------------------------------------------------------------------
    def _blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def pages_needed(self, slot: int, n_new: int) -> list:
        """Pages each paged group must add so the request can hold ``n_new`` more tokens."""
        request = self._take(slot)
        target = -(-(request.length + n_new) // self.page_size)
        held = request.n_blocks
        return [(target - held[g] if target > held[g] else 0) if paged else 0 for g, paged in self._paged]

    def room_for(self, slot: int, n_new: int, spare: list | None = None) -> list | None:
        """``pages_needed(slot, n_new)`` if ``reserve`` would succeed, else None.  ``spare[g]``
        pages of group g count as already taken."""
        needed = self.pages_needed(slot, n_new)
        for group, count in zip(self.groups, needed):
            if count > 0 and count > group.pool.available - (spare[group.index] if spare else 0):
                return None
        return needed if self._take(slot).length + n_new <= self.max_tokens_per_request else None

    def can_reserve(self, slot: int, n_new: int, spare: list | None = None) -> bool:
        """Would ``reserve`` succeed?  ``spare[g]`` pages of group g count as already taken."""
        return self.room_for(slot, n_new, spare) is not None

    def reserve(self, slot: int, n_new: int, needed: list | None = None) -> bool:
        """Make room for ``n_new`` more tokens in every group, or change nothing and return False.
        ``needed``: what ``pages_needed(slot, n_new)`` just returned, if the caller has it."""
        request = self._take(slot)
        if n_new < 0:
            raise ValueError("cannot reserve a negative number of tokens")
        if request.length + n_new > self.max_tokens_per_request:
            return False
        if needed is None:
            needed = self.pages_needed(slot, n_new)
        for group, count in zip(self.groups, needed):
            if group.paged and count > group.pool.available:
                return False
        for group, count in zip(self.groups, needed):
            if not group.paged or count == 0:
                continue
            pages = group.pool.alloc(count, slot)
            start = request.n_blocks[group.index]
            group.table[slot, start:start + count] = pages
            request.n_blocks[group.index] = start + count
        request.reserved = max(request.reserved, request.length + n_new)
        return True

    def unreserve(self, slot: int) -> None:
        """Give back the pages that were reserved beyond the committed length (a step that
        reserved them did not run to its end): the request is as it was before ``reserve``."""
        request = self._take(slot)
        keep = self._blocks_for(request.length)
        for group in self.groups:
            if not group.paged:
                continue
            held = request.n_blocks[group.index]
            if held > keep:
                row = group.table[slot]
                extra = [int(p) for p in row[keep:held] if p != NO_PAGE]
                group.pool.free(extra, slot)
                self._freed(group, extra)
                row[keep:held] = NO_PAGE
                request.n_blocks[group.index] = keep
        request.reserved = request.length

    def _freed(self, group, pages) -> None:
        if self.on_free is not None and pages:
            self.on_free(group.index, pages)

    def commit(self, slot: int, n_new: int) -> None:
        """``n_new`` tokens were stored.  Pages a window has passed are given back."""
        request = self._take(slot)
        if request.length + n_new > request.reserved:
            raise PageError(f"slot {slot}: committing {n_new} tokens beyond what was reserved")
        request.length += n_new
        for group in self.groups:
            if not group.paged or group.need.window is None:
                continue
            # The next query sits at position >= length and sees keys > length - window.
            first_needed = max(0, request.length - group.need.window + 1)
            keep_from = min(first_needed // self.page_size, request.n_blocks[group.index])
            first = request.first_block[group.index]
            if keep_from > first:
                row = group.table[slot]
                passed = [int(p) for p in row[first:keep_from]]
                group.pool.free(passed, slot)
                self._freed(group, passed)
                row[first:keep_from] = NO_PAGE
                request.first_block[group.index] = keep_from
                self.freed_by_window += len(passed)

    def block_table_row(self, group_index: int, slot: int) -> np.ndarray:
        return self.groups[group_index].table[slot]

    def pages_held(self, slot: int) -> list:
        request = self._take(slot)
        return [request.n_blocks[g.index] - request.first_block[g.index] if g.paged else 0 for g in self.groups]

    def pages_free(self) -> list:
        return [g.pool.available if g.paged else 0 for g in self.groups]

    def pages_in_use(self) -> list:
        return [g.pool.in_use if g.paged else 0 for g in self.groups]

    def check(self) -> None:
        """Invariants: pools are consistent, and every owned page is in exactly one table cell."""
        for group in self.groups:
            if not group.paged:
                continue
            group.pool.check()
            seen = {}
            for slot in range(self.max_requests):
                for block, page in enumerate(group.table[slot]):
                    if page == NO_PAGE:
                        continue
                    if slot not in self._requests:
                        raise PageError(f"group {group.index}: closed slot {slot} still lists page {page}")
                    if page in seen:
                        raise PageError(f"group {group.index}: page {page} is held twice: {seen[page]} and {(slot, block)}")
                    if group.pool.owner_of(int(page)) != slot:
                        raise PageError(f"group {group.index}: page {page} listed by slot {slot} but owned by {group.pool.owner_of(int(page))!r}")
                    seen[int(page)] = (slot, block)
            if len(seen) != group.pool.in_use:
                raise PageError(f"group {group.index}: {group.pool.in_use} pages are owned but {len(seen)} are listed: a page is lost")
        if len(set(self._free_slots)) != len(self._free_slots) or set(self._free_slots) & set(self._requests):
            raise PageError("a slot is free twice, or free and in use")
        if len(self._free_slots) + len(self._requests) != self.max_requests:
            raise PageError("a slot is lost")
