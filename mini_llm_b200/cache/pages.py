"""Page pool: fixed-size pages handed out and taken back, each owned at most once.

The reference has no pages: every sequence owns contiguous K and V buffers for
the full context (engine/src/gpt2_gpu.cu:147-159) and a Python free-list hands
out whole caches (pytorch/src/mini_llm/native.py:339-364).  Here the unit is a
page of ``page_size`` token slots, and the pool checks its own invariants: a
page is never handed out twice, never freed twice, never lost.
"""

from __future__ import annotations


class PageError(RuntimeError):
    pass


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise ValueError("a pool cannot have a negative number of pages")
        self.n_pages = int(n_pages)
        # LIFO: the page freed last is handed out first, so reuse happens at once.
        self._free = list(range(self.n_pages - 1, -1, -1))
        self._owner = [None] * self.n_pages
        self.allocations = 0          # pages handed out since the start
        self.reused = 0               # of these, pages that had been used before
        self._ever_used = [False] * self.n_pages

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.n_pages - len(self._free)

    def alloc(self, count: int, owner) -> list[int] | None:
        """``count`` pages for ``owner``, or None (and nothing changes) if fewer are free."""
        if count < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if count > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            if self._owner[page] is not None:
                raise PageError(f"page {page} was on the free list while owned by {self._owner[page]!r}")
            self._owner[page] = owner
            self.allocations += 1
            if self._ever_used[page]:
                self.reused += 1
            self._ever_used[page] = True
        return pages

    def free(self, pages, owner) -> None:
        for page in pages:
            if not 0 <= page < self.n_pages:
                raise PageError(f"page {page} is not in the pool")
            if self._owner[page] is None:
                raise PageError(f"page {page} freed twice")
            if self._owner[page] != owner:
                raise PageError(f"page {page} is owned by {self._owner[page]!r}, freed by {owner!r}")
            self._owner[page] = None
            self._free.append(page)

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is either free once or owned; none is lost."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageError("a page is on the free list twice")
        for page in range(self.n_pages):
            if (self._owner[page] is None) != (page in free):
                raise PageError(f"page {page} is neither free nor owned, or both")
