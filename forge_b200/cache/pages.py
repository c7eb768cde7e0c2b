"""A pool of fixed-size cache pages: which are free, which are held, and by whom.

Pure host bookkeeping (the device storage is one tensor per layer indexed by page id).  The free list is
LIFO, so a page given back is the next one handed out: tests with few pages see reuse at once.  Handing
out a page that is held, or taking back one that is free, is a bug in the caller and raises.
"""


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """Not enough free pages (or request slots) for what was asked; nothing was allocated."""


class PagePool:
    def __init__(self, num_pages):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))     # pop() hands out page 0 first
        self._owner = [None] * num_pages

    @property
    def num_free(self):
        return len(self._free)

    @property
    def num_held(self):
        return self.num_pages - len(self._free)

    def allocate(self, n, owner):
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} free of {self.num_pages}")
        pages = []
        for _ in range(n):
            p = self._free.pop()
            if self._owner[p] is not None:
                raise CacheError(f"page {p} on the free list is held by {self._owner[p]!r}")
            self._owner[p] = owner
            pages.append(p)
        return pages

    def release(self, page, owner):
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page id {page} out of range")
        if self._owner[page] is None:
            raise CacheError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise CacheError(f"page {page} is held by {self._owner[page]!r}, not by {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner(self, page):
        return self._owner[page]

    def check(self):
        """Invariant: every page is either free exactly once or held exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise CacheError(f"page {p} is both free and held, or neither")
