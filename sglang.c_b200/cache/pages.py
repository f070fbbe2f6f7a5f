"""Host-side allocator of page ids: a LIFO stack of free pages with reference
counts, all-or-nothing allocation (reference src/gpt2.c:135-138,158-182).
LIFO means a page given back is the next one handed out."""


class PagePoolError(RuntimeError):
    pass


class PagePool:
    def __init__(self, n_pages):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = int(n_pages)
        # top of the stack is the end of the list; page 0 pops first
        self._free = list(range(self.n_pages - 1, -1, -1))
        self._refs = [0] * self.n_pages

    @property
    def n_free(self):
        return len(self._free)

    def alloc(self, n):
        """n page ids with one reference each, or None if fewer than n are free."""
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._refs[p] = 1
        return out

    def ref(self, page):
        if not (0 <= page < self.n_pages) or self._refs[page] <= 0:
            raise PagePoolError(f"page {page} is not held; cannot add a reference")
        self._refs[page] += 1

    def unref(self, page):
        """Drop one reference; the page returns to the stack at zero."""
        if not (0 <= page < self.n_pages):
            raise PagePoolError(f"page {page} is outside the pool of {self.n_pages}")
        if self._refs[page] <= 0:
            raise PagePoolError(f"page {page} freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page):
        return self._refs[page]

    def check(self):
        """Invariants: every page is either free exactly once or held."""
        seen = set()
        for p in self._free:
            if p in seen:
                raise PagePoolError(f"page {p} is on the free stack twice")
            if self._refs[p] != 0:
                raise PagePoolError(f"page {p} is free but has references")
            seen.add(p)
        held = sum(1 for r in self._refs if r > 0)
        if held + len(self._free) != self.n_pages:
            raise PagePoolError("a page is neither free nor held")
        return True
