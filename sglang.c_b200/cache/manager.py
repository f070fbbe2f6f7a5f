"""The cache manager: pages of keys and values with a block table per request,
one pool per group of mixer calls with equal needs, and slots for per-request
state of fixed size.

The reference takes all pages of a request at admission (prompt + max_new + 1
one-position pages, src/scheduler.c:340-360) and returns them at the end
(:222-225).  Here pages hold `page_size` positions and a request grows page by
page; pages are returned when the request ends, is preempted, or, in a group
with a window, when the window has passed them.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .needs import CacheBinding, CacheNeed
from .pages import PagePool


class CacheError(RuntimeError):
    pass


@dataclass
class _Group:
    need: CacheNeed
    calls: List[int]                 # indices into the running order that own a cache here
    pool: Optional[PagePool] = None  # paged_kv only
    tensor: object = None            # [n_calls, n_pages, 2, Hkv, page_size, D] or [n_calls, n_slots, *shape]
    tables: Dict[object, List[int]] = field(default_factory=dict)   # request -> page per block (-1 = released)


class CacheManager:
    """needs[i] is the CacheNeed (or None) of the i-th call of the running
    order; cache_of[i] names the earlier call whose cache call i reads.
    `make_tensor(shape, dtype_name)` allocates device memory (None in host-only
    tests)."""

    def __init__(self, needs, cache_of, page_size, n_pages, max_requests, make_tensor=None,
                 cache_dtype="float32"):
        if page_size <= 0 or n_pages <= 0 or max_requests <= 0:
            raise ValueError("page_size, n_pages and max_requests must be positive")
        self.page_size = int(page_size)
        self.n_pages = int(n_pages)
        self.max_requests = int(max_requests)
        self.groups: List[_Group] = []
        self._call_group = {}          # owning call -> (group index, index within the group)
        self._bindings = {}
        by_need = {}
        for i, need in enumerate(needs):
            if need is None or cache_of[i] is not None:
                continue
            gi = by_need.get(need)
            if gi is None:
                gi = len(self.groups)
                by_need[need] = gi
                self.groups.append(_Group(need, []))
            g = self.groups[gi]
            self._call_group[i] = (gi, len(g.calls))
            g.calls.append(i)
        for g in self.groups:
            if g.need.kind == "paged_kv":
                g.pool = PagePool(self.n_pages)
                shape = (len(g.calls), self.n_pages, 2, g.need.n_kv_heads, self.page_size, g.need.head_dim)
                dt = cache_dtype
            elif g.need.kind == "state":
                shape = (len(g.calls), self.max_requests) + tuple(g.need.state_shape)
                dt = g.need.state_dtype
            else:
                raise CacheError(f"unknown cache need kind '{g.need.kind}'")
            g.tensor = make_tensor(shape, dt) if make_tensor is not None else None
        for i, need in enumerate(needs):
            if need is None:
                continue
            owner = i if cache_of[i] is None else cache_of[i]
            if owner not in self._call_group:
                raise CacheError(f"call {i} reads the cache of call {owner}, which keeps none")
            if needs[owner] != need:
                raise CacheError(f"call {i} reads the cache of call {owner} but their needs differ")
            gi, ci = self._call_group[owner]
            t = self.groups[gi].tensor
            self._bindings[i] = CacheBinding(need.kind, gi, t[ci] if t is not None else None,
                                             write=(owner == i))
        # per-request bookkeeping
        self._free_slots = list(range(self.max_requests - 1, -1, -1))
        self._slot = {}
        self._len = {}

    # -- requests -----------------------------------------------------------
    def binding(self, call_index):
        return self._bindings.get(call_index)

    def has_request(self, req):
        return req in self._slot

    def n_free_slots(self):
        return len(self._free_slots)

    def add_request(self, req):
        """Give the request a state slot (zeroed) and empty block tables.
        Returns the slot, or None when all slots are taken."""
        if req in self._slot:
            raise CacheError(f"request {req!r} is already live")
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._slot[req] = slot
        self._len[req] = 0
        for g in self.groups:
            if g.need.kind == "paged_kv":
                g.tables[req] = []
            elif g.tensor is not None:
                g.tensor[:, slot].zero_()
        return slot

    def slot(self, req):
        return self._slot[req]

    def length(self, req):
        return self._len[req]

    def _blocks_for(self, n_tokens):
        return (n_tokens + self.page_size - 1) // self.page_size

    def _first_needed_block(self, g, length):
        """First block a query at position >= `length` can still see."""
        if g.need.window is None:
            return 0
        first_pos = max(0, length - g.need.window + 1)
        return first_pos // self.page_size

    def pages_needed(self, req, new_len):
        """New pages per paged group to grow the request to new_len positions,
        after returning the pages a window has passed."""
        out = []
        old = self._len[req]
        for g in self.groups:
            if g.need.kind != "paged_kv":
                continue
            have = len(g.tables[req])
            need = max(0, self._blocks_for(new_len) - have)
            first = self._first_needed_block(g, old)
            reclaim = sum(1 for b in range(min(first, have)) if g.tables[req][b] >= 0)
            out.append((need, reclaim))
        return out

    def can_extend(self, req, new_len):
        i = 0
        for g in self.groups:
            if g.need.kind != "paged_kv":
                continue
            need, reclaim = self.pages_needed(req, new_len)[i]
            i += 1
            if need > g.pool.n_free + reclaim:
                return False
        return True

    def can_extend_all(self, wants):
        """Whether every (request, new_len) of `wants` can grow in one step."""
        paged = [g for g in self.groups if g.need.kind == "paged_kv"]
        for g in paged:
            budget = g.pool.n_free
            for req, new_len in wants:
                table = g.tables[req]
                first = self._first_needed_block(g, self._len[req])
                budget += sum(1 for b in range(min(first, len(table))) if table[b] >= 0)
                budget -= max(0, self._blocks_for(new_len) - len(table))
            if budget < 0:
                return False
        return True

    def extend(self, req, new_len):
        """Make room for positions up to new_len (exclusive) in every paged
        group, all or nothing.  Returns False, changing nothing but the return
        of passed window pages, when a pool has too few free pages."""
        if req not in self._slot:
            raise CacheError(f"request {req!r} is not live")
        old = self._len[req]
        if new_len < old:
            raise CacheError("a request cannot shrink")
        paged = [g for g in self.groups if g.need.kind == "paged_kv"]
        for g in paged:           # pages behind the window go back first
            table = g.tables[req]
            first = self._first_needed_block(g, old)
            for b in range(min(first, len(table))):
                if table[b] >= 0:
                    g.pool.unref(table[b])
                    table[b] = -1
        want = [max(0, self._blocks_for(new_len) - len(g.tables[req])) for g in paged]
        if any(w > g.pool.n_free for w, g in zip(want, paged)):
            return False
        for w, g in zip(want, paged):
            g.tables[req].extend(g.pool.alloc(w))
        self._len[req] = new_len
        return True

    def grow_by_one(self, reqs, needs_page):
        """One more position for each of `reqs`; needs_page holds the indices of those whose
        new position begins a page (the caller has checked can_extend_all for them).  Only for
        groups without a window: nothing is given back here."""
        for i, req in enumerate(reqs):
            if i in needs_page:
                ok = self.extend(req, self._len[req] + 1)
                if not ok:
                    raise CacheError("grow_by_one ran out of pages after can_extend_all")
            else:
                self._len[req] += 1

    def shrink_by_one(self, reqs, took_page):
        """Undo grow_by_one: one position less for each of `reqs`; those whose indices are in
        took_page give back the page that the position began."""
        for i, req in enumerate(reqs):
            self._len[req] -= 1
            if i in took_page:
                for g in self.groups:
                    if g.need.kind == "paged_kv":
                        g.pool.unref(g.tables[req].pop())

    def truncate(self, req, new_len):
        """Shorten a request to new_len positions: what lies beyond is forgotten and the pages it
        filled alone go back to the pool.  (What a step that failed half-way had taken is undone
        with it; a benchmark rewinds a request with it.)  A group with a window cannot go back
        past pages it has already released."""
        if req not in self._slot:
            raise CacheError(f"request {req!r} is not live")
        if not (0 <= new_len <= self._len[req]):
            raise CacheError(f"request {req!r} holds {self._len[req]} positions; cannot truncate to {new_len}")
        keep = self._blocks_for(new_len)
        for g in self.groups:
            if g.need.kind != "paged_kv":
                continue
            table = g.tables[req]
            first = self._first_needed_block(g, new_len)
            if any(table[b] < 0 for b in range(first, min(keep, len(table)))):
                raise CacheError(f"request {req!r}: a page that {new_len} positions still need was released "
                                 "when the window passed it")
        for g in self.groups:
            if g.need.kind != "paged_kv":
                continue
            table = g.tables[req]
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    g.pool.unref(p)
        self._len[req] = new_len

    def free_request(self, req):
        """Return every page and the state slot of a request."""
        if req not in self._slot:
            raise CacheError(f"request {req!r} is not live (freed twice?)")
        for g in self.groups:
            if g.need.kind == "paged_kv":
                for p in g.tables.pop(req):
                    if p >= 0:
                        g.pool.unref(p)
        self._free_slots.append(self._slot.pop(req))
        del self._len[req]

    # -- what a step needs --------------------------------------------------
    def block_table(self, group_index, req):
        return self.groups[group_index].tables[req]

    def slot_of_position(self, group_index, req, pos):
        page = self.groups[group_index].tables[req][pos // self.page_size]
        if page < 0:
            raise CacheError(f"position {pos} of request {req!r} lies in a released page")
        return page * self.page_size + pos % self.page_size

    def paged_groups(self):
        return [i for i, g in enumerate(self.groups) if g.need.kind == "paged_kv"]

    def n_free_pages(self, group_index=None):
        gs = self.paged_groups() if group_index is None else [group_index]
        return min((self.groups[i].pool.n_free for i in gs), default=self.n_pages)

    def live_requests(self):
        return list(self._slot)

    def check(self):
        """No page lost, held twice or freed twice; slots likewise."""
        for g in self.groups:
            if g.need.kind != "paged_kv":
                continue
            g.pool.check()
            held = [p for t in g.tables.values() for p in t if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError("a page is in two block tables")
            if len(held) + g.pool.n_free != g.pool.n_pages:
                raise CacheError("a page is lost: neither free nor in a block table")
            for p in held:
                if g.pool.refcount(p) != 1:
                    raise CacheError(f"page {p} has {g.pool.refcount(p)} references")
        slots = list(self._slot.values())
        if len(slots) != len(set(slots)) or len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a state slot is lost or held twice")
        return True
