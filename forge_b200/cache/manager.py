"""The cache manager: paged keys/values per group of layers, a block table per request and group, and
slots for per-request state of fixed size.

Layers whose mixers need the same kind of cache (same kv heads, head size and window) form a GROUP; a
group has its own page pool and every request has one block table per group, shared by the group's
layers (the reference's unused PagedKVCache keeps a table per layer although a block id reserves storage
in every layer, src/inference/paged_kv_cache.cpp:96-99, 196-207).  Pages go back to the pool when a
request ends, and, for a windowed group, as soon as every position in the page is older than the
window of every future query.  Beside pages, each request holds one SLOT (an index below max_requests)
that addresses its row in every fixed-size state tensor; a slot's rows are zeroed before first use.

This module is host bookkeeping only; `storage.py` owns the device tensors.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .pages import CacheError, OutOfPages, PagePool


@dataclass(frozen=True)
class GroupSpec:
    name: str
    num_pages: int
    window: Optional[int] = None      # None: all positions are kept


@dataclass
class _Request:
    slot: int
    num_tokens: int = 0
    # per group: logical page index -> page id, or -1 once the window has passed it
    tables: Dict[str, List[int]] = field(default_factory=dict)


class CacheManager:
    def __init__(self, groups, page_size, max_requests):
        if page_size <= 0 or max_requests <= 0:
            raise CacheError("page_size and max_requests must be positive")
        self.page_size, self.max_requests = page_size, max_requests
        self.groups = {g.name: g for g in groups}
        self.pools = {g.name: PagePool(g.num_pages) for g in groups}
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._fresh_slots = []
        self._requests: Dict[object, _Request] = {}

    # ------------------------------------------------------------------------------- admission
    def has_free_slot(self):
        return bool(self._free_slots)

    def admit(self, req_id):
        """Gives the request a slot (no pages yet).  The slot's state rows must be zeroed before the next
        step: ``take_fresh_slots`` tells the engine which."""
        if req_id in self._requests:
            raise CacheError(f"request {req_id!r} is already admitted")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        self._requests[req_id] = _Request(slot=slot, tables={g: [] for g in self.groups})
        self._fresh_slots.append(slot)
        return slot

    def take_fresh_slots(self):
        fresh, self._fresh_slots = self._fresh_slots, []
        return fresh

    def live_requests(self):
        return list(self._requests)

    def slot(self, req_id):
        return self._requests[req_id].slot

    def num_tokens(self, req_id):
        return self._requests[req_id].num_tokens

    # ------------------------------------------------------------------------------- pages
    def _pages_for(self, n_tokens):
        return (n_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, req_id, n_new):
        """{group: pages that appending n_new tokens would take from the pool}."""
        r = self._requests[req_id]
        return {g: self._pages_for(r.num_tokens + n_new) - len(t) for g, t in r.tables.items()}

    def pages_for_new_request(self, n_tokens):
        return {g: self._pages_for(n_tokens) for g in self.groups}

    def can_append(self, req_id, n_new, reserve=None):
        """``reserve``: {group: pages already promised to others in this step}."""
        need = self.pages_needed(req_id, n_new)
        return all(need[g] + (reserve or {}).get(g, 0) <= self.pools[g].num_free for g in need)

    def append(self, req_id, n_new):
        """Extends the request by n_new tokens: allocates the pages they need in every group (all or
        nothing) and returns {group: [slot of each new token]} with slot = page * page_size + offset."""
        r = self._requests[req_id]
        need = self.pages_needed(req_id, n_new)
        for g, n in need.items():
            if n > self.pools[g].num_free:
                raise OutOfPages(f"request {req_id!r}: group {g!r} needs {n} pages, {self.pools[g].num_free} free")
        start = r.num_tokens
        slots = {}
        for g, n in need.items():
            table = r.tables[g]
            table.extend(self.pools[g].allocate(n, req_id))
            out = []
            for pos in range(start, start + n_new):
                page = table[pos // self.page_size]
                if page < 0:
                    raise CacheError(f"request {req_id!r}: position {pos} lies in a page the window already released")
                out.append(page * self.page_size + pos % self.page_size)
            slots[g] = out
        r.num_tokens = start + n_new
        return slots

    def release_out_of_window(self, req_id):
        """After a step: gives back the pages of windowed groups that no future query can read.  The next
        query is at position >= num_tokens and reads keys > position - window, so a page whose last
        position is <= num_tokens - window is dead.  Returns the number of pages released."""
        r = self._requests[req_id]
        released = 0
        for g, spec in self.groups.items():
            if spec.window is None:
                continue
            table = r.tables[g]
            first_needed = r.num_tokens - spec.window + 1          # smallest key position a future query reads
            dead_pages = max(0, first_needed) // self.page_size     # pages wholly below it
            for i in range(min(dead_pages, len(table))):
                if table[i] >= 0:
                    self.pools[g].release(table[i], req_id)
                    table[i] = -1
                    released += 1
        return released

    def block_table(self, req_id, group):
        return self._requests[req_id].tables[group]

    def free(self, req_id):
        """The request is over (finished, aborted or preempted): all its pages and its slot go back."""
        r = self._requests.pop(req_id, None)
        if r is None:
            raise CacheError(f"request {req_id!r} is not admitted (freed twice?)")
        for g, table in r.tables.items():
            for p in reversed(table):
                if p >= 0:
                    self.pools[g].release(p, req_id)
        self._free_slots.append(r.slot)
        if r.slot in self._fresh_slots:
            self._fresh_slots.remove(r.slot)

    def reset(self):
        for rid in list(self._requests):
            self.free(rid)

    # ------------------------------------------------------------------------------- checks
    def num_free_pages(self, group=None):
        if group is not None:
            return self.pools[group].num_free
        return {g: p.num_free for g, p in self.pools.items()}

    def check(self):
        """No page lost, held twice or freed twice; no slot lost or shared."""
        for g, pool in self.pools.items():
            pool.check()
            held = [p for r in self._requests.values() for p in r.tables[g] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g!r}: a page is in two block tables")
            if len(held) != pool.num_held:
                raise CacheError(f"group {g!r}: {pool.num_held} pages held but {len(held)} in block tables")
            for rid, r in self._requests.items():
                for p in r.tables[g]:
                    if p >= 0 and pool.owner(p) != rid:
                        raise CacheError(f"group {g!r}: page {p} in the table of {rid!r} is held by {pool.owner(p)!r}")
        slots = [r.slot for r in self._requests.values()] + self._free_slots
        if sorted(slots) != list(range(self.max_requests)):
            raise CacheError("a request slot is lost or shared")
