"""The cache manager: pages of keys and values with a block table per request, and slots of
fixed-size state per request.

Policy only: this file decides which page holds which positions and when a page goes back; it
launches nothing (the reference keeps the same split, src/block_pool.h:14-15).  Device tensors
are made by ``make_storage`` and handed to the parts as views.

Groups.  Every cache entry of the run order states a need (``PagedKVNeed`` / ``StateNeed`` / none).
Paged entries with the same (kv heads, head size, window) form a *group*: the group has one page
pool and one block table per request, and a page id addresses the same page in every entry of the
group (the reference has one implicit group: one block id spans all layers,
kernels/batch_gpu.cu:75,114-118).  Groups with a window give pages back as soon as every later
query is past them; their block tables then hold -1 at that place.

Life of a request: ``admit`` (takes a state slot, zeroes its state) -> repeated ``reserve(n)``
(pages for the next n positions in every group, all or nothing) + ``advance(n)`` (the positions
are now filled; pages behind a window are freed) -> ``release`` (everything goes back).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Mapping, Optional, Sequence, Tuple

import torch

from ..parts.base import PagedKVNeed, StateNeed


class CacheError(RuntimeError):
    """A misuse of the manager: unknown request, double free, advancing past what was reserved."""


class PagePool:
    """Page ids 0..n-1 with a reference count each. Pages that came back last go out first, so a
    freed page is reused as early as possible."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))   # pop() hands out 0 first
        self._ref = [0] * n_pages
        self.peak_in_use = 0

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_in_use(self) -> int:
        return self.n_pages - len(self._free)

    def alloc(self) -> Optional[int]:
        if not self._free:
            return None
        p = self._free.pop()
        if self._ref[p] != 0:
            raise CacheError(f"page {p} was on the free list while still referenced")
        self._ref[p] = 1
        self.peak_in_use = max(self.peak_in_use, self.n_in_use)
        return p

    def retain(self, page: int) -> None:
        if self._ref[page] <= 0:
            raise CacheError(f"page {page} is not allocated")
        self._ref[page] += 1

    def free(self, page: int) -> None:
        if not 0 <= page < self.n_pages or self._ref[page] <= 0:
            raise CacheError(f"page {page} freed twice or never allocated")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._ref[page]


@dataclass
class CacheGroup:
    index: int
    need: PagedKVNeed
    cache_ids: List[int]                 # entries of the run order's caches that live in this group
    pool: PagePool
    page_size: int
    k: Optional[torch.Tensor] = None     # [len(cache_ids), n_pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None

    @property
    def window(self) -> Optional[int]:
        return self.need.window


@dataclass
class RequestCache:
    rid: Hashable
    slot: int
    length: int = 0                                  # positions filled
    reserved: int = 0                                # positions that have pages (>= length)
    tables: List[List[int]] = field(default_factory=list)   # per group: page id per page index, -1 = given back


@dataclass
class PagedKVView:
    """What an attention part gets for one cache entry."""
    group: int
    k: torch.Tensor          # [n_pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    page_size: int
    window: Optional[int]


class CacheManager:
    def __init__(self, needs: Mapping[int, object], n_pages: int, page_size: int = 16, n_slots: int = 8):
        """needs: cache index -> PagedKVNeed | StateNeed | None. n_pages: pages in every group's pool."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.n_slots = page_size, n_slots
        self.groups: List[CacheGroup] = []
        self.group_of_cache: Dict[int, Tuple[int, int]] = {}     # cache id -> (group index, index in group)
        self.state_needs: Dict[int, StateNeed] = {}
        self.state: Dict[int, Dict[str, torch.Tensor]] = {}
        by_key: Dict[Tuple, CacheGroup] = {}
        for cid in sorted(needs):
            need = needs[cid]
            if isinstance(need, PagedKVNeed):
                key = (need.num_kv_heads, need.head_dim, need.window)
                g = by_key.get(key)
                if g is None:
                    g = CacheGroup(len(self.groups), need, [], PagePool(n_pages), page_size)
                    by_key[key] = g
                    self.groups.append(g)
                self.group_of_cache[cid] = (g.index, len(g.cache_ids))
                g.cache_ids.append(cid)
            elif isinstance(need, StateNeed):
                self.state_needs[cid] = need
            elif need is not None:
                raise TypeError(f"cache {cid}: unknown kind of need {need!r}")
        self._free_slots = list(range(n_slots - 1, -1, -1))
        self.requests: Dict[Hashable, RequestCache] = {}

    # ------------------------------------------------------------------ storage

    def make_storage(self, dtype: torch.dtype, device) -> None:
        """Allocates the page tensors of every group and the state tensors of every state entry."""
        for g in self.groups:
            shape = (len(g.cache_ids), g.pool.n_pages, g.need.num_kv_heads, self.page_size, g.need.head_dim)
            g.k = torch.zeros(shape, dtype=dtype, device=device)
            g.v = torch.zeros(shape, dtype=dtype, device=device)
        for cid, need in self.state_needs.items():
            self.state[cid] = {name: torch.zeros((self.n_slots,) + tuple(shape), dtype=dt, device=device)
                               for name, (shape, dt) in need.shapes.items()}

    def storage_bytes(self, dtype: torch.dtype) -> int:
        item = torch.empty((), dtype=dtype).element_size()
        return sum(2 * len(g.cache_ids) * g.pool.n_pages * g.need.num_kv_heads * self.page_size * g.need.head_dim * item
                   for g in self.groups)

    def view(self, cache_id: int):
        """PagedKVView, the dict of state tensors, or None for the given cache entry."""
        if cache_id in self.group_of_cache:
            gi, li = self.group_of_cache[cache_id]
            g = self.groups[gi]
            if g.k is None:
                raise CacheError("make_storage() has not been called")
            return PagedKVView(gi, g.k[li], g.v[li], self.page_size, g.window)
        if cache_id in self.state_needs:
            return self.state[cache_id]
        return None

    # ------------------------------------------------------------------ requests

    def _req(self, rid) -> RequestCache:
        try:
            return self.requests[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not admitted") from None

    def has_slot(self) -> bool:
        return bool(self._free_slots)

    def admit(self, rid) -> RequestCache:
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already admitted")
        if not self._free_slots:
            raise CacheError("no free request slot")
        slot = self._free_slots.pop()
        for tensors in self.state.values():
            for t in tensors.values():
                t[slot].zero_()
        rc = RequestCache(rid, slot, tables=[[] for _ in self.groups])
        self.requests[rid] = rc
        return rc

    def _first_needed_page(self, g: CacheGroup, length: int) -> int:
        """Index of the first page that a query at position >= length can still read."""
        if g.window is None:
            return 0
        return max(0, length - g.window + 1) // self.page_size

    def pages_needed(self, rid, n_new: int) -> List[int]:
        """Per group: pages that reserve(rid, n_new) would take from the pool."""
        rc = self._req(rid)
        end = max(rc.reserved, rc.length + n_new)
        last_page = (end - 1) // self.page_size if end > 0 else -1
        return [max(0, last_page + 1 - len(t)) for t in rc.tables]

    def can_reserve(self, wanted: Sequence[Tuple[Hashable, int]]) -> bool:
        """True if reserve() would succeed for every (rid, n) of the list, taken together."""
        total = [0] * len(self.groups)
        for rid, n in wanted:
            for gi, k in enumerate(self.pages_needed(rid, n)):
                total[gi] += k
        return all(total[gi] <= g.pool.n_free for gi, g in enumerate(self.groups))

    def reserve(self, rid, n_new: int) -> bool:
        """Pages for positions [length, length+n_new) in every group. All or nothing."""
        rc = self._req(rid)
        if n_new < 0:
            raise CacheError("cannot reserve a negative number of positions")
        need = self.pages_needed(rid, n_new)
        if any(k > g.pool.n_free for k, g in zip(need, self.groups)):
            return False
        for g, k, table in zip(self.groups, need, rc.tables):
            for _ in range(k):
                table.append(g.pool.alloc())
        rc.reserved = max(rc.reserved, rc.length + n_new)
        return True

    def unreserve(self, rid) -> None:
        """Gives back pages that were reserved beyond the filled length (a step that did not run)."""
        rc = self._req(rid)
        keep = (rc.length + self.page_size - 1) // self.page_size
        for g, table in zip(self.groups, rc.tables):
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    g.pool.free(p)
        rc.reserved = rc.length

    def advance(self, rid, n: int) -> None:
        """The next n positions are filled. Pages that no later query can read go back."""
        rc = self._req(rid)
        if n < 0 or rc.length + n > rc.reserved:
            raise CacheError(f"request {rid!r}: advancing {n} from {rc.length} passes the reserved {rc.reserved}")
        rc.length += n
        for g, table in zip(self.groups, rc.tables):
            first = min(self._first_needed_page(g, rc.length), len(table))
            for i in range(first):
                if table[i] >= 0:
                    g.pool.free(table[i])
                    table[i] = -1

    def release(self, rid) -> None:
        rc = self._req(rid)
        for g, table in zip(self.groups, rc.tables):
            for p in table:
                if p >= 0:
                    g.pool.free(p)
            table.clear()
        self._free_slots.append(rc.slot)
        del self.requests[rid]

    # ------------------------------------------------------------------ inspection

    def length(self, rid) -> int:
        return self._req(rid).length

    def slot(self, rid) -> int:
        return self._req(rid).slot

    def block_table(self, rid, group: int) -> List[int]:
        return self._req(rid).tables[group]

    def pages_in_use(self) -> List[int]:
        return [g.pool.n_in_use for g in self.groups]

    def pages_total(self) -> List[int]:
        return [g.pool.n_pages for g in self.groups]

    def pages_free(self) -> List[int]:
        return [g.pool.n_free for g in self.groups]

    def check_invariants(self) -> None:
        """No page lost, held twice, or free while held. For tests."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, int] = {}
            for rc in self.requests.values():
                for p in rc.tables[gi]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            free = list(g.pool._free)
            if len(set(free)) != len(free):
                raise CacheError(f"group {gi}: a page is on the free list twice")
            for p, n in held.items():
                if n != g.pool.refcount(p):
                    raise CacheError(f"group {gi}: page {p} is held {n} times but counted {g.pool.refcount(p)}")
                if p in free:
                    raise CacheError(f"group {gi}: page {p} is held and free")
            if len(held) + len(free) != g.pool.n_pages:
                raise CacheError(f"group {gi}: {g.pool.n_pages - len(held) - len(free)} pages are lost")
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.n_slots:
            raise CacheError("a state slot is lost")
