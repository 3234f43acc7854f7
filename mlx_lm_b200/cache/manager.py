"""The cache manager: pages of keys and values with a block table per
request, and slots of fixed size for per-request state.

It replaces the contiguous, growing ``KVCache`` / left-padded ``BatchKVCache``
of mlx-lm (mlx_lm/models/cache.py:325-407, 921-1139) and, for state of fixed
size, its ``ArraysCache`` (:594-733).

Groups.  Caches (one per block that has one) with equal needs — the same
number of key/value heads, head size and window — form a *group*.  A group
has its own pool of pages ``[caches in group, n_pages, heads, page, head_dim]``
for K and for V, its own free list and, per request, its own block table:
logical page ``p // page`` of the request -> page id, or -1 where the request
holds no page (not reached yet, or given back because the window has passed
it).  All caches of a group share the request's block table: page id ``i``
means row ``i`` of every cache's pool in that group.

Life of a request: ``add_request`` takes a state slot; before a step
``reserve(rid, n)`` takes the pages positions ``length .. length+n-1`` need
(all groups, or nothing if one runs out: ``OutOfPages``); after the step
``commit(rid)`` advances the length and gives back pages a window has passed
(``rollback(rid)`` instead, if the step failed: the reservation is undone);
``truncate`` rewinds; ``release`` gives everything back.  Freed pages go on
top of the free list (LIFO), so a small pool re-uses pages at once.

The bookkeeping is plain Python and runs without a GPU; device tensors are
created only when a device is given.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from ..parts.base import PagedKVSpec, StateSpec


class OutOfPages(RuntimeError):
    """A group's pool cannot give the pages a reservation needs."""


class NoFreeSlot(RuntimeError):
    """All per-request slots are taken."""


class PagePool:
    """Free list over ``n_pages`` page ids with checks against double use."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))  # pop() gives 0 first
        self._held = [False] * n_pages
        self.high_water = 0
        self.n_allocations = 0

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.pop()
        assert not self._held[p], f"page {p} was on the free list while held"
        self._held[p] = True
        self.n_allocations += 1
        self.high_water = max(self.high_water, self.n_held)
        return p

    def free(self, p: int) -> None:
        if not 0 <= p < self.n_pages:
            raise ValueError(f"page id {p} is outside the pool of {self.n_pages}")
        if not self._held[p]:
            raise RuntimeError(f"page {p} freed twice")
        self._held[p] = False
        self._free.append(p)

    def is_held(self, p: int) -> bool:
        return self._held[p]


@dataclass
class KVGroup:
    spec: PagedKVSpec
    cache_ids: List[int]
    pool: PagePool
    k: object = None   # device tensor [len(cache_ids), n_pages, heads, page, head_dim]
    v: object = None

    def index_of(self, cache_id: int) -> int:
        return self.cache_ids.index(cache_id)


@dataclass
class StateGroup:
    spec: StateSpec
    cache_ids: List[int]
    data: object = None   # device tensor [len(cache_ids), n_slots, *shape] float32

    def index_of(self, cache_id: int) -> int:
        return self.cache_ids.index(cache_id)


@dataclass
class RequestCache:
    rid: Hashable
    slot: int
    length: int = 0          # positions whose keys/values (or state) are committed
    reserved: int = 0        # positions reserved for the step in flight
    pages: List[List[int]] = field(default_factory=list)   # per KV group: logical page -> page id or -1


class CacheManager:
    def __init__(self, cache_specs: Dict[int, object], page_size: int = 16, n_pages: int = 64,
                 max_requests: int = 64, max_len: int = 1024, dtype=None, device=None):
        if page_size <= 0 or page_size & (page_size - 1):
            raise ValueError(f"page size {page_size} must be a power of two")
        self.page_size, self.max_requests, self.max_len = page_size, max_requests, max_len
        self.table_width = (max_len + page_size - 1) // page_size
        self.dtype, self.device = dtype, device
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._where: Dict[int, Tuple[str, int]] = {}   # cache id -> ("kv" | "state", group index)
        for cid in sorted(cache_specs):
            spec = cache_specs[cid]
            if isinstance(spec, PagedKVSpec):
                for gi, g in enumerate(self.kv_groups):
                    if g.spec == spec:
                        g.cache_ids.append(cid)
                        break
                else:
                    gi = len(self.kv_groups)
                    self.kv_groups.append(KVGroup(spec, [cid], PagePool(n_pages)))
                self._where[cid] = ("kv", gi)
            elif isinstance(spec, StateSpec):
                for gi, g in enumerate(self.state_groups):
                    if g.spec == spec:
                        g.cache_ids.append(cid)
                        break
                else:
                    gi = len(self.state_groups)
                    self.state_groups.append(StateGroup(spec, [cid]))
                self._where[cid] = ("state", gi)
            else:
                raise TypeError(f"cache {cid}: spec {spec!r} is neither PagedKVSpec nor StateSpec")
        self.requests: Dict[Hashable, RequestCache] = {}
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        if device is not None:
            self._allocate_device(n_pages)

    # ------------------------------------------------------------ device side
    def _allocate_device(self, n_pages: int) -> None:
        import torch

        for g in self.kv_groups:
            shape = (len(g.cache_ids), n_pages, g.spec.n_kv_heads, self.page_size, g.spec.head_dim)
            # zeros, not empty: a masked key's value row is multiplied by a zero weight and must be finite
            g.k = torch.zeros(shape, dtype=self.dtype, device=self.device)
            g.v = torch.zeros(shape, dtype=self.dtype, device=self.device)
        for g in self.state_groups:
            shape = (len(g.cache_ids), self.max_requests) + tuple(g.spec.shape)
            g.data = torch.zeros(shape, dtype=torch.float32, device=self.device)

    def nbytes(self) -> int:
        n = 0
        for g in self.kv_groups:
            if g.k is not None:
                n += 2 * g.k.numel() * g.k.element_size()
        for g in self.state_groups:
            if g.data is not None:
                n += g.data.numel() * 4
        return n

    def where(self, cache_id: int) -> Tuple[str, int]:
        return self._where[cache_id]

    # ------------------------------------------------------------ requests
    def add_request(self, rid: Hashable) -> int:
        if rid in self.requests:
            raise KeyError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self.requests[rid] = RequestCache(rid, slot, pages=[[] for _ in self.kv_groups])
        for g in self.state_groups:
            if g.data is not None:
                g.data[:, slot].zero_()
        return slot

    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def length(self, rid: Hashable) -> int:
        return self.requests[rid].length

    def _window_floor(self, spec: PagedKVSpec, length: int) -> int:
        """First logical page a request of ``length`` committed tokens still needs."""
        if spec.window is None:
            return 0
        first_key = max(0, length - spec.window + 1)
        return first_key // self.page_size

    def pages_needed(self, rid: Hashable, n: int) -> List[int]:
        """New pages per KV group that reserving ``n`` more positions would take."""
        r = self.requests[rid]
        end = r.length + r.reserved + n
        need_pages = (end + self.page_size - 1) // self.page_size
        return [max(0, need_pages - len(pl)) for pl in r.pages]

    def can_reserve(self, wants: Sequence[Tuple[Hashable, int]]) -> bool:
        total = [0] * len(self.kv_groups)
        for rid, n in wants:
            for gi, c in enumerate(self.pages_needed(rid, n)):
                total[gi] += c
        return all(t <= g.pool.n_free for t, g in zip(total, self.kv_groups))

    def reserve(self, rid: Hashable, n: int) -> int:
        """Take pages for the next ``n`` positions; returns the first of these positions.
        Takes nothing if any group runs out."""
        r = self.requests[rid]
        if n <= 0:
            raise ValueError(f"reserve of {n} positions")
        if r.length + r.reserved + n > self.max_len:
            raise ValueError(f"request {rid!r}: {r.length + r.reserved + n} positions exceed the maximum "
                             f"length {self.max_len}")
        need = self.pages_needed(rid, n)
        for c, g in zip(need, self.kv_groups):
            if c > g.pool.n_free:
                raise OutOfPages(f"request {rid!r} needs {c} more page(s), pool has {g.pool.n_free} free "
                                 f"of {g.pool.n_pages}")
        for gi, (c, g) in enumerate(zip(need, self.kv_groups)):
            for _ in range(c):
                r.pages[gi].append(g.pool.alloc())
        start = r.length + r.reserved
        r.reserved += n
        return start

    def commit(self, rid: Hashable) -> None:
        """The step that used the reservation has been issued: the positions are part of the request."""
        r = self.requests[rid]
        r.length += r.reserved
        r.reserved = 0
        for gi, g in enumerate(self.kv_groups):
            if g.spec.window is None:
                continue
            floor = min(self._window_floor(g.spec, r.length), len(r.pages[gi]))
            for lp in range(floor):
                if r.pages[gi][lp] >= 0:
                    g.pool.free(r.pages[gi][lp])
                    r.pages[gi][lp] = -1

    def rollback(self, rid: Hashable) -> None:
        """The step that held the reservation did not run: forget the reserved positions and give back the
        pages that were taken for them.  (State of fixed size that the failed step may have touched is not
        restored: a request with such state has to be released and run again.)"""
        r = self.requests[rid]
        r.reserved = 0
        keep = (r.length + self.page_size - 1) // self.page_size
        for gi, g in enumerate(self.kv_groups):
            while len(r.pages[gi]) > keep:
                p = r.pages[gi].pop()
                if p >= 0:
                    g.pool.free(p)

    def truncate(self, rid: Hashable, new_len: int) -> None:
        """Forget positions ``new_len ..``; whole pages beyond are given back
        (``KVCache.trim``, mlx_lm/models/cache.py:378-381, for pages)."""
        r = self.requests[rid]
        if r.reserved:
            raise RuntimeError(f"request {rid!r} has a reservation in flight")
        if not 0 <= new_len <= r.length:
            raise ValueError(f"truncate {rid!r} to {new_len}: it holds {r.length}")
        if self.state_groups and new_len != r.length:
            raise RuntimeError("state of fixed size cannot be rewound; release the request and run it again")
        keep = (new_len + self.page_size - 1) // self.page_size
        for gi, g in enumerate(self.kv_groups):
            floor = self._window_floor(g.spec, new_len)
            if any(p < 0 for p in r.pages[gi][floor:keep]):
                raise RuntimeError(f"request {rid!r}: pages the window of length {new_len} needs were given back")
            while len(r.pages[gi]) > keep:
                p = r.pages[gi].pop()
                if p >= 0:
                    g.pool.free(p)
        r.length = new_len

    def release(self, rid: Hashable) -> None:
        r = self.requests.pop(rid)
        for gi, g in enumerate(self.kv_groups):
            for p in reversed(r.pages[gi]):
                if p >= 0:
                    g.pool.free(p)
        self._free_slots.append(r.slot)

    # ------------------------------------------------------------ views for a step
    def block_table(self, group: int, rids: Sequence[Hashable], out: Optional[np.ndarray] = None) -> np.ndarray:
        """``int32 [len(rids), table_width]``, -1 where a request holds no page."""
        if out is None:
            out = np.empty((len(rids), self.table_width), dtype=np.int32)
        out.fill(-1)
        for i, rid in enumerate(rids):
            pl = self.requests[rid].pages[group]
            out[i, :len(pl)] = pl
        return out

    def slots(self, rids: Sequence[Hashable]) -> List[int]:
        return [self.requests[r].slot for r in rids]

    # ------------------------------------------------------------ accounting
    def pages_in_use(self) -> List[int]:
        return [g.pool.n_held for g in self.kv_groups]

    def pages_free(self) -> List[int]:
        return [g.pool.n_free for g in self.kv_groups]

    def high_water(self) -> List[int]:
        return [g.pool.high_water for g in self.kv_groups]

    def check(self) -> None:
        """Invariants: every held page belongs to exactly one request, every free page to none,
        slots likewise.  Raises AssertionError with the first violation."""
        for gi, g in enumerate(self.kv_groups):
            owners: Dict[int, Hashable] = {}
            for rid, r in self.requests.items():
                for p in r.pages[gi]:
                    if p < 0:
                        continue
                    assert p not in owners, f"group {gi}: page {p} held by {owners[p]!r} and {rid!r}"
                    assert g.pool.is_held(p), f"group {gi}: page {p} of {rid!r} is on the free list"
                    owners[p] = rid
            assert len(owners) == g.pool.n_held, (f"group {gi}: {g.pool.n_held} pages are held but requests "
                                                  f"account for {len(owners)}")
            assert len(set(g.pool._free)) == len(g.pool._free), f"group {gi}: a page is on the free list twice"
            assert g.pool.n_free + g.pool.n_held == g.pool.n_pages
        slots = [r.slot for r in self.requests.values()]
        assert len(set(slots)) == len(slots), "two requests share a slot"
        assert not set(slots) & set(self._free_slots), "a live request's slot is on the free list"
        assert len(slots) + len(self._free_slots) == self.max_requests
