"""The cache manager: pages of keys and values in groups, a block table for each request
and group, and slots of fixed-size per-request state.

What the reference has (src/qwen25vl_lite/cache.py): one pool shared by all layers
(``PagedKVCache``, :394-431), a block table per request grown on demand
(``SequenceState.block_table``, :584-629; src/qwen25vl_lite/engine.py:285-291), pages
given back when a request finishes or is preempted (engine.py:483-486, 719, 855), and the
per-request ``rope_delta`` / ``num_computed_tokens`` kept on the request (:594,601).

What is different here:

* layers are sorted into *groups* by what their mixer needs (kv heads, head size, and
  whether it reads all keys or only a window of them).  Each group has a pool and page
  tensors of its own, and each request has one block table per group;
* a group with a window gives a page back as soon as every key in it lies behind the
  window of the request's next token, not only when the request ends;
* per-request fixed-size state lives in numbered *slots*: the request's token count and
  position offset, and one tensor ``[max_requests, *shape]`` for every mixer that asks for
  state of its own, zeroed when a slot is handed out.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVCacheNeed, StateNeed
from .page_pool import OutOfPages, PagePool


class NoFreeSlot(RuntimeError):
    """All per-request state slots are taken."""


@dataclass
class StopNeeds:
    """What one schedule stop asks of the cache manager."""

    cache: Optional[KVCacheNeed] = None
    state: Optional[StateNeed] = None
    cache_of: Optional[int] = None


@dataclass
class CacheGroup:
    index: int
    need: KVCacheNeed
    page_size: int
    stops: List[int]
    pool: PagePool
    pages: Optional[torch.Tensor] = None   # [len(stops), 2, num_pages, kv_heads, page_size, head_dim]

    @property
    def window(self) -> Optional[int]:
        return self.need.window

    def first_needed_page(self, num_tokens: int) -> int:
        """Logical page of the oldest key that the token at index ``num_tokens`` still sees."""
        if self.window is None:
            return 0
        return max(0, num_tokens - self.window + 1) // self.page_size

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * len(self.stops) * self.need.kv_heads * self.need.head_dim * element_size


@dataclass(eq=False)
class RequestCache:
    """What one live request holds: a state slot and, per group, its block table (the
    physical page of each logical page; -1 where none is held)."""

    slot: int
    tables: List[List[int]]
    num_tokens: int = 0
    position_offset: int = 0      # added to a token's index to get its position when none is given
    max_position: int = -1        # largest position any of the request's tokens had
    open: bool = True
    # per group: how many leading entries of the table have been given back (a window passed them).
    # A table holds a page at every index from there to its end, so the book-keeping of a step is
    # arithmetic on lengths, not a walk over the table.
    released: List[int] = field(default_factory=list)
    # tokens that the tables of all groups reach (the shortest table's length in tokens): up to
    # there ``ensure`` has nothing to do, which is the case in 15 of 16 decode steps
    reach: int = 0

    def held_pages(self, group: int) -> List[int]:
        return [p for p in self.tables[group] if p >= 0]


class CacheManager:
    def __init__(self, stops: Sequence[StopNeeds], num_pages: int, page_size: int, max_requests: int):
        if page_size <= 0 or num_pages <= 0 or max_requests <= 0:
            raise ValueError("page_size, num_pages and max_requests must be positive")
        self.page_size = int(page_size)
        self.num_pages = int(num_pages)
        self.max_requests = int(max_requests)
        self.groups: List[CacheGroup] = []
        self.location: Dict[int, Tuple[int, int]] = {}   # stop -> (group, layer within the group)
        self.state_needs: Dict[int, StateNeed] = {}
        self.states: Dict[int, torch.Tensor] = {}
        by_need: Dict[KVCacheNeed, CacheGroup] = {}
        for i, s in enumerate(stops):
            if s.state is not None:
                self.state_needs[i] = s.state
            if s.cache is None or s.cache_of is not None:
                continue
            g = by_need.get(s.cache)
            if g is None:
                g = CacheGroup(len(self.groups), s.cache, self.page_size, [], PagePool(self.num_pages))
                by_need[s.cache] = g
                self.groups.append(g)
            self.location[i] = (g.index, len(g.stops))
            g.stops.append(i)
        for i, s in enumerate(stops):
            if s.cache_of is None:
                continue
            if s.cache_of not in self.location:
                raise ValueError(f"stop {i} reads the cache of stop {s.cache_of}, which keeps none")
            owner = self.groups[self.location[s.cache_of][0]].need
            if s.cache is None or (s.cache.kv_heads, s.cache.head_dim) != (owner.kv_heads, owner.head_dim):
                raise ValueError(f"stop {i} cannot read the cache of stop {s.cache_of}: shapes differ")
            if owner.window is not None and (s.cache.window is None or s.cache.window > owner.window):
                raise ValueError(f"stop {i} needs keys that stop {s.cache_of}'s window no longer keeps")
            self.location[i] = self.location[s.cache_of]
        self._free_slots: List[int] = list(range(self.max_requests - 1, -1, -1))

    # ---- device memory -----------------------------------------------------------------
    def allocate_device(self, device, dtype: torch.dtype) -> None:
        for g in self.groups:
            g.pages = torch.zeros((len(g.stops), 2, self.num_pages, g.need.kv_heads, self.page_size, g.need.head_dim),
                                  dtype=dtype, device=device)
        for i, need in self.state_needs.items():
            self.states[i] = torch.zeros((self.max_requests, *need.shape), dtype=getattr(torch, need.dtype), device=device)

    def nbytes(self) -> int:
        return sum(g.pages.numel() * g.pages.element_size() for g in self.groups if g.pages is not None)

    def stop_pages(self, stop: int) -> Tuple[CacheGroup, torch.Tensor, torch.Tensor]:
        gi, li = self.location[stop]
        g = self.groups[gi]
        return g, g.pages[li, 0], g.pages[li, 1]

    # ---- requests ----------------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def open(self) -> RequestCache:
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        for t in self.states.values():
            t[slot].zero_()
        return RequestCache(slot, [[] for _ in self.groups], released=[0] * len(self.groups))

    def pages_missing(self, req: RequestCache, upto: int) -> List[int]:
        """New pages each group must find so that tokens [req.num_tokens, upto) can run."""
        out = []
        last = -(-upto // self.page_size)
        for g in self.groups:
            first = max(g.first_needed_page(req.num_tokens), len(req.tables[g.index]))
            out.append(max(0, last - first))
        return out

    def can_hold(self, req: RequestCache, upto: int) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_missing(req, upto), self.groups))

    def ensure(self, req: RequestCache, upto: int) -> None:
        """Makes every page that tokens [req.num_tokens, upto) read or write held; takes
        either all the pages it needs or none (``OutOfPages``)."""
        if not req.open:
            raise ValueError("request is closed")
        if upto <= req.reach:
            return
        missing = self.pages_missing(req, upto)
        for n, g in zip(missing, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"cache group {g.index} needs {n} more pages for {upto} tokens, "
                                 f"{g.pool.num_free} of {g.pool.num_pages} free")
        last = -(-upto // self.page_size)
        for n, g in zip(missing, self.groups):
            if n:
                table = req.tables[g.index]
                if len(table) < last - n:          # pages before the first one needed were never held
                    table.extend([-1] * (last - n - len(table)))
                    req.released[g.index] = len(table)
                table.extend(g.pool.allocate(n))
        req.reach = min(len(t) for t in req.tables) * self.page_size

    def advance(self, req: RequestCache, n_tokens: int) -> None:
        """``n_tokens`` more tokens are in the cache; pages wholly behind a window go back."""
        req.num_tokens += int(n_tokens)
        for g in self.groups:
            if g.window is None:
                continue
            table = req.tables[g.index]
            upto = min(g.first_needed_page(req.num_tokens), len(table))
            for i in range(req.released[g.index], upto):
                if table[i] >= 0:
                    g.pool.free([table[i]])
                    table[i] = -1
            req.released[g.index] = max(req.released[g.index], upto)

    def close(self, req: RequestCache) -> None:
        """Gives back everything the request holds.  Closing twice is an error."""
        if not req.open:
            raise ValueError("request cache was already closed")
        for g in self.groups:
            g.pool.free(req.held_pages(g.index))
            req.tables[g.index] = []
        self._free_slots.append(req.slot)
        req.open = False
        req.num_tokens = 0
        req.reach = 0

    # ---- checks ------------------------------------------------------------------------
    def pages_in_use(self) -> List[int]:
        return [g.pool.in_use() for g in self.groups]

    def check(self, live: Iterable[RequestCache]) -> None:
        """No page lost, held twice or free while held; no slot shared.  For tests."""
        live = list(live)
        slots = [r.slot for r in live]
        assert len(set(slots)) == len(slots), "two live requests share a state slot"
        assert set(slots).isdisjoint(self._free_slots), "a live request's slot is on the free list"
        assert len(slots) + len(self._free_slots) == self.max_requests, "a state slot was lost"
        for g in self.groups:
            g.pool.check()
            held: List[int] = []
            for r in live:
                held += r.held_pages(g.index)
            assert len(set(held)) == len(held), f"group {g.index}: a page is in two block tables"
            assert len(held) == g.pool.in_use(), (
                f"group {g.index}: {g.pool.in_use()} pages taken from the pool, {len(held)} in block tables")
            for p in held:
                assert g.pool.refcount(p) == 1
