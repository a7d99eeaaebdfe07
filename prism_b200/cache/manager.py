"""Cache manager: pages of keys and values with a block table per request,
and slots for per-request state of fixed size.  Host-side bookkeeping only;
the device tensors live in ``storage.py``.

andre-fu/prism's cache (engine/kv_cache.py:15-153) has one uniform pool, a
LIFO free list (:49), per-sequence page lists (:52-54), lazy allocation
(:116-121) and gives pages back only when a sequence ends (:87-91).  Kept:
the LIFO list (page 0 first out, freed pages re-used first) and the lazy
allocation.  Added: several groups of layers with different needs, each with
pages of its own; windowed groups that give pages back as soon as the window
has passed them; an all-or-nothing ``append`` that is asked before a step
for exactly the tokens of that step; slots for fixed-size state.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..parts.base import CacheNeed


class OutOfPages(RuntimeError):
    """A group has fewer free pages than the request needs (kv_cache.py:119-120)."""


class OutOfSlots(RuntimeError):
    """Every request slot is taken."""


@dataclass
class CacheGroup:
    """Schedule entries whose caches have the same shape and policy."""
    index: int
    need: CacheNeed
    entries: List[int] = field(default_factory=list)     # schedule entries that own a plane here

    @property
    def kind(self):
        return self.need.kind

    @property
    def num_planes(self):
        return len(self.entries)


def plan_groups(cache_needs: Sequence[Optional[CacheNeed]], reads: Sequence[Optional[int]]):
    """Group the cache planes of a model.  ``cache_needs[e]``: what schedule
    entry e owns (None if it reads entry ``reads[e]``'s plane, or needs
    nothing).  Returns ``(groups, where)`` with ``where[e] = (group index,
    plane index, owns)`` or None."""
    groups: List[CacheGroup] = []
    by_key: Dict[tuple, CacheGroup] = {}
    where: List[Optional[Tuple[int, int, bool]]] = [None] * len(cache_needs)
    for e, need in enumerate(cache_needs):
        if need is None or need.kind == "none":
            continue
        g = by_key.get(need.group_key())
        if g is None:
            g = CacheGroup(len(groups), need)
            groups.append(g)
            by_key[need.group_key()] = g
        where[e] = (g.index, len(g.entries), True)
        g.entries.append(e)
    for e, src in enumerate(reads):
        if src is not None:
            gi, pi, _ = where[src]
            where[e] = (gi, pi, False)
    return groups, where


def pool_sizes(groups: Sequence[CacheGroup], page_size: int, elem_bytes: int, max_seq_len: int, max_seqs: int,
               max_portion: int, num_pages: Optional[int] = None, budget_bytes: Optional[float] = None) -> List[int]:
    """Pages of every cache group's pool (0 for groups that are not paged).  Groups that keep all keys
    get ``num_pages``, or what ``budget_bytes`` pays for once the windowed groups are paid, at most what
    ``max_seqs`` requests of ``max_seq_len`` tokens hold and at least 16.  A group whose layers see a window
    needs, per request, the pages under the window and under one step's portion (``max_portion`` tokens)
    plus one - pages behind the window come back when the step is committed - so it gets that many for
    every request slot, never more than the other groups."""
    P = int(page_size)
    cap = max_seqs * ((max_seq_len + P - 1) // P)
    page_bytes = {g.index: 2 * g.num_planes * P * g.need.num_kv_heads * g.need.head_dim * elem_bytes
                  for g in groups if g.kind == "paged"}
    windowed = {g.index: min(cap, max_seqs * ((g.need.window + max_portion + P - 1) // P + 1))
                for g in groups if g.kind == "paged" and g.need.window is not None}
    if num_pages:
        full = int(num_pages)
    else:
        left = float(budget_bytes or 0) - sum(page_bytes[gi] * n for gi, n in windowed.items())
        per_page = sum(b for gi, b in page_bytes.items() if gi not in windowed) or 1
        full = max(16, min(int(max(left, 0) // per_page), cap))
    return [0 if g.kind != "paged" else min(full, windowed.get(g.index, full)) for g in groups]


class PageAllocator:
    """LIFO free list over ``num_pages`` pages; page 0 is handed out first and a
    freed page is the next one re-used (kv_cache.py:49,82,90)."""

    def __init__(self, num_pages: int):
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))
        self._held = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages(f"Out of KV cache pages ({self.num_pages} total)")
        p = self._free.pop()
        assert not self._held[p], f"page {p} handed out twice"
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        assert 0 <= page < self.num_pages and self._held[page], f"page {page} freed but not held"
        self._held[page] = False
        self._free.append(page)

    def held(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


@dataclass
class RequestCache:
    slot: int
    length: int = 0                                   # tokens committed
    pages: List[List[int]] = field(default_factory=list)    # per group: logical page -> physical, -1 once given back


class CacheManager:
    def __init__(self, groups: Sequence[CacheGroup], page_size: int, num_pages, max_seqs: int,
                 max_seq_len: int):
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.max_seqs = int(max_seqs)
        self.max_seq_len = int(max_seq_len)
        self.table_width = (self.max_seq_len + self.page_size - 1) // self.page_size
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        self.allocators: List[Optional[PageAllocator]] = [
            PageAllocator(n) if g.kind == "paged" else None for g, n in zip(self.groups, num_pages)]
        self._paged = [g.index for g in self.groups if g.kind == "paged"]
        self._free_slots = list(range(self.max_seqs - 1, -1, -1))
        self.requests: Dict[object, RequestCache] = {}
        self.fresh_slots: List[int] = []        # slots handed out since the last drain (state to be cleared)
        self.pages_high_water = 0

    # ---- requests --------------------------------------------------------
    def add_request(self, req_id) -> int:
        if req_id in self.requests:
            raise KeyError(f"request {req_id!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_seqs} request slots are taken")
        slot = self._free_slots.pop()
        self.requests[req_id] = RequestCache(slot, 0, [[] for _ in self.groups])
        self.fresh_slots.append(slot)
        return slot

    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def length(self, req_id) -> int:
        return self.requests[req_id].length

    def slot(self, req_id) -> int:
        return self.requests[req_id].slot

    def free_request(self, req_id) -> None:
        rc = self.requests.pop(req_id)
        for g, pages in zip(self.groups, rc.pages):
            if g.kind == "paged":
                for p in reversed(pages):
                    if p >= 0:
                        self.allocators[g.index].free(p)
        self._free_slots.append(rc.slot)

    def free_all(self) -> None:
        for r in list(self.requests):
            self.free_request(r)

    # ---- pages -------------------------------------------------------------
    def _pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, req_id, n_new: int) -> List[int]:
        """Pages each group must hand out before ``n_new`` more tokens can be written."""
        rc = self.requests[req_id]
        total = (rc.length + n_new + self.page_size - 1) // self.page_size
        need = [0] * len(self.groups)
        for gi in self._paged:
            k = total - len(rc.pages[gi])
            if k > 0:
                need[gi] = k
        return need

    def can_append(self, req_id, n_new: int, reserve: Optional[List[int]] = None) -> bool:
        """``reserve``: pages per group already promised to other requests of the same step."""
        if self.requests[req_id].length + n_new > self.max_seq_len:
            return False
        need = self.pages_needed(req_id, n_new)
        for gi in self._paged:
            if need[gi] and self.allocators[gi].num_free - (reserve[gi] if reserve else 0) < need[gi]:
                return False
        return True

    def append(self, req_id, n_new: int) -> None:
        """Make room for ``n_new`` more tokens in every group, or raise
        ``OutOfPages`` having changed nothing."""
        rc = self.requests[req_id]
        if rc.length + n_new > self.max_seq_len:
            raise ValueError(f"request {req_id!r}: {rc.length + n_new} tokens exceed max_seq_len {self.max_seq_len}")
        need = self.pages_needed(req_id, n_new)
        for gi in self._paged:
            if need[gi] > self.allocators[gi].num_free:
                raise OutOfPages(f"Out of KV cache pages for request {req_id!r} (+{n_new} tokens)")
        grew = False
        for gi in self._paged:
            for _ in range(need[gi]):
                rc.pages[gi].append(self.allocators[gi].alloc())
                grew = True
        if grew:
            self.pages_high_water = max(self.pages_high_water, self.pages_in_use())

    def commit(self, req_id, n_new: int) -> None:
        """The step has written ``n_new`` tokens: advance the length and give
        back the pages of windowed groups that no later query can see."""
        rc = self.requests[req_id]
        rc.length += n_new
        total = (rc.length + self.page_size - 1) // self.page_size
        for gi in self._paged:
            assert total <= len(rc.pages[gi]), "commit beyond the pages appended"
        for g in self.groups:
            if g.kind != "paged" or g.need.window is None:
                continue
            # the next query sits at position `length` and sees keys > length - window
            first_visible = rc.length - g.need.window + 1
            pages = rc.pages[g.index]
            for idx in range(len(pages)):
                if (idx + 1) * self.page_size > first_visible:
                    break
                if pages[idx] >= 0:
                    self.allocators[g.index].free(pages[idx])
                    pages[idx] = -1

    def block_table_row(self, req_id, group: int) -> List[int]:
        return self.requests[req_id].pages[group]

    # ---- accounting ----------------------------------------------------------
    def num_free_pages(self, group: int = 0) -> int:
        return self.allocators[group].num_free

    def pages_in_use(self) -> int:
        return sum(a.num_pages - a.num_free for a in self.allocators if a is not None)

    def drain_fresh_slots(self) -> List[int]:
        s, self.fresh_slots = self.fresh_slots, []
        return s

    def check_invariants(self) -> None:
        """No page lost, none held twice; every slot free or owned once."""
        for g in self.groups:
            if g.kind != "paged":
                continue
            a = self.allocators[g.index]
            owned = [p for rc in self.requests.values() for p in rc.pages[g.index] if p >= 0]
            assert len(owned) == len(set(owned)), f"group {g.index}: a page is held by two requests"
            assert sorted(owned) == a.held(), f"group {g.index}: allocator and requests disagree"
            assert len(set(a._free)) == len(a._free) and not set(a._free) & set(owned)
            assert len(a._free) + len(owned) == a.num_pages, f"group {g.index}: a page is lost"
        slots = [rc.slot for rc in self.requests.values()]
        assert len(set(slots)) == len(slots) and not set(slots) & set(self._free_slots)
        assert len(slots) + len(self._free_slots) == self.max_seqs
