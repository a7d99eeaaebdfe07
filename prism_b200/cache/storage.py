"""Device tensors behind the cache manager, and the views a step hands to the
mixers.

Keys and values: per paged group one K and one V tensor
``[planes, num_pages + 1, page_size, num_kv_heads, head_dim]`` in the engine's
dtype (andre-fu/prism allocates ``[max_pages, page_size, nkv, hd]`` per layer,
engine/kv_cache.py:37-46; pages are not cleared on re-use).  The extra last
page is scratch: padded rows of a captured decode graph write there.  State:
per state group ``[planes, max_seqs + 1, *state_shape]``, cleared when a slot
is handed to a new request.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .manager import CacheGroup


@dataclass
class PagedCacheView:
    """One cache plane for one step."""
    k: torch.Tensor                 # [num_pages + 1, P, nkv, hd]
    v: torch.Tensor
    block_table: torch.Tensor       # int32 [S, W] on the device
    num_pages: int                  # page ids < num_pages + 1 are legal (the last is scratch)
    page_size: int
    write: bool                     # False: this run reads another entry's plane
    window: Optional[int]
    group: int


@dataclass
class StateCacheView:
    state: torch.Tensor             # [max_seqs + 1, *state_shape]
    slots: torch.Tensor             # int32 [S] on the device
    host_slots: Optional[List[int]]
    write: bool
    group: int


class CacheStorage:
    def __init__(self, groups: List[CacheGroup], where, page_size: int, num_pages: List[int],
                 max_seqs: int, device, dtype: torch.dtype):
        self.groups, self.where = groups, where
        self.page_size, self.num_pages, self.max_seqs = page_size, list(num_pages), max_seqs
        self.k, self.v, self.state = {}, {}, {}
        for g in groups:
            if g.kind == "paged":
                shape = (g.num_planes, num_pages[g.index] + 1, page_size, g.need.num_kv_heads, g.need.head_dim)
                self.k[g.index] = torch.empty(shape, dtype=dtype, device=device)
                self.v[g.index] = torch.empty(shape, dtype=dtype, device=device)
            elif g.kind == "state":
                sd = getattr(torch, g.need.state_dtype)
                self.state[g.index] = torch.zeros((g.num_planes, max_seqs + 1) + tuple(g.need.state_shape),
                                                  dtype=sd, device=device)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in (self.k, self.v, self.state) for t in d.values())

    def clear_slots(self, slots: List[int]) -> None:
        """State of requests that have just been admitted starts at zero."""
        if slots and self.state:
            idx = torch.tensor(slots, dtype=torch.long, device=next(iter(self.state.values())).device)
            for t in self.state.values():
                t[:, idx] = 0

    def views(self, block_tables, slots_dev, host_slots) -> list:
        """Per schedule entry the view its mixer gets (None if it needs no cache)."""
        out = []
        for w in self.where:
            if w is None:
                out.append(None)
                continue
            gi, plane, owns = w
            g = self.groups[gi]
            if g.kind == "paged":
                out.append(PagedCacheView(self.k[gi][plane], self.v[gi][plane], block_tables[gi],
                                          self.num_pages[gi] + 1, self.page_size, owns, g.need.window, gi))
            else:
                out.append(StateCacheView(self.state[gi][plane], slots_dev, host_slots, owns, gi))
        return out
