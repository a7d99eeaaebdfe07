"""The batch a step runs: segments of (request, its next tokens), flattened.

andre-fu/prism has three entry points with three batch shapes - one whole
prompt (engine/executor.py:77), one decode token (:203), B decode tokens
(:320) - and builds block tables with per-element device writes
(engine/kv_cache.py:147-151).  Here every step is the same thing: segments
with ``q_len >= 1`` new tokens and ``cached_len >= 0`` tokens already in the
cache, described by int32 arrays that are packed on the host in pinned memory
and reach the device in one copy:

    token_ids[T] positions[T] tok_seg[T] seg_start[S+1] cached_len[S]
    q_len[S] state_slots[S] logit_rows[R] block_tables[G][S, W]
    decode_items[G][n_g, 4] decode_starts[G][S]

``decode_items[g]`` is the decode attention kernel's work in paged cache group g
for the single-token segments at the head of the batch: one item
``{token, split | used << 16, position, segment}`` per CTA and kv head, as many
per request as its own context asks for, so that a ragged batch is shared among
equally loaded CTAs (``ops.decode_work_items``); token -1: a place the step
does not use.  ``decode_starts[g][t]``: token t's first item | its items << 16.  A layout
without items (``decode_items`` empty) leaves the kernel to equal splits.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class Segment:
    """A request's next tokens in this step.  ``want``: places among these
    tokens whose logits are wanted."""
    req_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class BatchLayout:
    """Offsets (in int32 elements) of each array in the packed descriptor."""
    T: int
    S: int
    R: int
    W: int
    paged_groups: List[int]
    decode_items: Optional[Dict[int, int]] = None       # group -> items in the descriptor

    def __post_init__(self):
        o = 0
        self.off = {}
        for name, n in (("token_ids", self.T), ("positions", self.T), ("tok_seg", self.T),
                        ("seg_start", self.S + 1), ("cached_len", self.S), ("q_len", self.S),
                        ("state_slots", self.S), ("logit_rows", self.R)):
            self.off[name] = (o, n)
            o += (n + 3) // 4 * 4               # keep every array 16-byte aligned
        for g in self.paged_groups:
            self.off[f"bt{g}"] = (o, self.S * self.W)
            o += (self.S * self.W + 3) // 4 * 4
        for g, n in (self.decode_items or {}).items():
            self.off[f"items{g}"] = (o, 4 * n)
            o += 4 * n
            self.off[f"starts{g}"] = (o, self.S)
            o += (self.S + 3) // 4 * 4
        self.total = max(o, 4)

    def view(self, buf, name):
        o, n = self.off[name]
        return buf[o:o + n]


class StepContext:
    """What the parts see of a step: device arrays, counts, the compute dtype,
    an allocator for activations and the device error word."""

    def __init__(self, layout: BatchLayout, dev_buf: torch.Tensor, dtype, device, err, max_positions,
                 host: Optional[dict], max_q_len: int, max_kv_len: int):
        self.layout, self.buf = layout, dev_buf
        self.T, self.S, self.R, self.W = layout.T, layout.S, layout.R, layout.W
        self.dtype, self.device, self.err = dtype, device, err
        self.max_positions = int(max_positions)
        self.host = host                       # host copies of the arrays (None inside a captured graph)
        self.max_q_len, self.max_kv_len = int(max_q_len), int(max_kv_len)
        self.decode_only = max_q_len == 1
        self.scratch = {}                      # per-step values shared by parts (e.g. the rotary table)
        v = lambda n: layout.view(dev_buf, n)
        self.token_ids, self.positions, self.tok_seg = v("token_ids"), v("positions"), v("tok_seg")
        self.seg_start, self.cached_len, self.q_len = v("seg_start"), v("cached_len"), v("q_len")
        self.state_slots, self.logit_rows = v("state_slots"), v("logit_rows")
        self.block_tables = {g: v(f"bt{g}").view(layout.S, layout.W) for g in layout.paged_groups}
        # group -> (items [n, 4], starts [S], most items of a token (1: no merge kernel), tokens the items are for);
        # the runner sets the last two
        self.decode_work = {g: (v(f"items{g}").view(n, 4), v(f"starts{g}"), 2, 0)
                            for g, n in (layout.decode_items or {}).items()}

    def alloc(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)


def pack_batch(layout: BatchLayout, token_ids, positions, tok_seg, seg_start, cached_len, q_len,
               slots, logit_rows, block_rows: Dict[int, List[List[int]]], pad_page: Dict[int, int],
               decode_work: Optional[Dict[int, tuple]] = None):
    """Fill a pinned int32 tensor with the descriptor.  ``block_rows[g][s]`` is
    request s's logical-page -> physical-page list in group g; entries beyond
    it (and pages already given back) read ``pad_page[g]``, the scratch page.
    ``decode_work[g]``: ``(items, starts)`` of group g as int32 arrays (``ops.decode_work_items``); the layout's
    places beyond them are marked unused."""
    host = torch.empty(layout.total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
    a = host.numpy()
    a[:] = 0
    for name, vals in (("token_ids", token_ids), ("positions", positions), ("tok_seg", tok_seg),
                       ("seg_start", seg_start), ("cached_len", cached_len), ("q_len", q_len),
                       ("state_slots", slots), ("logit_rows", logit_rows)):
        o, n = layout.off[name]
        if n:
            a[o:o + n] = np.asarray(vals, dtype=np.int32)
    for g, n in (layout.decode_items or {}).items():
        items, starts = decode_work[g][:2]
        o, _ = layout.off[f"items{g}"]
        region = a[o:o + 4 * n].reshape(n, 4)
        region[:len(items)] = items
        region[len(items):] = -1
        o, m = layout.off[f"starts{g}"]
        a[o:o + len(starts)] = starts                   # segments after the decoding ones: no items (0)
    for g in layout.paged_groups:
        o, n = layout.off[f"bt{g}"]
        bt = a[o:o + n].reshape(layout.S, layout.W)
        bt[:] = pad_page[g]
        for s, row in enumerate(block_rows[g]):
            if row:
                r = np.asarray(row[:layout.W], dtype=np.int32)
                bt[s, :len(r)] = np.where(r >= 0, r, pad_page[g])
    return host
