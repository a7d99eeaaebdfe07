"""The step function: one batch of (request, its next tokens) in, logits at
the wanted places out.

It replaces andre-fu/prism's ``prefill`` / ``decode_step`` /
``batched_decode_step`` (engine/executor.py:77,203,320): portions of prompts
and single decode tokens are one flat batch, each token attends to its
request's pages, and only the given tokens are computed.  A new token's key
is stored at the slot equal to its position (the number of tokens cached
before it); the reference's decode entry points advance the length first and
so store one slot late (executor.py:205-208) - that is not reproduced.

Pure-decode steps replay a CUDA graph captured per batch-size bucket
(the reference: executor.py:164-201,272-310); rows added to fill a bucket use
position 0 and the scratch page and their logits are dropped.
"""

from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import torch

from ..cache.manager import CacheManager, OutOfPages, plan_groups
from ..cache.storage import CacheStorage
from ..models.decoder import DecoderModel
from .batch import BatchLayout, Segment, StepContext, pack_batch


class DeviceError(RuntimeError):
    """A kernel met an index it must not follow (see csrc/common.cuh)."""


_ERR_TEXT = {1: "token id outside the vocabulary", 2: "page id outside the pool",
             3: "position outside max_position_embeddings", 4: "a kernel's bounded wait ran out"}


def cache_groups(model: DecoderModel):
    """``(groups, where)`` of a model's cache planes (see ``plan_groups``)."""
    return plan_groups(model.cache_needs(), [e.reads_cache_of for e in model.schedule])


class ModelRunner:
    def __init__(self, model: DecoderModel, device, dtype: torch.dtype, page_size: int, num_pages,
                 max_seqs: int, max_seq_len: Optional[int] = None, use_cuda_graph: bool = False,
                 graph_batch_sizes: Sequence[int] = (1, 2, 4, 8, 16, 32, 64)):
        """``num_pages``: the pool size of every paged cache group, or one size per group (in the order
        of ``cache_groups(model)``; entries of groups that are not paged are ignored): a group whose
        layers see a window of keys needs far fewer pages than one that keeps them all."""
        if not torch.cuda.is_available():
            raise RuntimeError("prism_b200 needs a CUDA device; there is no CPU path")
        self.model, self.device, self.dtype = model, torch.device(device), dtype
        spec = model.spec
        self.max_positions = spec.max_positions
        self.max_seq_len = int(min(max_seq_len or spec.max_positions, spec.max_positions))
        self.groups, self.where = cache_groups(model)
        self.paged_groups = [g.index for g in self.groups if g.kind == "paged"]
        pages = [int(num_pages)] * len(self.groups) if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(pages) != len(self.groups):
            raise ValueError(f"num_pages has {len(pages)} entries, the model has {len(self.groups)} cache groups")
        self.cache = CacheManager(self.groups, page_size, pages, max_seqs, self.max_seq_len)
        self.storage = CacheStorage(self.groups, self.where, page_size, pages, max_seqs, self.device, dtype)
        self.pad_page = {g: pages[g] for g in self.paged_groups}      # each group's scratch page
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        # a mixer that needs the host's copy of the step (a state mixer, unless it says otherwise) keeps
        # the whole model out of graphs: such steps run eagerly, with the same results
        from ..parts.base import Mixer
        self.graph_safe = all(
            (m.graph_safe if m.graph_safe is not None else m.cache_need().kind != "state")
            for m in model.walk() if isinstance(m, Mixer))
        self.use_cuda_graph = bool(use_cuda_graph) and self.graph_safe
        self.graph_batch_sizes = sorted(set(int(b) for b in graph_batch_sizes if b <= max_seqs)) or [1]
        from .. import ops
        self._sms = ops.num_sms(self.device)
        self._graphs: Dict[tuple, dict] = {}     # (bucket, decode attention places, merge kernels) -> captured step
        self._work_memo: Dict[int, dict] = {}    # per cache group: the last step's decode work items
        self.graph_kernel_launches = 0       # kernels of this library replayed inside graphs
        self.last_h2d_bytes = 0              # bytes of the last step's batch descriptor (host to device)

    # ---- bookkeeping around a step -------------------------------------------
    def begin_request(self, req_id) -> None:
        self.cache.add_request(req_id)

    def end_request(self, req_id) -> None:
        self.cache.free_request(req_id)

    def can_run(self, segments: Sequence[Segment]) -> bool:
        reserve = [0] * len(self.groups)
        for s in segments:
            if not self.cache.can_append(s.req_id, len(s.tokens), reserve):
                return False
            for g, n in enumerate(self.cache.pages_needed(s.req_id, len(s.tokens))):
                reserve[g] += n
        return True

    # ---- the step ----------------------------------------------------------------
    def step(self, segments: Sequence[Segment], token_source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the tokens of ``segments`` as one batch from the cache that
        earlier steps left; append them to the cache; return float32 logits
        ``[R, V]`` in the order of the segments and of their ``want`` lists
        (None if nothing is wanted).  Nothing here waits for the GPU.
        ``token_source`` (device int32, one token per segment, every segment a
        single token): the token ids are taken from there on the device instead of
        from ``segments`` - the previous step's sampled tokens, not yet read by the host."""
        if not segments:
            return None
        for s in segments:
            if len(s.tokens) < 1:
                raise ValueError(f"request {s.req_id!r}: a segment needs at least one token")
        if len({s.req_id for s in segments}) != len(segments):
            raise ValueError("a request may appear once per step")
        if not self.can_run(segments):
            raise OutOfPages("Out of KV cache pages for this step")
        for s in segments:
            self.cache.append(s.req_id, len(s.tokens))
        self.storage.clear_slots(self.cache.drain_fresh_slots())

        tok, pos, seg_of, seg_start, cached, qlen, slots, rows = [], [], [], [0], [], [], [], []
        for i, s in enumerate(segments):
            c = self.cache.length(s.req_id)
            n = len(s.tokens)
            for w in s.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {s.req_id!r}: wanted place {w} outside its {n} tokens")
                rows.append(len(tok) + w)
            tok.extend(int(t) for t in s.tokens)
            pos.extend(range(c, c + n))
            seg_of.extend([i] * n)
            seg_start.append(len(tok))
            cached.append(c)
            qlen.append(n)
            slots.append(self.cache.slot(s.req_id))
        block_rows = {g: [self.cache.block_table_row(s.req_id, g) for s in segments] for g in self.paged_groups}
        max_q, max_kv = max(qlen), max(c + n for c, n in zip(cached, qlen))
        host_meta = dict(seg_start=seg_start, cached_len=cached, q_len=qlen, slots=slots, tok_seg=seg_of)

        S = len(segments)
        if self.use_cuda_graph and max_q == 1 and S <= self.graph_batch_sizes[-1]:
            logits = self._step_graph(tok, pos, cached, slots, rows, block_rows, token_source)
        else:
            work = self._decode_work(cached, qlen)
            layout = BatchLayout(len(tok), S, len(rows), self.cache.table_width, self.paged_groups,
                                 {g: len(w[0]) for g, w in work.items()})
            host = pack_batch(layout, tok, pos, seg_of, seg_start, cached, qlen, slots, rows,
                              block_rows, self.pad_page, work)
            dev = host.to(self.device, non_blocking=True)
            self.last_h2d_bytes = host.numel() * 4
            if token_source is not None:
                assert max_q == 1 and token_source.shape[0] >= S
                layout.view(dev, "token_ids").copy_(token_source[:S], non_blocking=True)
            ctx = StepContext(layout, dev, self.dtype, self.device, self.err, self.max_positions,
                              host_meta, max_q, max_kv)
            for g, w in work.items():                  # the host knows whether any request has more than one item
                ctx.decode_work[g] = ctx.decode_work[g][:2] + (w[2], len(w[1]))
            views = self.storage.views(ctx.block_tables, ctx.state_slots, slots)
            logits = self.model.forward(ctx, views)
        for s in segments:
            self.cache.commit(s.req_id, len(s.tokens))
        return logits

    def _decode_work(self, cached, qlen, n_real: Optional[int] = None) -> Dict[int, tuple]:
        """The decode attention kernel's work items for the single-token segments at the head of the batch, per
        paged cache group: ``{group: (items, starts, most items of a request)}`` from the requests' own contexts,
        so that a long context among short ones is shared among many CTAs (``ops.decode_work_items``).  Empty
        when the batch starts with a prompt portion.  ``n_real``: the segments after these are padding."""
        from .. import ops
        lead = 0
        while lead < len(qlen) and qlen[lead] == 1:
            lead += 1
        if not lead or os.environ.get("PRISM_DECODE_SPLITS", "0") != "0":
            return {}
        work = {}
        for g in self.paged_groups:
            need = self.groups[g].need
            work[g] = ops.decode_work_items(cached[:lead], need.num_kv_heads, need.window, self._sms, n_real,
                                            self._work_memo.setdefault(g, {}))
        return work

    # ---- decode graphs ---------------------------------------------------------------
    def _bucket(self, n: int) -> int:
        for b in self.graph_batch_sizes:
            if b >= n:
                return b
        raise ValueError(n)

    def _graph_places(self, items: Dict[int, int]) -> tuple:
        """The decode attention kernel's grid is part of a captured graph: it has as many places for work items
        as fill the GPU once (two CTAs per SM), twice, ... - the fewest that hold the step's items.  A bucket has
        one graph for each number of waves that its steps have asked for, seldom more than two."""
        out = []
        for g in self.paged_groups if items else ():
            wave = max(1, 2 * self._sms // self.groups[g].need.num_kv_heads)
            out.append(-(-max(1, items[g]) // wave) * wave)
        return tuple(out)

    def _capture(self, B: int, places: tuple, merge: bool) -> dict:
        """Capture the decode step for a bucket of B one-token segments: static
        descriptor buffer, every row's logits computed.  ``places``: the decode attention
        kernel's places for work items in each paged group (``_graph_places``); ``merge``: whether
        a request may have more than one item (else the graph has no merge kernels)."""
        layout = BatchLayout(B, B, B, self.cache.table_width, self.paged_groups, dict(zip(self.paged_groups, places)))
        dev = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
        pad_rows = {g: [[] for _ in range(B)] for g in self.paged_groups}
        host = pack_batch(layout, [0] * B, [0] * B, list(range(B)), list(range(B + 1)), [0] * B, [1] * B,
                          [self.cache.max_seqs] * B, list(range(B)), pad_rows, self.pad_page,
                          self._decode_work([0] * B, [1] * B))
        dev.copy_(host)
        def fresh_ctx():
            # every run gets its own context: values parts keep for the length of a step (the
            # rotary table) must be produced inside the capture, in the graph's own memory
            c = StepContext(layout, dev, self.dtype, self.device, self.err, self.max_positions, None,
                            1, self.max_seq_len)
            for g in c.decode_work:
                c.decode_work[g] = c.decode_work[g][:2] + (2 if merge else 1, B)
            return c, self.storage.views(c.block_tables, c.state_slots, None)
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):                       # warm-up: lazy library set-up happens outside capture
                self.model.forward(*fresh_ctx())
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        from .. import ops
        before = ops.launch_count
        ctx, views = fresh_ctx()
        with torch.cuda.graph(graph, stream=stream):
            out = self.model.forward(ctx, views)
        torch.cuda.synchronize(self.device)
        return dict(graph=graph, layout=layout, dev=dev, out=out, launches=ops.launch_count - before)

    def _step_graph(self, tok, pos, cached, slots, rows, block_rows, token_source=None):
        S = len(tok)
        B = self._bucket(S)
        work = self._decode_work(cached + [0] * (B - S), [1] * B, S)    # padded rows: one item each, at position 0
        key = (B, self._graph_places({g: len(w[0]) for g, w in work.items()}), any(w[2] > 1 for w in work.values()))
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = self._capture(*key)
        pad = B - S
        scratch_slot = self.cache.max_seqs
        br = {k: v + [[] for _ in range(pad)] for k, v in block_rows.items()}
        host = pack_batch(g["layout"], tok + [0] * pad, pos + [0] * pad, list(range(B)), list(range(B + 1)),
                          cached + [0] * pad, [1] * B, slots + [scratch_slot] * pad, list(range(B)),
                          br, self.pad_page, work)
        g["dev"].copy_(host, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4
        if token_source is not None:
            g["layout"].view(g["dev"], "token_ids")[:S].copy_(token_source[:S], non_blocking=True)
        g["graph"].replay()
        self.graph_kernel_launches += g["launches"]
        if not rows:
            return None
        out = g["out"]
        if rows == list(range(S)):
            return out[:S]
        return out[torch.tensor(rows, device=self.device)]

    def warmup_graphs(self, sizes: Optional[Sequence[int]] = None) -> None:
        """Capture the decode graphs ahead of time (executor.py:312-318): for every bucket the two graphs
        (with and without the merge of split contexts) whose decode attention grid fills the GPU once.  The
        graphs with larger grids (many requests of very unequal length) follow at their first use."""
        if self.use_cuda_graph:
            for b in sizes or self.graph_batch_sizes:
                if b > self.graph_batch_sizes[-1]:
                    continue
                work = self._decode_work([0] * b, [1] * b)
                places = self._graph_places({g: len(w[0]) for g, w in work.items()})
                for merge in ((True, False) if work else (False,)):
                    key = (b, places, merge)
                    if key not in self._graphs:
                        self._graphs[key] = self._capture(*key)

    def invalidate_graphs(self) -> None:
        self._graphs.clear()

    # ---- errors ---------------------------------------------------------------------
    def check_errors(self) -> None:
        """Read the device error word (synchronises) and raise if a kernel set it."""
        from .. import ops
        ops.check_tc_errors()
        code = int(self.err.item())
        if code:
            self.err.zero_()
            raise DeviceError(f"device error {code}: {_ERR_TEXT.get(code, 'unknown')}")
