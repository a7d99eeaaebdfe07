"""The model as data: a ``ModelSpec`` (embedding, layers, the order in which
layers run, final norm, head) and ``DecoderModel``, which builds the parts a
spec names and runs them.  andre-fu/prism has this loop inline
(engine/executor.py:99-130); here the loop is generic and the architecture is
the spec.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from ..parts.base import CacheNeed, Part, PartSpec, build_part


@dataclass
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` (a layer
    may appear in several entries: its weights are shared, each run has a cache
    plane of its own).  ``reads_cache_of``: index of an earlier entry whose
    cache plane this run reads instead of writing its own."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[PartSpec]                 # block specs
    final_norm: PartSpec
    head: PartSpec
    schedule: Optional[List[ScheduleEntry]] = None   # default: every layer once, in order
    eos_token_id: tuple = ()               # every id that ends a sequence

    def run_order(self) -> List[ScheduleEntry]:
        return self.schedule if self.schedule is not None else [ScheduleEntry(i) for i in range(len(self.layers))]


class DecoderModel(Part):
    """Parts built from a spec.  Parameter paths: ``embedding.``,
    ``layers.<i>.``, ``final_norm.``, ``head.``."""

    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = self.add_child("embedding", build_part("embedding", spec.embedding))
        self.layers = [self.add_child(f"layers.{i}", build_part("block", s)) for i, s in enumerate(spec.layers)]
        self.final_norm = self.add_child("final_norm", build_part("norm", spec.final_norm))
        self.head = self.add_child("head", build_part("head", spec.head))
        self.schedule = spec.run_order()
        for e, ent in enumerate(self.schedule):
            if not 0 <= ent.layer < len(self.layers):
                raise ValueError(f"schedule entry {e} names layer {ent.layer}, the model has {len(self.layers)}")
            if ent.reads_cache_of is not None:
                src = ent.reads_cache_of
                if not 0 <= src < e or self.schedule[src].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {e} must read the cache of an earlier entry that owns one")
                if self.layers[ent.layer].cache_need().group_key() != self.layers[self.schedule[src].layer].cache_need().group_key():
                    raise ValueError(f"schedule entry {e} reads a cache of a different shape")

    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """Per schedule entry: the cache plane it owns (None if it reads another's)."""
        return [None if ent.reads_cache_of is not None else self.layers[ent.layer].cache_need()
                for ent in self.schedule]

    def forward(self, ctx, cache_views):
        """Run the step's tokens; returns float32 logits ``[R, V]`` for
        ``ctx.logit_rows``.  ``cache_views[e]`` is the cache view of schedule entry e."""
        residual = self.embedding.forward(ctx)
        delta = None
        for e, ent in enumerate(self.schedule):
            residual, delta = self.layers[ent.layer].forward(ctx, residual, delta, cache_views[e])
        if ctx.R == 0:
            return None
        h = self.final_norm.forward(ctx, residual, delta, rows=ctx.logit_rows)
        return self.head.forward(ctx, h)
