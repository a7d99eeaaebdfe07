"""Interfaces of the parts a decoder is put together from, and the registry
that maps a part's kind (a string in the layer plan) to its class.

andre-fu/prism writes the whole forward pass inline, three times over
(engine/executor.py:77-130, 132-162, 239-270).  Here each piece of that
loop is a part with its sizes and constants as constructor parameters:

====================  =========================================================
category              interface (see the class of that name below)
====================  =========================================================
``norm``              ``forward(ctx, residual, delta, rows=None) -> normed``
``position``          ``rotary() -> RotaryParams | None`` and ``apply(ctx, q, k)``
``mixer``             ``cache_need()``, ``forward(ctx, x, cache) -> delta``
``feed_forward``      ``forward(ctx, x) -> delta``
``block``             ``forward(ctx, residual, delta, cache) -> (residual, delta)``
``embedding``         ``forward(ctx) -> residual``
``head``              ``forward(ctx, normed_rows) -> float32 logits``
====================  =========================================================

A part never learns which model it is in: the architecture gives it a name
prefix for its tensors and nothing else.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple


# --------------------------------------------------------------------------
# weights a part asks for
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class WeightSource:
    """One tensor of the model file: its name relative to the part's prefix,
    its shape, and how random-weights mode draws it
    (``matrix`` | ``bias`` | ``norm``)."""
    name: str
    shape: Tuple[int, ...]
    init: str = "matrix"


@dataclass(frozen=True)
class ParamSpec:
    """One parameter of a part as the kernels see it: the file tensors in
    ``sources`` stacked along dim 0 (the fused qkv and gate_up buffers of
    engine/weight_pool.py:169-182,194-197).  ``optional``: all sources may be
    absent together, and then ``absent`` says what the part gets: ``"zeros"``
    or ``"none"``.  ``alias_of`` names another parameter (qualified) whose
    storage is shared when every source is absent (a tied head)."""
    name: str
    sources: Tuple[WeightSource, ...]
    optional: bool = False
    absent: str = "none"
    alias_of: Optional[str] = None

    @property
    def shape(self) -> Tuple[int, ...]:
        first = self.sources[0].shape
        return (sum(s.shape[0] for s in self.sources),) + tuple(first[1:])


# --------------------------------------------------------------------------
# what a mixer needs from the cache manager
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class CacheNeed:
    """``paged``: keys and values of ``num_kv_heads x head_dim`` per token in
    pages; ``window`` None keeps every key, an integer keeps the last
    ``window`` positions (older pages are given back).  ``state``: one tensor
    of ``state_shape`` per request, in a slot.  ``none``: nothing."""
    kind: str = "none"
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"

    def group_key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window,
                tuple(self.state_shape), self.state_dtype)


@dataclass
class RotaryParams:
    """What the fused rotate-and-store kernel needs of a position encoding:
    a float32 table of ``rotary_dim/2`` inverse frequencies on the device."""
    inv_freq: object          # torch.Tensor [rotary_dim // 2] float32
    rotary_dim: int


# --------------------------------------------------------------------------
# part base classes
# --------------------------------------------------------------------------

@dataclass
class PartSpec:
    """One entry of a layer plan: which kind of part, its constructor
    arguments (sizes and constants, nested ``PartSpec`` for sub-parts), and the
    prefix of its tensors' names in the model file."""
    kind: str
    args: dict = field(default_factory=dict)
    prefix: str = ""


class Part:
    """Common life cycle: constructed from the layer plan's arguments, asked
    for its ``params()`` (own) and ``children`` (sub-parts), then ``bind``
    receives one device tensor per own parameter (None for an absent optional
    one) and is called on the children in turn."""

    category = ""
    prefix = ""

    @property
    def children(self) -> Dict[str, "Part"]:
        return getattr(self, "_children", {})

    def add_child(self, name: str, part: "Part") -> "Part":
        if not hasattr(self, "_children"):
            self._children = {}
        self._children[name] = part
        return part

    def params(self) -> List[ParamSpec]:
        return []

    def named_params(self, path: str = ""):
        """Yield ``(qualified name, ParamSpec with absolute tensor names)`` for
        this part and everything below it."""
        for p in self.params():
            srcs = tuple(WeightSource(self.prefix + s.name, s.shape, s.init) for s in p.sources)
            yield path + p.name, ParamSpec(p.name, srcs, p.optional, p.absent, p.alias_of)
        for cname, child in self.children.items():
            yield from child.named_params(f"{path}{cname}.")

    def bind(self, tensors: Dict[str, object], device, dtype, path: str = "") -> None:
        """``tensors`` maps qualified names to device tensors."""
        self.device = device
        self.dtype = dtype
        self.w = {p.name: tensors.get(path + p.name) for p in self.params()}
        for cname, child in self.children.items():
            child.bind(tensors, device, dtype, f"{path}{cname}.")
        self.on_bound()

    def on_bound(self) -> None:
        """Hook: create device buffers that are not weights (tables, scratch)."""

    def walk(self):
        """This part and every part below it."""
        yield self
        for child in self.children.values():
            yield from child.walk()


class Norm(Part):
    category = "norm"

    def forward(self, ctx, residual, delta, rows=None):
        """``residual += delta`` (float32, in place; ``delta`` may be None or a
        stack of split partial sums) and return the normed rows in the compute
        dtype.  ``rows``: device int32 indices of the rows wanted (all if None)."""
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"

    def rotary(self) -> Optional[RotaryParams]:
        """Parameters for the fused rotate-and-store kernel, or None when this
        encoding is not a rotary one (then ``apply`` is called instead)."""
        return None

    def apply(self, ctx, q, k) -> None:
        """Encode positions into ``q [T, nh, hd]`` and ``k [T, nkv, hd]`` in place."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"
    # Whether a pure-decode step with this mixer may be replayed from a captured CUDA graph.  Inside a
    # graph there is no host copy of the step (``ctx.host`` and ``StateCacheView.host_slots`` are None)
    # and every value must come from device arrays.  None: yes unless the mixer keeps per-request state
    # (``cache_need().kind == "state"``); a state mixer that works from ``cache.slots`` alone sets True.
    graph_safe: Optional[bool] = None

    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, ctx, x, cache):
        """``x [T, H]`` normed rows -> ``delta [T, H]`` (or split partial sums
        ``[k, T, H]`` float32) to be added to the residual stream.  ``cache`` is
        the view of this layer's cache plane for this step (``None`` if the
        mixer needs none)."""
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, ctx, x):
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer, a feed-forward and their norms."""
    category = "block"

    def cache_need(self) -> CacheNeed:
        return self.mixer.cache_need()

    def forward(self, ctx, residual, delta, cache):
        raise NotImplementedError


class Embedding(Part):
    category = "embedding"

    def forward(self, ctx):
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, ctx, normed_rows):
        raise NotImplementedError


# --------------------------------------------------------------------------
# registry of part kinds
# --------------------------------------------------------------------------

_PARTS: Dict[Tuple[str, str], Callable] = {}

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")


def register_part(category: str, kind: str):
    """Class decorator: ``@register_part("mixer", "gqa_attention")``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def deco(cls):
        _PARTS[(category, kind)] = cls
        return cls
    return deco


def part_class(category: str, kind: str):
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for (c, k) in _PARTS if c == category)
        raise KeyError(f"no {category} part of kind {kind!r}; registered: {known}") from None


def build_part(category: str, spec: PartSpec) -> Part:
    """Construct the part a ``PartSpec`` names and give it its tensor prefix."""
    part = part_class(category, spec.kind)(**spec.args)
    part.prefix = spec.prefix
    return part


def registered_parts(category: Optional[str] = None):
    return sorted(k for k in _PARTS if category is None or k[0] == category)
