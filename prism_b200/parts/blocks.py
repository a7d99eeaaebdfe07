"""Arrangements of parts into a layer.  ``prenorm``: andre-fu/prism's decoder
layer (engine/executor.py:106-127): norm, mixer, residual add, norm,
feed-forward, residual add.  Each residual add is carried out by the norm
that follows it (the next block's first norm, or the final norm)."""

from __future__ import annotations

from .base import Block, PartSpec, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, ff_norm: PartSpec):
        self.mixer_norm = self.add_child("mixer_norm", build_part("norm", mixer_norm))
        self.mixer = self.add_child("mixer", build_part("mixer", mixer))
        self.ff_norm = self.add_child("ff_norm", build_part("norm", ff_norm))
        self.feed_forward = self.add_child("feed_forward", build_part("feed_forward", feed_forward))

    def forward(self, ctx, residual, delta, cache):
        h = self.mixer_norm.forward(ctx, residual, delta)
        d = self.mixer.forward(ctx, h, cache)
        h = self.ff_norm.forward(ctx, residual, d)
        d = self.feed_forward.forward(ctx, h)
        return residual, d
