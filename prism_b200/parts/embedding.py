"""Embedding and output-head parts (andre-fu/prism engine/executor.py:74-75,130)."""

from __future__ import annotations

from .base import Embedding, Head, ParamSpec, WeightSource, register_part
from .. import ops


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    """Row gather without scaling; the output is the float32 residual stream."""

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)

    def params(self):
        return [ParamSpec("weight", (WeightSource("embed_tokens.weight", (self.vocab_size, self.hidden_size)),))]

    def forward(self, ctx):
        out = ctx.alloc((ctx.T, self.hidden_size), ops.torch.float32)
        ops.embed(ctx.token_ids, self.w["weight"], out, ctx.err)
        return out


@register_part("head", "linear")
class LinearHead(Head):
    """``logits = h @ W^T`` in float32, no bias, soft-cap or scale.  ``tied_to``
    names the parameter whose storage is shared when the model file has no
    head tensor (engine/weight_manager.py:84-86; the reference copies into a
    second buffer, engine/weight_pool.py:157-160: here it is one buffer)."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: str = None):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.tied_to = tied_to

    def params(self):
        return [ParamSpec("weight", (WeightSource("weight", (self.vocab_size, self.hidden_size)),),
                          optional=self.tied_to is not None, absent="none", alias_of=self.tied_to)]

    def forward(self, ctx, normed_rows):
        return ops.linear(normed_rows, self.w["weight"], None, out_dtype=ops.torch.float32)
