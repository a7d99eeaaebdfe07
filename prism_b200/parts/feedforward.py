"""Feed-forward parts.  ``swiglu``: andre-fu/prism's dense MLP
(engine/executor.py:125-127): fused gate/up projection, ``silu(gate) * up``,
down projection; no biases (engine/weight_pool.py:194-199)."""

from __future__ import annotations

from .base import FeedForward, ParamSpec, WeightSource, register_part
from .. import ops


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)

    def params(self):
        H, I = self.hidden_size, self.intermediate_size
        return [
            ParamSpec("gate_up_w", (WeightSource("gate_proj.weight", (I, H)),
                                    WeightSource("up_proj.weight", (I, H)))),
            ParamSpec("down_w", (WeightSource("down_proj.weight", (H, I)),)),
        ]

    def forward(self, ctx, x):
        return ops.feed_forward_swiglu(ctx, x, self.w["gate_up_w"], self.w["down_w"])
