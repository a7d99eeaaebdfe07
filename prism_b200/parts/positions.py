"""Position-encoding parts.  ``rotary``: andre-fu/prism's RoPE
(engine/executor.py:45-57): ``inv_freq_j = theta^(-2j/hd)``, rotate-half
pairing ``(j, j + hd/2)``, the whole head rotated, no scaling.  The table of
inverse frequencies is float32 and angles are formed from the position in the
kernel, so there is neither a rounded table nor a cap on positions."""

from __future__ import annotations

import torch

from .base import PositionEncoding, RotaryParams, register_part


_INV_FREQ = {}      # (device, theta, rotary_dim) -> float32 inverse frequencies on that device


@register_part("position", "rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim {self.head_dim}")
        self._params = None

    def on_bound(self):
        rd = self.rotary_dim
        # the formula of executor.py:50, evaluated in float32 on the host
        # layers with the same constants share one device table, so the per-step cos/sin table that
        # the kernels build from it is built once per step, not once per layer
        key = (str(self.device), self.theta, rd)
        inv = _INV_FREQ.get(key)
        if inv is None:
            inv = (1.0 / (self.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))).to(self.device)
            _INV_FREQ[key] = inv
        self._params = RotaryParams(inv, rd)

    def rotary(self):
        return self._params


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Keys and queries are used as projected."""

    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    def rotary(self):
        return None

    def apply(self, ctx, q, k):
        return None
