"""Sampling parameters and the device sampler.

andre-fu/prism samples greedily when ``temperature <= 0`` and otherwise with
``softmax(logits / temperature)`` + ``torch.multinomial``
(engine/scheduler.py:266-272, engine/executor.py:423-427); it has no top-k,
top-p or penalties, and neither has this.  Differences: logits are float32,
the first token is sampled like every other (the reference always takes the
argmax there, scheduler.py:219), and the draw is the inverse CDF at a seeded
uniform number (``rng.uniform``) instead of an unseeded multinomial.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .rng import uniform
from .. import ops


@dataclass
class SamplingParams:
    """``max_new_tokens`` default 100 as ``Request.max_new_tokens``
    (engine/request_manager.py:24); ``temperature`` 0.0 = greedy (:25)."""
    max_new_tokens: int = 100
    temperature: float = 0.0
    seed: Optional[int] = None
    eos_token_id: Optional[int] = None
    ignore_eos: bool = False


class Sampler:
    """One kernel launch per step for all rows; token ids come back through a
    pinned buffer."""

    def __init__(self, device, max_rows: int = 256):
        self.device = torch.device(device)
        self.max_rows = max_rows
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._host = torch.empty(max_rows, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], us: Sequence[float]) -> List[int]:
        R = logits.shape[0]
        if R > self.max_rows:
            self.__init__(self.device, max(R, 2 * self.max_rows))
        out = self._out[:R]
        if any(t > 0 for t in temperatures):
            tu = torch.tensor([list(temperatures), list(us)], dtype=torch.float32, pin_memory=True)
            tu = tu.to(self.device, non_blocking=True)
            ops.sample(logits, tu[0], tu[1], out)
        else:
            ops.sample(logits, None, None, out)
        self._host[:R].copy_(out, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self._host[:R].tolist()
